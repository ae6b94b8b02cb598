"""CPU suite: the C-ABI library loads, exports every symbol include/hkv.h declares, rejects
bad geometry before touching a device, and its host-side planning arithmetic is right.
No compute call is made here (no GPU in this suite)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(REPO, "include", "hkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(hkv):
    lib = C.CDLL(hkv._capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/hkv.h but not exported"
    assert set(names) == set(hkv._capi.SIGNATURES), "ctypes table and header disagree"
    assert hkv._capi.load().hkv_abi_version() == hkv._capi.ABI_VERSION == 2


def test_dist_library_exports_every_declared_symbol(hkv):
    """libhkv_dist.so (the C++ multi-GPU host) exports what include/hkv_dist.h declares and the
    Python binding binds exactly those. Loading it needs no GPU."""
    text = open(os.path.join(REPO, "include", "hkv_dist.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(hkvd_[a-z0-9_]+)\s*\(", text)))
    lib = hkv.dist.load_dist()
    assert len(names) == 13
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/hkv_dist.h but not exported"
    assert set(names) == set(lib._hkvd_symbols)
    buf = C.create_string_buffer(hkv.dist.UNIQUE_ID_BYTES)
    assert lib.hkvd_unique_id(None) == 1          # HKV_ERR_INVALID_ARG, before NCCL is touched
    assert lib.hkvd_step(None, 0, None) == 1 and lib.hkvd_wait(None, 10) == 1
    del buf
    # argument checks of the creating call come before any device or communicator work
    g = hkv.Geometry(batch=2, num_heads=8, num_kv_heads=2, head_dim=64, slots=128).to_c()
    for exchange, wait_ms in ((7, 0), (-1, 0), (2, 20000), (0, -5)):
        handle = C.c_void_p()
        assert lib.hkvd_create_with(C.byref(handle), C.byref(g), 2, None, 0.0, None, exchange, wait_ms) == 1
        assert b"exchange" in lib.hkvd_last_error(handle)
        assert lib.hkvd_exchange(handle, None) == 1
        lib.hkvd_destroy(handle)


def test_product_library_has_no_oracle_or_torch_dependency(hkv):
    """The shipped libraries must not link the test oracle or PyTorch."""
    import subprocess
    for path in (hkv._capi.LIB_PATH, hkv.dist.DIST_LIB_PATH):
        out = subprocess.run(["ldd", path], capture_output=True, text=True).stdout
        assert "oracle" not in out and "torch" not in out and "libc10" not in out, path


def test_geometry_validation_needs_no_device(hkv):
    bad = [
        (dict(num_heads=14, num_kv_heads=3, head_dim=64), 2),     # H % KVH != 0 (reference guard)
        (dict(num_heads=8, num_kv_heads=8, head_dim=513), 2),     # head_dim > 512
        (dict(num_heads=8, num_kv_heads=8, head_dim=0), 2),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, batch=0), 1),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, slots=0), 1),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, layout=7), 1),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, shard_count=2, shard_rank=2), 1),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, shard_count=2, shard_block=100), 1),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, shard_count=2, layout=1), 2),
        (dict(num_heads=8, num_kv_heads=8, head_dim=64, slots=100, batch_stride_elems=8), 1),
    ]
    for kw, status in bad:
        with pytest.raises(hkv.HkvError) as e:
            hkv.Context(hkv.Geometry(**kw))
        assert e.value.status == status, (kw, e.value)


def test_no_cpu_fallback(hkv):
    """Without a CUDA device a valid geometry must fail loudly, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(hkv.HkvError) as e:
        hkv.Context(hkv.Geometry(batch=1, num_heads=14, num_kv_heads=2, head_dim=64, slots=2048))
    assert e.value.status in (4, 5)


def _plan(hkv, g, total, ct):
    lib = hkv._capi.load()
    vals = [C.c_int32() for _ in range(4)]
    st = lib.hkv_plan_sequence(C.byref(g.to_c()), total, ct, *[C.byref(v) for v in vals])
    assert st == 0
    return [v.value for v in vals]


def test_slot_maps_linear_ring_sharded(hkv):
    lib = hkv._capi.load()
    lin = hkv.Geometry(num_heads=4, num_kv_heads=2, head_dim=64, slots=100)
    g = lin.to_c()
    assert lib.hkv_slot_of_position(C.byref(g), 99) == 99
    assert lib.hkv_slot_of_position(C.byref(g), 100) == -1      # dropped, as the reference does
    ring = hkv.Geometry(num_heads=4, num_kv_heads=2, head_dim=64, slots=16, layout=1, window_size=16).to_c()
    for p in range(80):
        s = lib.hkv_slot_of_position(C.byref(ring), p)
        assert s == p % 16
        assert lib.hkv_position_of_slot(C.byref(ring), s, p + 1) == p
    # every row of a full ring holds one of the last 16 positions
    held = sorted(lib.hkv_position_of_slot(C.byref(ring), s, 50) for s in range(16))
    assert held == list(range(34, 50))
    # block-cyclic sequence split: every position has exactly one owner, rows are dense per rank
    N, BLK, slots = 4, 64, 256
    seen = {}
    for r in range(N):
        gr = hkv.Geometry(num_heads=4, num_kv_heads=2, head_dim=64, slots=slots, shard_rank=r,
                          shard_count=N, shard_block=BLK).to_c()
        for p in range(N * slots):
            s = lib.hkv_slot_of_position(C.byref(gr), p)
            if s >= 0:
                assert p not in seen
                seen[p] = (r, s)
                assert lib.hkv_position_of_slot(C.byref(gr), s, N * slots) == p
    assert len(seen) == N * slots
    for r in range(N):
        rows = sorted(s for (rr, s) in seen.values() if rr == r)
        assert rows == list(range(slots))


def test_split_plan_covers_attended_rows_exactly_once(hkv):
    lib = hkv._capi.load()
    rng = np.random.default_rng(0)
    for kw in (dict(slots=1000), dict(slots=1000, window_size=130), dict(slots=128, layout=1, window_size=128),
               dict(slots=300, layout=1, window_size=100)):
        geo = hkv.Geometry(num_heads=4, num_kv_heads=2, head_dim=64, **kw)
        g = geo.to_c()
        for total in [0, 1, 63, 64, 65, 127, 128, 129, 999, 1000] + list(rng.integers(1, 2000, 10)):
            total = int(total)
            if geo.layout == 0 and total > geo.slots:
                continue
            for ct in (1, 3, 16):
                first, tile_lo, n_tiles, n_chunks = _plan(hkv, geo, total, ct)
                assert n_chunks == -(-n_tiles // ct)
                attended = set(range(max(first, 0), total))
                covered = set()
                for s in range(tile_lo * 64, min((tile_lo + n_tiles) * 64, geo.slots)):
                    p = lib.hkv_position_of_slot(C.byref(g), s, total)
                    if first <= p < total:
                        assert p not in covered
                        covered.add(p)
                assert covered == attended, (kw, total, ct)


def test_sharded_plans_partition_the_sequence(hkv):
    lib = hkv._capi.load()
    N, BLK = 8, 128
    for total in (1, 127, 128, 129, 5000, 16384, 131072):
        covered = set()
        for r in range(N):
            geo = hkv.Geometry(num_heads=4, num_kv_heads=2, head_dim=64, slots=16384, shard_rank=r,
                               shard_count=N, shard_block=BLK)
            g = geo.to_c()
            first, tile_lo, n_tiles, _ = _plan(hkv, geo, total, 4)
            for s in range(tile_lo * 64, (tile_lo + n_tiles) * 64, 64):  # tile starts suffice
                p0 = lib.hkv_position_of_slot(C.byref(g), s, total)
                for p in range(p0, p0 + 64):
                    if p < total:
                        assert p not in covered
                        covered.add(p)
        assert len(covered) == total


def test_workspace_bytes_formula(hkv):
    geo = hkv.Geometry(batch=8, num_heads=28, num_kv_heads=4, head_dim=128, slots=4096, chunk_tiles=4)
    lib = hkv._capi.load()
    n = lib.hkv_workspace_bytes(C.byref(geo.to_c()))
    assert n == 8 * (4096 // 64 // 4) * 28 * (128 + 2) * 4
    assert lib.hkv_partial_floats(C.byref(geo.to_c())) == 130


def test_cache_owner_position_bookkeeping(hkv):
    """advance clamps, rewind_to only moves back, reset zeroes (src/kv_cache.hpp:93-96, :243-248)."""
    c = hkv.KVCache()
    c._max_seq = 10
    c.advance(4)
    assert c.position() == 4
    c.rewind_to(7)
    assert c.position() == 4
    c.rewind_to(2)
    assert c.position() == 2
    c.advance(100)
    assert c.position() == 10
    c.reset()
    assert c.position() == 0
    cfg = hkv.KVCacheConfig(num_layers=28, num_kv_heads=4, head_dim=128, max_batch_size=64, max_seq_len=32768)
    assert cfg.total_bytes() == 28 * 2 * 64 * 32768 * 4 * 128 * 2
    assert not hkv.KVCache().allocate(hkv.KVCacheConfig())  # zero dims refused like the reference


def _plan_prefill(hkv, g, seq_new, past, sms=148):
    lib = hkv._capi.load()
    vals = [C.c_int32() for _ in range(4)]
    st = lib.hkv_plan_prefill(C.byref(g.to_c()), seq_new, past, sms, *[C.byref(v) for v in vals])
    assert st == 0
    return [v.value for v in vals]   # tiles in flight, items, splits, min span


def test_prefill_plan_never_leaves_a_key_split_empty(hkv):
    """Host plan of the tensor-core prefill launch (no device needed): kernel choice, work items and
    key-range splits. With a sliding window the key span differs from item to item by a tile
    depending on how the window falls on the 128-row tile grid, so the split count must be bounded
    by the SHORTEST span over all items — a plan with an empty split makes the kernel wait for a
    tile that is never loaded."""
    # the headline shape: long pasts get split (148 SMs, 228 pair items x 4 kv heads... ), short ones do not
    g = hkv.Geometry(num_heads=28, num_kv_heads=4, head_dim=128, slots=131072, max_seq_new=2048)
    # 228 work items on 148 SMs: one full round of whole items, then the 80 shortest items' key tiles
    # cut into equal spans over all SMs (reported as splits == 0) — when the spans are long enough to pay
    assert _plan_prefill(hkv, g, 2048, 30720)[:3] == [2, 148, 0]
    # planes beyond the L2 (264 MB here) keep whole items in lockstep and take uniform key splits instead
    tif, items, splits, span = _plan_prefill(hkv, g, 2048, 129024)
    assert tif == 2 and splits > 1 and splits <= span and items == 57 * 4 * splits
    # short key ranges: pieces of a few tiles cost more than the idle SMs of the last round
    tif, items, splits, span = _plan_prefill(hkv, g, 2048, 0)
    assert (tif, items, splits) == (2, 228, 1) and span == 1
    # a forced split count keeps the uniform key splits of whole items
    gf = hkv.Geometry(num_heads=28, num_kv_heads=4, head_dim=128, slots=131072, max_seq_new=2048, tune_prefill_splits=3)
    assert _plan_prefill(hkv, gf, 2048, 129024)[:3] == [2, 57 * 4 * 3, 3]
    # a chunk that fits one query tile takes the one-tile kernel
    assert _plan_prefill(hkv, g, 18, 5000)[0] == 1 and _plan_prefill(hkv, g, 19, 5000)[0] == 2
    # without a workspace for partials there is no split
    g0 = hkv.Geometry(num_heads=28, num_kv_heads=4, head_dim=128, slots=131072, max_seq_new=0)
    assert _plan_prefill(hkv, g0, 2048, 129024)[2] == 1
    # head_dim 96 is staged as 128 and takes the same kernels; head_dim 256 only the one-tile kernel,
    # with 64-row key tiles
    g96 = hkv.Geometry(num_heads=32, num_kv_heads=32, head_dim=96, slots=4096, max_seq_new=0)
    assert _plan_prefill(hkv, g96, 256, 100) == [2, 1 * 32, 1, 3]
    g256 = hkv.Geometry(num_heads=16, num_kv_heads=8, head_dim=256, slots=4096, max_seq_new=0)
    tif, items, splits, span = _plan_prefill(hkv, g256, 2048, 1024)
    assert (tif, items, splits) == (1, 32 * 8, 1) and span == (1024 + 64) // 64 - 0
    # geometries the tensor-core kernels do not take: SIMT, one CTA per (query, head)
    g80 = hkv.Geometry(num_heads=32, num_kv_heads=32, head_dim=80, slots=4096, max_seq_new=256)
    assert _plan_prefill(hkv, g80, 256, 100) == [0, 256 * 32, 1, 0]
    # a ring plane whose rows are not a whole number of key tiles also falls to the SIMT kernel
    gring = hkv.Geometry(num_heads=8, num_kv_heads=8, head_dim=128, slots=200, window_size=50, layout=1)
    assert _plan_prefill(hkv, gring, 64, 1000)[0] == 0
    # window 119 over 36-query items: spans of 2 and 3 tiles alternate; forcing 3 or 4 splits must clamp to 2
    for forced in (1, 2, 3, 4):
        gw = hkv.Geometry(num_heads=7, num_kv_heads=1, head_dim=128, slots=1231, window_size=119, max_seq_new=345,
                          tune_prefill_splits=forced)
        tif, items, splits, span = _plan_prefill(hkv, gw, 345, 734)
        assert span == 2 and splits == min(forced, 2), (forced, splits, span)
    # and whatever the cost model picks on its own, over many shapes
    import numpy as np
    rng = np.random.default_rng(5)
    for _ in range(300):
        G = int(rng.choice([1, 2, 4, 7, 8])); KVH = int(rng.choice([1, 2, 4, 8]))
        S = int(rng.integers(1, 4000)); past = int(rng.integers(0, 200000))
        win = int(rng.choice([0, int(rng.integers(1, 5000))]))
        gg = hkv.Geometry(num_heads=G * KVH, num_kv_heads=KVH, head_dim=int(rng.choice([64, 96, 128, 256])),
                          slots=past + S + int(rng.integers(0, 300)), window_size=win, max_seq_new=S)
        sms = int(rng.choice([132, 148]))
        tif, items, splits, span = _plan_prefill(hkv, gg, S, past, sms=sms)
        assert tif in (1, 2) and items >= 1
        assert (splits == 0 and tif == 2 and items <= sms) or 1 <= splits <= min(span, 4)


def test_preferred_prefill_chunk_makes_items_a_multiple_of_the_sms(hkv):
    lib = hkv._capi.load()
    g = hkv.Geometry(num_heads=28, num_kv_heads=4, head_dim=128, slots=131072, max_seq_new=4096)
    gc = g.to_c()
    assert lib.hkv_preferred_prefill_chunk(C.byref(gc), 148, 2048) == 1332     # 37 pairs x 36 queries
    assert lib.hkv_preferred_prefill_chunk(C.byref(gc), 148, 3000) == 2664
    assert lib.hkv_preferred_prefill_chunk(C.byref(gc), 148, 100) == 1332      # never below one round
    g1 = hkv.Geometry(num_heads=28, num_kv_heads=4, head_dim=128, slots=131072, max_seq_new=4096, tune_prefill_splits=1)
    for target in (1332, 2664, 3996):
        tif, items, splits, span = _plan_prefill(hkv, g1, target, 30720)
        assert tif == 2 and splits == 1 and items % 148 == 0
    mha = hkv.Geometry(num_heads=8, num_kv_heads=8, head_dim=64, slots=4096, max_seq_new=4096)
    assert lib.hkv_preferred_prefill_chunk(C.byref(mha.to_c()), 148, 10000) == 9472   # 37 pairs x 256
    simt = hkv.Geometry(num_heads=32, num_kv_heads=32, head_dim=80, slots=4096)
    assert lib.hkv_preferred_prefill_chunk(C.byref(simt.to_c()), 148, 777) == 777
    # head_dim 256: one query tile per item (64 queries at group 2), 148 items x ... / gcd(148, 8) = 37 tiles a round
    g256 = hkv.Geometry(num_heads=16, num_kv_heads=8, head_dim=256, slots=4096)
    assert lib.hkv_preferred_prefill_chunk(C.byref(g256.to_c()), 148, 3000) == 37 * 64
    assert lib.hkv_preferred_prefill_chunk(C.byref(gc), 0, 2048) < 0


def test_decode_tile_run_of_a_ring_larger_than_its_window_covers_exactly_the_window(hkv):
    """Index arithmetic of the decode kernel's tile walk (csrc/hkv_common.cuh: tma_tile_range), checked on
    the host over random rings: the cyclic run of tiles holds every row with an attended position, every
    tile of the run holds at least one such row (nothing is read for nothing), and it never laps the ring."""
    lib = hkv._capi.load()
    rng = np.random.default_rng(11)
    for _ in range(400):
        ring_tiles = int(rng.integers(2, 40))
        slots = ring_tiles * 64
        window = int(rng.integers(1, slots))
        total = int(rng.integers(slots + 1, slots * 6))
        g = hkv.Geometry(batch=1, num_heads=8, num_kv_heads=2, head_dim=64, slots=slots, window_size=window, layout=1).to_c()
        tl, nt, wt = C.c_int32(), C.c_int32(), C.c_int32()
        assert lib.hkv_plan_decode_tiles(C.byref(g), total, C.byref(tl), C.byref(nt), C.byref(wt)) == 0
        assert wt.value == ring_tiles and 1 <= nt.value <= ring_tiles and 0 <= tl.value < ring_tiles
        run = [(tl.value + t) % ring_tiles for t in range(nt.value)]
        assert len(set(run)) == len(run), "the run laps the ring"
        attended_tiles = {(p % slots) // 64 for p in range(total - window, total)}
        assert attended_tiles == set(run), (slots, window, total, run, sorted(attended_tiles))
    # planes that are not such rings walk a plain run: no wrap
    for geo in (dict(slots=1024, window_size=1024, layout=1), dict(slots=4096, window_size=0, layout=0),
                dict(slots=4096, window_size=512, layout=0), dict(slots=1000, window_size=256, layout=1)):
        g = hkv.Geometry(batch=1, num_heads=8, num_kv_heads=2, head_dim=64, **geo).to_c()
        tl, nt, wt = C.c_int32(), C.c_int32(), C.c_int32()
        assert lib.hkv_plan_decode_tiles(C.byref(g), 5000, C.byref(tl), C.byref(nt), C.byref(wt)) == 0
        assert wt.value == 0 and (tl.value + nt.value) * 64 <= ((geo["slots"] + 63) // 64) * 64


def test_equal_span_schedule_agrees_between_the_decode_and_the_merge_side(hkv):
    """The decode kernel cuts the line of tiles at floor(T*c/S); the merge kernel finds a sequence's
    partials with the inverse (span_owner). Over random batches: a span overlaps a sequence exactly when
    the merge side lists it, and the partial slot span + b is used by one piece only."""
    lib = hkv._capi.load()
    rng = np.random.default_rng(5)
    for _ in range(300):
        B = int(rng.integers(1, 70))
        slots = int(rng.integers(1, 600)) * 64
        g = hkv.Geometry(batch=B, num_heads=8, num_kv_heads=2, head_dim=64, slots=slots).to_c()
        totals = rng.integers(0, slots + 1, size=B).astype(np.int32)
        totals[rng.random(B) < 0.1] = 0                      # free batch slots
        want = int(rng.choice([1, 37, 74, 148, 296]))
        first, parts = np.zeros(B, np.int32), np.zeros(B, np.int32)
        T, S = C.c_int32(), C.c_int32()
        assert lib.hkv_plan_decode_spans(C.byref(g), totals.ctypes.data, want, first.ctypes.data, parts.ctypes.data,
                                         C.byref(T), C.byref(S)) == 0
        tiles = (totals.astype(np.int64) + 63) // 64
        pre = np.concatenate([[0], np.cumsum(tiles)])
        assert T.value == pre[-1] and S.value == min(want, max(T.value, 0))
        used = set()
        for c in range(S.value):
            u0, u1 = T.value * c // S.value, T.value * (c + 1) // S.value
            assert u1 > u0, "an empty span"
            for b in range(B):
                overlaps = tiles[b] > 0 and pre[b] < u1 and pre[b + 1] > u0
                listed = parts[b] > 0 and first[b] <= c < first[b] + parts[b]
                assert overlaps == listed, (B, want, c, b)
                if overlaps:
                    assert c + b not in used, "two pieces share a partial slot"
                    used.add(c + b)
        assert all(parts[b] == 0 for b in range(B) if tiles[b] == 0)
        assert max(used, default=0) < S.value + B            # the workspace holds spans + batch slots
