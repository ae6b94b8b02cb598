"""GPU parity of prefill-over-cache attention (hkv_prefill_attention) against the oracle:
the tcgen05 tensor-core kernels (head_dim 64 / 96 / 128 / 256, linear and ring planes) and the
any-geometry SIMT kernel, on the same seeded inputs. Tolerance: |x - ref| <= 2e-3 + 1e-2*|ref| per fp16 element."""
import math

import numpy as np
import pytest

from _util import assert_close, normal_f16, to_dev

pytestmark = pytest.mark.gpu

CASES = [
    # name, H, KVH, HD, slots, past_len, S_new, window
    ("qwen7b_group7_multi_tile", 28, 4, 128, 2048, 1000, 200, 0),
    ("qwen7b_from_empty_cache", 28, 4, 128, 512, 0, 300, 0),
    ("qwen05b_hd64_group7", 14, 2, 64, 1024, 333, 77, 0),
    ("mha_hd64", 8, 8, 64, 640, 100, 260, 0),
    ("group2_window", 16, 8, 128, 1024, 500, 150, 96),
    ("group16_window_small", 32, 2, 64, 512, 40, 90, 17),
    ("single_query", 28, 4, 128, 256, 130, 1, 0),
    ("fills_plane_exactly", 28, 4, 128, 384, 256, 128, 0),
    ("phi3_mha_hd96", 8, 8, 96, 1024, 450, 170, 0),
    ("hd96_group4_window", 16, 4, 96, 768, 300, 100, 130),
    ("gemma_hd256_group2", 16, 8, 256, 1024, 500, 150, 0),
    ("gemma_hd256_window_from_empty", 8, 4, 256, 512, 0, 333, 100),
    ("hd256_single_query", 4, 2, 256, 256, 200, 1, 0),
]


@pytest.mark.parametrize("kernel", [0, 1], ids=["tensor_core", "simt"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_prefill_matches_oracle(hkv, cuda, oracle, case, kernel):
    torch = cuda
    name, H, KVH, HD, slots, past, S_new, window = case
    rng = np.random.default_rng(len(name) * 7919 + HD)
    k = normal_f16(rng, 1, slots, KVH, HD)
    v = normal_f16(rng, 1, slots, KVH, HD)
    # rows past the chunk are stale memory in a real cache: poison them
    k[0, past + S_new:] = np.float16(np.nan)
    v[0, past + S_new:] = np.float16(np.inf)
    q = normal_f16(rng, S_new, H, HD)
    for scale in (1.0 / math.sqrt(HD), 1.0):
        ref = oracle.prefill(q, k[0], v[0], past, scale, window=window, threads=8)
        ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                       window_size=window, kernel_select=kernel, max_seq_new=S_new))
        out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
        ctx.prefill_attention(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out, S_new, past, scale)
        assert ctx.device_status() == 0
        got = out.cpu().numpy()
        assert not np.isnan(got.astype(np.float32)).any()
        assert_close(oracle, got, ref, f"{name} scale={scale:.3f}")
        ctx.close()


def test_chunked_prefill_then_decode_agree(hkv, cuda, oracle):
    """Append a chunk, attend it with the prefill kernel, then decode the next token: the
    last query of the chunk through prefill equals a decode call at that position."""
    torch = cuda
    H, KVH, HD, slots, past, S_new = 28, 4, 128, 1024, 300, 140
    rng = np.random.default_rng(99)
    kc = normal_f16(rng, 1, slots, KVH, HD)
    vc = normal_f16(rng, 1, slots, KVH, HD)
    nk, nv = normal_f16(rng, 1, S_new, KVH, HD), normal_f16(rng, 1, S_new, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    ctx.append_at(to_dev(torch, nk), to_dev(torch, nv), dk, dv, past, S_new)      # KV_CACHE_UPDATE first
    out = torch.zeros(S_new, H, HD, dtype=torch.float16, device="cuda")
    ctx.prefill_attention(to_dev(torch, q), dk, dv, out, S_new, past, scale)      # then ATTENTION_PREFILL_CACHED
    one = torch.zeros(1, H, HD, dtype=torch.float16, device="cuda")
    ctx.decode_attention_len(to_dev(torch, q[-1:]), dk, dv, one, past + S_new, scale)
    assert ctx.device_status() == 0
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, np.array([past], np.int32))
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    ref = oracle.prefill(q, ref_k[0], ref_v[0], past, scale, threads=8)
    assert_close(oracle, out.cpu().numpy(), ref, "chunk through prefill")
    assert_close(oracle, one.cpu().numpy()[0], ref[-1], "last query through decode")
    ctx.close()


VARIANT_CASES = [CASES[0], CASES[2], CASES[4], CASES[8], CASES[10]]


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 4], ids=["own_schedule", "1", "2", "3", "4"])
@pytest.mark.parametrize("tiles_in_flight", [1, 2], ids=["one_tile_kernel", "two_tile_kernel"])
@pytest.mark.parametrize("case", VARIANT_CASES, ids=lambda c: c[0])
def test_prefill_kernel_variants_and_key_splits(hkv, cuda, oracle, case, tiles_in_flight, splits):
    """Both tensor-core kernels and every key-split count (normally chosen by the cost model; forced
    here through the tune_* fields of the geometry) give the oracle's result."""
    torch = cuda
    name, H, KVH, HD, slots, past, S_new, window = case
    rng = np.random.default_rng(4242 + splits)
    k = normal_f16(rng, 1, slots, KVH, HD)
    v = normal_f16(rng, 1, slots, KVH, HD)
    k[0, past + S_new:] = np.float16(np.nan)
    v[0, past + S_new:] = np.float16(np.inf)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.prefill(q, k[0], v[0], past, scale, window=window, threads=8)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   window_size=window, max_seq_new=S_new, tune_prefill_kernel=tiles_in_flight,
                                   tune_prefill_splits=splits))
    out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    for _ in range(3):   # repeated launches reuse the split workspace
        ctx.prefill_attention(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out, S_new, past, scale)
    assert ctx.device_status() == 0
    assert_close(oracle, out.cpu().numpy(), ref, f"{name} kernel={tiles_in_flight} splits={splits}")
    ctx.close()


@pytest.mark.parametrize("tiles_in_flight", [1, 2], ids=["one_tile_kernel", "two_tile_kernel"])
def test_prefill_row_maxima_that_keep_growing(hkv, cuda, oracle, tiles_in_flight):
    """Keys whose magnitude grows with the position make every tile's row maximum outgrow the
    running reference by far more than 2^8: the in-place rescale of O in tensor memory runs on
    (almost) every tile, and scores span hundreds of units."""
    torch = cuda
    H, KVH, HD, slots, past, S_new = 14, 2, 128, 2048, 1500, 120
    rng = np.random.default_rng(77)
    k = normal_f16(rng, 1, slots, KVH, HD).astype(np.float32)
    k *= (0.25 + np.arange(slots, dtype=np.float32) / 256.0)[None, :, None, None]   # up to 8x at the end
    k = k.astype(np.float16)
    v = normal_f16(rng, 1, slots, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0   # scores ~ N(0, HD) * growth: far apart
    ref = oracle.prefill(q, k[0], v[0], past, scale, threads=8)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, max_seq_new=S_new,
                                   tune_prefill_kernel=tiles_in_flight))
    out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.prefill_attention(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out, S_new, past, scale)
    assert ctx.device_status() == 0
    got = out.cpu().numpy()
    assert not np.isnan(got.astype(np.float32)).any()
    assert_close(oracle, got, ref, f"growing maxima, kernel={tiles_in_flight}")
    ctx.close()


def test_prefill_seeded_random_shapes(hkv, cuda, oracle):
    """Thirty seeded random geometries (group size, head_dim 64/96/128/256, chunk and past lengths that are
    not multiples of any tile, windows, forced key splits, both tensor-core kernels): every one must
    match the oracle. Catches protocol slips that only show for particular tile counts per item."""
    torch = cuda
    rng = np.random.default_rng(20241125)
    for i in range(30):
        HD = int(rng.choice([64, 128, 96, 256]))
        KVH = int(rng.choice([1, 2, 4]))
        G = int(rng.choice([1, 2, 4, 7, 8]))
        H = KVH * G
        S_new = int(rng.integers(1, 420))
        past = int(rng.integers(0, 1500))
        slots = int(past + S_new + rng.integers(0, 200))
        window = int(rng.choice([0, 0, int(rng.integers(1, 700))]))
        kernel_variant = int(rng.choice([1, 2]))
        forced_splits = int(rng.choice([0, 0, 1, 2, 3, 4]))   # 0: the library's own schedule (equal spans)
        k = normal_f16(rng, 1, slots, KVH, HD)
        v = normal_f16(rng, 1, slots, KVH, HD)
        k[0, past + S_new:] = np.float16(np.nan)
        v[0, past + S_new:] = np.float16(np.inf)
        q = normal_f16(rng, S_new, H, HD)
        scale = float(rng.choice([1.0 / math.sqrt(HD), 0.5]))
        ref = oracle.prefill(q, k[0], v[0], past, scale, window=window, threads=8)
        ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                       window_size=window, max_seq_new=S_new, tune_prefill_kernel=kernel_variant,
                                       tune_prefill_splits=forced_splits))
        out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
        ctx.prefill_attention(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out, S_new, past, scale)
        assert ctx.device_status() == 0, f"case {i}"
        got = out.cpu().numpy()
        assert not np.isnan(got.astype(np.float32)).any(), f"case {i}: NaN"
        assert_close(oracle, got, ref, f"case {i}: H={H} KVH={KVH} HD={HD} S_new={S_new} past={past} "
                                        f"slots={slots} window={window}")
        ctx.close()


RING_CASES = [
    # name, H, KVH, HD, ring rows, window, past_len, S_new
    ("ring_not_wrapped_yet", 16, 8, 256, 512, 128, 100, 200),
    ("ring_wrapped_hd256", 16, 8, 256, 512, 128, 1900, 300),          # 300 + 128 - 1 <= 512
    ("ring_wrapped_hd128_group7", 28, 4, 128, 1024, 256, 5000, 700),
    ("ring_wrapped_hd96", 8, 8, 96, 256, 100, 777, 150),
    ("ring_exact_fit", 8, 2, 64, 256, 129, 1000, 128),               # 128 + 129 - 1 == 256
]


@pytest.mark.parametrize("kernel", [0, 1], ids=["tensor_core", "simt"])
@pytest.mark.parametrize("case", RING_CASES, ids=lambda c: c[0])
def test_prefill_over_a_ring_plane_equals_linear_plane_with_window(hkv, cuda, oracle, case, kernel):
    """A sliding-window layer kept in a ring plane (position p in row p % rows; not in the reference,
    which keeps a linear plane and masks): a prefill chunk appended into the ring and attended there
    equals the oracle on the linear plane with the same window, as long as chunk + window - 1 fits the
    ring. The chunk's rows are appended by the library itself (hkv_append_at wraps)."""
    torch = cuda
    name, H, KVH, HD, rows, window, past, S_new = case
    rng = np.random.default_rng(len(name) * 31 + HD)
    total = past + S_new
    lin_k = normal_f16(rng, 1, total, KVH, HD)
    lin_v = normal_f16(rng, 1, total, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.prefill(q, lin_k[0], lin_v[0], past, scale, window=window, threads=8)
    # the ring before the chunk: the last `rows` positions below past_len, everything else poison
    ring_k = np.full((1, rows, KVH, HD), np.nan, np.float16)
    ring_v = np.full((1, rows, KVH, HD), np.inf, np.float16)
    for p in range(max(0, past - rows), past):
        ring_k[0, p % rows], ring_v[0, p % rows] = lin_k[0, p], lin_v[0, p]
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=rows,
                                   window_size=window, layout=hkv.LAYOUT_RING, kernel_select=kernel, max_seq_new=S_new))
    dk, dv = to_dev(torch, ring_k), to_dev(torch, ring_v)
    ctx.append_at(to_dev(torch, lin_k[:, past:]), to_dev(torch, lin_v[:, past:]), dk, dv, past, S_new)
    out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.prefill_attention(to_dev(torch, q), dk, dv, out, S_new, past, scale)
    assert ctx.device_status() == 0
    got = out.cpu().numpy()
    assert not np.isnan(got.astype(np.float32)).any()
    assert_close(oracle, got, ref, name)
    assert ctx.plan_prefill(S_new, past)[0] == (0 if kernel == 1 else (1 if HD == 256 or S_new <= 128 // (H // KVH) else 2))
    ctx.close()


def test_prefill_refuses_a_chunk_that_overwrites_what_it_attends(hkv, cuda):
    """Ring of 256 rows, window 200, chunk of 100 at position 1000: the first query needs position 801,
    which the chunk's last row (1099 -> row 1099 % 256) has overwritten (100 + 200 - 1 > 256)."""
    torch = cuda
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=4, num_kv_heads=4, head_dim=64, slots=256, window_size=200,
                                   layout=hkv.LAYOUT_RING))
    t = torch.zeros(256 * 4 * 64, dtype=torch.float16, device="cuda")
    with pytest.raises(hkv.HkvError) as e:
        ctx.prefill_attention(t, t, t, t, 100, 1000, 1.0)
    assert e.value.status == 2 and "do not fit the ring" in str(e.value)
    ctx.prefill_attention(t, t, t, t, 57, 1000, 1.0)    # 57 + 200 - 1 == 256 fits
    ctx.prefill_attention(t, t, t, t, 100, 100, 1.0)    # nothing overwritten yet
    torch.cuda.synchronize()
    ctx.close()


EXACT_RING_CASES = [
    # name, H, KVH, HD, ring rows (= window), past_len, S_new
    ("gemma_local_first_chunk", 16, 8, 256, 1024, 0, 512),
    ("gemma_local_second_chunk_fills_the_ring", 16, 8, 256, 1024, 512, 512),
    ("gemma_local_wrapped", 16, 8, 256, 1024, 30720, 512),
    ("hd128_group7_wrapped_ragged", 28, 4, 128, 256, 1000, 200),
    ("hd96_wrapped_chunk_as_long_as_the_ring", 8, 8, 96, 256, 777, 256),
    ("hd64_single_query", 8, 2, 64, 128, 5000, 1),
]


@pytest.mark.parametrize("case", EXACT_RING_CASES, ids=lambda c: c[0])
def test_prefill_chunk_into_a_ring_of_exactly_window_rows(hkv, cuda, oracle, case):
    """A sliding-window layer whose ring holds exactly `window` rows cannot take a chunk and then attend it
    (the chunk would overwrite rows its first queries still need): hkv_prefill_append_attention attends
    first — the cached rows and the chunk's own K/V in two tensor-core passes, merged — and appends
    afterwards. Output equals the oracle on a linear plane with the same window; the ring afterwards holds
    the last `rows` positions bit-exact."""
    torch = cuda
    name, H, KVH, HD, rows, past, S_new = case
    window = rows
    rng = np.random.default_rng(len(name) * 17 + HD)
    total = past + S_new
    lin_k = normal_f16(rng, 1, total, KVH, HD)
    lin_v = normal_f16(rng, 1, total, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.prefill(q, lin_k[0], lin_v[0], past, scale, window=window, threads=8)
    ring_k = np.full((1, rows, KVH, HD), np.nan, np.float16)     # rows never written: poison
    ring_v = np.full((1, rows, KVH, HD), np.inf, np.float16)
    for p in range(max(0, past - rows), past):
        ring_k[0, p % rows], ring_v[0, p % rows] = lin_k[0, p], lin_v[0, p]
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=rows,
                                   window_size=window, layout=hkv.LAYOUT_RING, max_seq_new=512))
    dk, dv = to_dev(torch, ring_k), to_dev(torch, ring_v)
    out = torch.full((S_new, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.prefill_append_attention(to_dev(torch, q), to_dev(torch, lin_k[0, past:]), to_dev(torch, lin_v[0, past:]),
                                 dk, dv, out, S_new, past, scale)
    assert ctx.device_status() == 0
    got = out.cpu().numpy()
    assert not np.isnan(got.astype(np.float32)).any()
    assert_close(oracle, got, ref, name)
    want_k, want_v = ring_k.copy(), ring_v.copy()
    for p in range(past, total):
        want_k[0, p % rows], want_v[0, p % rows] = lin_k[0, p], lin_v[0, p]
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), want_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), want_v.view(np.uint16))
    ctx.close()


def test_prefill_append_attention_on_a_linear_plane_is_append_then_attend(hkv, cuda, oracle):
    """Where the plane holds the chunk next to what it attends the combined entry point is the
    reference's own pair of ops: KV_CACHE_UPDATE, then ATTENTION_PREFILL_CACHED."""
    torch = cuda
    H, KVH, HD, slots, past, S_new = 28, 4, 128, 1024, 300, 140
    rng = np.random.default_rng(5)
    kc, vc = normal_f16(rng, 1, slots, KVH, HD), normal_f16(rng, 1, slots, KVH, HD)
    nk, nv = normal_f16(rng, 1, S_new, KVH, HD), normal_f16(rng, 1, S_new, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, np.array([past], np.int32))
    ref = oracle.prefill(q, ref_k[0], ref_v[0], past, scale, threads=8)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, max_seq_new=512))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.zeros(S_new, H, HD, dtype=torch.float16, device="cuda")
    ctx.prefill_append_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out, S_new, past, scale)
    assert ctx.device_status() == 0
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert_close(oracle, out.cpu().numpy(), ref, "append then attend")
    ctx.close()
