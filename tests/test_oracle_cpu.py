"""CPU suite: pins the oracle (oracle/hkv_oracle.cpp) against the reference's own
known-answer cases and checks its internal consistency. No GPU needed."""
import numpy as np
import pytest

from _kat import build, load_kats
from _util import ATOL, RTOL, make_case, normal_f16

KATS = load_kats()


@pytest.mark.parametrize("case", KATS["cases"], ids=lambda c: c["name"])
@pytest.mark.parametrize("mode", [0, 1], ids=["exact", "ref16"])
def test_reference_known_answers(oracle, case, mode):
    q, k, v, scale, expect = build(case)
    if case["op"] == "decode":
        out = oracle.decode(q.reshape(1, case["H"], case["HD"]), k, v, [case["seq_len"]], scale,
                            window=case["window"], mode=mode)
        got = out.astype(np.float32).reshape(1, -1)
    else:
        if mode == 1:
            pytest.skip("prefill has one oracle mode")
        out = oracle.prefill(q, k[0], v[0], case["past_len"], scale, window=case["window"])
        got = out.astype(np.float32).reshape(case["seq_new"], -1)
    assert np.all(np.abs(got - expect) < 0.01), (got, expect)  # the reference's own tolerance


def test_heterogeneous_layout_bytes(oracle, hkv):
    L = KATS["layout"]
    n = L["layers"]
    is_global = [1 if i % L["global_every"] == L["global_every"] - 1 else 0 for i in range(n)]
    head_dim = [L["head_dim_global"] if g else L["head_dim_local"] for g in is_global]
    total, source, offset, rows = oracle.gemma4_layout(head_dim, is_global, L["num_kv_shared_layers"],
                                                       L["num_kv_heads"], L["batch"], L["max_seq"])
    assert total * 2 * 2 == L["total_bytes"]
    assert n - L["num_kv_shared_layers"] == L["physical_slots"]
    for layer, src in L["aliases"].items():
        assert source[int(layer)] == src
        assert offset[int(layer)] == offset[src]
    # the host package's layout arithmetic agrees with the oracle's
    layers = [hkv.Gemma4Layer(hd, bool(g)) for hd, g in zip(head_dim, is_global)]
    lay = hkv.gemma4_layout(layers, L["num_kv_shared_layers"], L["num_kv_heads"], L["batch"], L["max_seq"])
    assert lay.elements_per_plane == total and lay.first_shared == L["physical_slots"]
    assert lay.source == list(source) and lay.offset == list(offset) and lay.rows == list(rows)
    # invalid layouts are refused like the reference's allocate()
    assert hkv.gemma4_layout(layers, n, 1, 1, 8) is None          # every layer shared
    assert hkv.gemma4_layout(layers, n + 1, 1, 1, 8) is None
    assert hkv.gemma4_layout([], 0, 1, 1, 8) is None
    # ring planes for local owners shrink the budget
    ring = hkv.gemma4_layout(layers, L["num_kv_shared_layers"], 1, 1, 4096, ring_window=512)
    lin = hkv.gemma4_layout(layers, L["num_kv_shared_layers"], 1, 1, 4096)
    assert ring.elements_per_plane < lin.elements_per_plane
    assert all(r == (4096 if g else 512) for r, g in zip(ring.rows[:15], is_global[:15]))


def test_exact_and_reference_order_agree(oracle):
    """The position-ordered two-pass oracle and the reference's 16-chunk online order differ
    only by rounding: both modes must sit well inside the path's tolerance of each other."""
    for seed, (B, H, KVH, HD, slots, window) in enumerate([
            (2, 14, 2, 64, 600, 0), (1, 28, 4, 128, 1500, 0), (2, 32, 32, 96, 300, 0),
            (1, 16, 8, 256, 700, 256), (3, 4, 2, 32, 40, 7)]):
        totals = np.random.default_rng(seed).integers(1, slots + 1, size=B).astype(np.int32)
        q, _, _, kc, vc = make_case(seed, B, H, KVH, HD, slots, totals)
        for scale in (1.0 / np.sqrt(HD), 1.0):
            a = oracle.decode(q, kc, vc, totals, scale, window=window, mode=0)
            b = oracle.decode(q, kc, vc, totals, scale, window=window, mode=1)
            ok, err = oracle.within_tolerance(b, a, ATOL / 2, RTOL / 2)
            assert ok, (seed, scale, err)


def test_decode_edge_cases(oracle):
    q, _, _, kc, vc = make_case(7, 3, 4, 2, 16, 32, fill="garbage")
    # total = 0 -> zeros (kernels/attention.cu:478); total = 1 -> output = V row 0
    out = oracle.decode(q, kc, vc, [0, 1, 32], 0.25)
    assert np.all(out[0] == 0)
    G = 2
    for h in range(4):
        assert np.array_equal(out[1, h], vc[1, 0, h // G])
    # rows past `total` are never read: garbage there changes nothing
    kc2, vc2 = kc.copy(), vc.copy()
    kc2[1, 1:] = np.float16(np.nan)
    vc2[1, 1:] = np.float16(np.inf)
    out2 = oracle.decode(q, kc2, vc2, [0, 1, 32], 0.25)
    assert np.array_equal(out.view(np.uint16), out2.view(np.uint16))
    # a window covering everything equals no window
    a = oracle.decode(q, kc, vc, [5, 9, 32], 0.25, window=64)
    b = oracle.decode(q, kc, vc, [5, 9, 32], 0.25, window=0)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_append_semantics(oracle):
    rng = np.random.default_rng(3)
    B, S, KVH, HD, slots = 3, 4, 2, 8, 10
    nk, nv = normal_f16(rng, B, S, KVH, HD), normal_f16(rng, B, S, KVH, HD)
    kc = normal_f16(rng, B, slots, KVH, HD)
    vc = normal_f16(rng, B, slots, KVH, HD)
    k0, v0 = kc.copy(), vc.copy()
    pos = np.array([0, 5, 8], dtype=np.int32)  # sequence 2 runs off the end: rows 10, 11 dropped
    oracle.append(nk, nv, kc, vc, pos)
    for b in range(B):
        for s in range(S):
            p = pos[b] + s
            if p < slots:
                assert np.array_equal(kc[b, p], nk[b, s]) and np.array_equal(vc[b, p], nv[b, s])
    untouched = np.ones((B, slots), dtype=bool)
    for b in range(B):
        untouched[b, pos[b]:min(pos[b] + S, slots)] = False
    assert np.array_equal(kc[untouched], k0[untouched]) and np.array_equal(vc[untouched], v0[untouched])
    # ring layout wraps instead of dropping
    kr, vr = k0.copy(), v0.copy()
    oracle.append(nk, nv, kr, vr, pos, layout=1)
    assert np.array_equal(kr[2, 0], nk[2, 2]) and np.array_equal(kr[2, 1], nk[2, 3])


def test_ring_equals_linear_window(oracle):
    """A ring of W rows indexed by pos mod W must give what the reference computes on a
    linear cache with window_size = W (the reference has no ring layout)."""
    rng = np.random.default_rng(11)
    B, H, KVH, HD, W, ctx = 2, 4, 2, 32, 16, 50
    lin_k = np.zeros((B, ctx, KVH, HD), np.float16)
    lin_v = np.zeros_like(lin_k)
    ring_k = np.zeros((B, W, KVH, HD), np.float16)
    ring_v = np.zeros_like(ring_k)
    for p in range(ctx):
        nk, nv = normal_f16(rng, B, 1, KVH, HD), normal_f16(rng, B, 1, KVH, HD)
        pos = np.full(B, p, np.int32)
        oracle.append(nk, nv, lin_k, lin_v, pos, layout=0)
        oracle.append(nk, nv, ring_k, ring_v, pos, layout=1)
        q = normal_f16(rng, B, H, HD)
        tot = pos + 1
        a = oracle.decode(q, lin_k, lin_v, tot, 0.2, window=W, layout=0)
        b = oracle.decode(q, ring_k, ring_v, tot, 0.2, window=W, layout=1)
        # same attended set in the same position order -> identical bits
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16)), p


def test_prefill_equals_decode_per_query(oracle):
    rng = np.random.default_rng(5)
    H, KVH, HD, slots, past, S_new, window = 6, 2, 32, 64, 20, 9, 12
    k = normal_f16(rng, 1, slots, KVH, HD)
    v = normal_f16(rng, 1, slots, KVH, HD)
    q = normal_f16(rng, S_new, H, HD)
    out = oracle.prefill(q, k[0], v[0], past, 0.3, window=window)
    for i in range(S_new):
        ref = oracle.decode(q[i:i + 1], k, v, [past + i + 1], 0.3, window=window)
        assert np.array_equal(out[i].view(np.uint16), ref[0].view(np.uint16))


def test_synthetic_stream_properties(oracle):
    x = oracle.fill(0x48454B56, 0, 200000).astype(np.float32)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    # counter based: any window of the stream can be regenerated on its own
    y = oracle.fill(0x48454B56, 1234, 100)
    assert np.array_equal(y.view(np.uint16), oracle.fill(0x48454B56, 0, 200000)[1234:1334].view(np.uint16))
