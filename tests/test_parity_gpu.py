"""GPU parity suite: libhkv's CUDA kernels, called through the C ABI, against the CPU
oracle on the same seeded inputs. Append: bit-exact over the whole plane. Attention:
|x - ref| <= 2e-3 + 1e-2*|ref| on every fp16 output element."""
import math
import zlib

import numpy as np
import pytest

from _kat import build, load_kats
from _util import assert_close, make_case, normal_f16, to_dev

pytestmark = pytest.mark.gpu
KATS = load_kats()

GENERIC, TMA = 1, 2


def run_decode(hkv, torch, q, kc, vc, totals, scale, *, H, KVH, HD, window=0, layout=0, kernel=0,
               chunk_tiles=0):
    B, slots = kc.shape[0], kc.shape[1]
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   window_size=window, layout=layout, kernel_select=kernel,
                                   chunk_tiles=chunk_tiles))
    dq, dk, dv = to_dev(torch, q), to_dev(torch, kc), to_dev(torch, vc)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    dt = to_dev(torch, np.asarray(totals, dtype=np.int32))
    ctx.decode_attention(dq, dk, dv, out, dt, scale)
    assert ctx.device_status() == 0
    res = out.cpu().numpy()
    kern = ctx.kernel
    ctx.close()
    return res, kern


# ---------------------------------------------------------------------------
# known answers of the reference's own test, through the GPU path
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("case", KATS["cases"], ids=lambda c: c["name"])
def test_reference_known_answers_on_gpu(hkv, cuda, case):
    torch = cuda
    q, k, v, scale, expect = build(case)
    H, KVH, HD, S = case["H"], case["KVH"], case["HD"], case["max_seq"]
    if case["op"] == "decode":
        out = torch.zeros(1, H, HD, dtype=torch.float16, device="cuda")
        # host-length launcher, as the reference test calls it (engine.execute, no device pos)
        hkv.launch_attention_cached_fp16(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out, 1,
                                         case["seq_len"], H, KVH, HD, S, scale, case["window"])
        got = out.cpu().numpy().astype(np.float32).reshape(1, -1)
    else:
        out = torch.zeros(case["seq_new"], H, HD, dtype=torch.float16, device="cuda")
        hkv.launch_attention_prefill_cached_fp16(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v),
                                                 out, case["seq_new"], case["past_len"], H, KVH, HD, S,
                                                 scale, case["window"])
        got = out.cpu().numpy().astype(np.float32).reshape(case["seq_new"], -1)
    torch.cuda.synchronize()
    assert np.all(np.abs(got - expect) < 0.01), (got, expect)


# ---------------------------------------------------------------------------
# append: bit-exact
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("B,S,KVH,HD,slots,layout", [
    (1, 1, 2, 64, 2048, 0),     # config 1 shape
    (8, 1, 4, 128, 4096, 0),    # config 2 shape
    (16, 1, 32, 96, 512, 0),    # config 3 shape (non power of two head_dim)
    (8, 1, 8, 256, 1024, 1),    # config 4 local layer: ring
    (3, 5, 2, 64, 40, 0),       # multi-token, runs off the end for one sequence
    (3, 5, 2, 64, 16, 1),       # multi-token ring wrap
    (2, 3, 1, 2, 9, 0),         # tiny head_dim: 2-byte path
    (2, 1, 3, 7, 9, 0),         # odd row size: 2-byte path
])
def test_append_bit_exact(hkv, cuda, oracle, B, S, KVH, HD, slots, layout):
    torch = cuda
    rng = np.random.default_rng(B * 1000 + HD)
    nk, nv = normal_f16(rng, B, S, KVH, HD), normal_f16(rng, B, S, KVH, HD)
    kc, vc = normal_f16(rng, B, slots, KVH, HD), normal_f16(rng, B, slots, KVH, HD)
    if layout == 1:
        pos = rng.integers(0, 5 * slots, size=B).astype(np.int32)
    else:
        pos = rng.integers(0, slots, size=B).astype(np.int32)
        pos[-1] = slots - 2  # crosses the end when S > 2: rows past the plane are dropped
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos, layout=layout)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=KVH, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   layout=layout))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    ctx.append(to_dev(torch, nk), to_dev(torch, nv), dk, dv, to_dev(torch, pos), S)
    torch.cuda.synchronize()
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    # host-position twin (launch_kv_cache_update): every sequence writes at the same position
    if layout == 0:
        ref_k, ref_v = kc.copy(), vc.copy()
        oracle.append(nk, nv, ref_k, ref_v, np.full(B, 3, np.int32))
        dk, dv = to_dev(torch, kc), to_dev(torch, vc)
        hkv.launch_kv_cache_update(to_dev(torch, nk), to_dev(torch, nv), dk, dv, B, S, KVH, HD, slots, 3)
        torch.cuda.synchronize()
        assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
        assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    ctx.close()


def test_append_unaligned_views_use_narrow_stores(hkv, cuda, oracle):
    """k_new/v_new may be views into a fused QKV buffer that are only 2-byte aligned."""
    torch = cuda
    rng = np.random.default_rng(9)
    B, KVH, HD, slots = 2, 2, 64, 32
    nk, nv = normal_f16(rng, B, 1, KVH, HD), normal_f16(rng, B, 1, KVH, HD)
    kc, vc = normal_f16(rng, B, slots, KVH, HD), normal_f16(rng, B, slots, KVH, HD)
    pos = np.array([4, 31], np.int32)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos)
    buf = torch.zeros(nk.size + nv.size + 8, dtype=torch.float16, device="cuda")
    buf[1:1 + nk.size] = to_dev(torch, nk).flatten()            # offset by one half: 2-byte aligned
    buf[3 + nk.size:3 + nk.size + nv.size] = to_dev(torch, nv).flatten()
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=KVH, num_kv_heads=KVH, head_dim=HD, slots=slots))
    ctx.append(buf[1:], buf[3 + nk.size:], dk, dv, to_dev(torch, pos), 1)
    torch.cuda.synchronize()
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    ctx.close()


# ---------------------------------------------------------------------------
# decode attention vs the oracle
# ---------------------------------------------------------------------------
DECODE_CASES = [
    # name, B, H, KVH, HD, slots, window, totals (None = seeded ragged)
    ("cfg1_qwen05b", 1, 14, 2, 64, 2048, 0, [512]),
    ("cfg2_qwen7b_ragged", 4, 28, 4, 128, 4096, 0, None),
    ("cfg3_phi3_mha", 3, 32, 32, 96, 1024, 0, None),
    ("cfg4_gemma_global", 2, 16, 8, 256, 2048, 0, None),
    ("cfg4_gemma_local_window", 2, 16, 8, 256, 2048, 1024, [2048, 1500]),
    ("group16", 2, 32, 2, 64, 700, 0, None),
    ("tiny_lengths", 6, 14, 2, 64, 256, 0, [0, 1, 2, 63, 64, 65]),
    ("window_edges", 5, 8, 4, 128, 512, 100, [1, 99, 100, 101, 512]),
]


@pytest.mark.parametrize("kernel", [GENERIC, TMA], ids=["generic", "tma"])
@pytest.mark.parametrize("case", DECODE_CASES, ids=lambda c: c[0])
def test_decode_matches_oracle(hkv, cuda, oracle, case, kernel):
    name, B, H, KVH, HD, slots, window, totals = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    if totals is None:
        totals = rng.integers(slots // 2, slots + 1, size=B)
    totals = np.asarray(totals, dtype=np.int32)
    # rows past `total` hold garbage (incl. NaN bit patterns) to prove they are never used
    q, _, _, kc, vc = make_case(int(rng.integers(1 << 30)), B, H, KVH, HD, slots, totals, fill="garbage")
    for b, t in enumerate(totals):
        kc[b, t:] = np.float16(np.nan)
        vc[b, t:] = np.float16(np.inf)
    for scale in (1.0 / math.sqrt(HD), 1.0):  # 1.0 = the reference's Gemma setting (near one-hot softmax)
        ref = oracle.decode(q, kc, vc, totals, scale, window=window, threads=8)
        for ct in (0, 1, 3):
            got, kern = run_decode(hkv, cuda, q, kc, vc, totals, scale, H=H, KVH=KVH, HD=HD,
                                   window=window, kernel=kernel, chunk_tiles=ct)
            assert kern == kernel
            assert not np.isnan(got.astype(np.float32)).any()
            assert_close(oracle, got, ref, f"{name} scale={scale:.3f} chunk_tiles={ct}")


@pytest.mark.parametrize("kernel", [GENERIC, TMA], ids=["generic", "tma"])
def test_ring_cache_equals_linear_window(hkv, cuda, oracle, kernel):
    """Ring plane of W rows (pos mod W) vs the reference semantics: linear cache + window W."""
    torch = cuda
    rng = np.random.default_rng(21)
    B, H, KVH, HD, W, ctx_len = 3, 16, 8, 256, 128, 500
    lin_k = normal_f16(rng, B, ctx_len, KVH, HD)
    lin_v = normal_f16(rng, B, ctx_len, KVH, HD)
    totals = np.array([ctx_len, 301, 77], np.int32)   # wrapped twice, wrapped, not yet full
    ring_k = np.zeros((B, W, KVH, HD), np.float16)
    ring_v = np.zeros_like(ring_k)
    for b, t in enumerate(totals):
        for p in range(t):
            ring_k[b, p % W] = lin_k[b, p]
            ring_v[b, p % W] = lin_v[b, p]
    q = normal_f16(rng, B, H, HD)
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.decode(q, lin_k, lin_v, totals, scale, window=W, threads=8)
    got, _ = run_decode(hkv, torch, q, ring_k, ring_v, totals, scale, H=H, KVH=KVH, HD=HD, window=W,
                        layout=1, kernel=kernel)
    assert_close(oracle, got, ref, "ring vs linear+window")


# ---------------------------------------------------------------------------
# fused append + decode == append, then decode
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", [GENERIC, TMA], ids=["generic", "tma"])
@pytest.mark.parametrize("shape", [
    (1, 14, 2, 64, 2048, 0, 0, [511]),                # config 1: append at cache_pos = 511
    (4, 28, 4, 128, 1024, 0, 0, [0, 63, 64, 1023]),   # tile edges, first and last row
    (3, 16, 8, 256, 128, 128, 1, [5, 128, 1000]),     # ring
    (2, 32, 32, 96, 300, 0, 0, [17, 299]),
    (3, 16, 8, 256, 320, 128, 1, [5, 319, 1000]),     # ring larger than its window: the window's tiles wrap (3, 4, 0)
    (2, 28, 4, 128, 448, 256, 1, [447, 5000]),
], ids=["cfg1", "edges", "ring", "hd96", "ring_gt_window_hd256", "ring_gt_window_hd128"])
def test_fused_append_decode(hkv, cuda, oracle, shape, kernel):
    torch = cuda
    B, H, KVH, HD, slots, window, layout, pos = shape
    pos = np.asarray(pos, np.int32)
    rng = np.random.default_rng(B + HD)
    q, nk, nv, kc, vc = make_case(int(rng.integers(1 << 30)), B, H, KVH, HD, slots, fill="garbage")
    scale = 1.0 / math.sqrt(HD)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos, layout=layout)
    ref = oracle.decode(q, ref_k, ref_v, pos + 1, scale, window=window, layout=layout, threads=8)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   window_size=window, layout=layout, kernel_select=kernel))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
    ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out,
                                to_dev(torch, pos), scale)
    assert ctx.device_status() == 0
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16)), "cache K not bit-exact"
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16)), "cache V not bit-exact"
    assert_close(oracle, out.cpu().numpy(), ref, "fused op")
    # host-buffer entry point: same result through pinned host tensors
    hq = torch.from_numpy(q).pin_memory()
    hk = torch.from_numpy(nk).pin_memory()
    hv = torch.from_numpy(nv).pin_memory()
    ho = torch.zeros(B, H, HD, dtype=torch.float16).pin_memory()
    dk2, dv2 = to_dev(torch, kc), to_dev(torch, vc)
    ctx.append_decode_attention_host(hq, hk, hv, dk2, dv2, ho, to_dev(torch, pos), scale)
    torch.cuda.synchronize()
    assert np.array_equal(ho.numpy().view(np.uint16), out.cpu().numpy().view(np.uint16))
    assert np.array_equal(dk2.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    # pipelined form: copies on the context's own streams; ten calls cycle the four staging sets more than
    # twice, each call with its own host buffers and planes, all outputs complete after one flush
    n = 10
    hos = [torch.zeros(B, H, HD, dtype=torch.float16).pin_memory() for _ in range(n)]
    planes = [(to_dev(torch, kc), to_dev(torch, vc)) for _ in range(n)]
    dpos = to_dev(torch, pos)
    torch.cuda.synchronize()
    for i in range(n):
        ctx.append_decode_attention_host_pipelined(hq, hk, hv, planes[i][0], planes[i][1], hos[i], dpos, scale)
    ctx.host_flush()
    torch.cuda.synchronize()
    for i in range(n):
        assert np.array_equal(hos[i].numpy().view(np.uint16), out.cpu().numpy().view(np.uint16)), f"pipelined call {i}"
        assert np.array_equal(planes[i][0].cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert ctx.device_status() == 0
    ctx.close()


def test_fused_decode_seeded_random_shapes(hkv, cuda, oracle):
    """Forty seeded random geometries of the fused append + decode op: group sizes 1..16, every
    TMA head_dim and two that only the generic kernel takes, linear and ring planes, windows,
    ragged positions (first row, tile edges, last row, past the plane = dropped append), forced
    split sizes, inactive sequences (position -1). Cache planes bit-exact, outputs within
    tolerance, rows beyond each position poisoned."""
    torch = cuda
    rng = np.random.default_rng(31415)
    for i in range(40):
        HD = int(rng.choice([64, 96, 128, 256, 80, 32]))
        KVH = int(rng.choice([1, 2, 4, 8]))
        G = int(rng.choice([1, 2, 4, 7, 8, 16]))
        H = KVH * G
        B = int(rng.integers(1, 7))
        ring = bool(rng.integers(0, 3) == 0)
        slots = int(rng.integers(1, 9)) * 64 if ring else int(rng.integers(1, 900))
        window = slots if ring else int(rng.choice([0, 0, int(rng.integers(1, 300))]))
        layout = 1 if ring else 0
        hi = 4 * slots if ring else slots + 2          # linear: up to two positions past the plane
        pos = rng.integers(-1, hi, size=B).astype(np.int32)
        pos[rng.integers(0, B)] = int(rng.choice([0, 63, 64, slots - 1]))
        ct = int(rng.choice([0, 0, 1, 2, 5]))
        q, nk, nv, kc, vc = make_case(int(rng.integers(1 << 30)), B, H, KVH, HD, slots, fill="garbage")
        if not ring:
            for b, p_ in enumerate(pos):   # rows at and past the append position are stale memory
                kc[b, max(int(p_), 0) + 1:] = np.float16(np.nan)
                vc[b, max(int(p_), 0) + 1:] = np.float16(np.inf)
        scale = float(rng.choice([1.0 / math.sqrt(HD), 1.0]))
        ref_k, ref_v = kc.copy(), vc.copy()
        oracle.append(nk, nv, ref_k, ref_v, pos, layout=layout)
        totals = np.where(pos >= 0, pos + 1, 0).astype(np.int32)
        ref = oracle.decode(q, ref_k, ref_v, totals, scale, window=window, layout=layout, threads=8)
        ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                       window_size=window, layout=layout, chunk_tiles=ct))
        dk, dv = to_dev(torch, kc), to_dev(torch, vc)
        out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
        ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out,
                                    to_dev(torch, pos), scale)
        what = (f"case {i}: B={B} H={H} KVH={KVH} HD={HD} slots={slots} window={window} ring={ring} "
                f"pos={pos.tolist()} chunk_tiles={ct} kernel={ctx.kernel}")
        assert ctx.device_status() == 0, what
        assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16)), what + ": K plane"
        assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16)), what + ": V plane"
        got = out.cpu().numpy()
        assert not np.isnan(got.astype(np.float32)).any(), what + ": NaN"
        assert_close(oracle, got, ref, what)
        ctx.close()


def test_strided_batch_and_engine_scalar_position(hkv, cuda, oracle):
    """batch = 1 with scalar device positions is the engine's own contract; a batch stride
    larger than one sequence's plane addresses sequences inside a bigger allocation."""
    torch = cuda
    B, H, KVH, HD, slots = 2, 28, 4, 128, 256
    pad = 64 * KVH * HD
    rng = np.random.default_rng(4)
    q, _, _, kc, vc = make_case(5, B, H, KVH, HD, slots, fill="garbage")
    totals = np.array([200, 131], np.int32)
    ref = oracle.decode(q, kc, vc, totals, 0.1, threads=4)
    stride = slots * KVH * HD + pad
    big_k = torch.zeros(B * stride, dtype=torch.float16, device="cuda")
    big_v = torch.zeros(B * stride, dtype=torch.float16, device="cuda")
    for b in range(B):
        big_k[b * stride:b * stride + slots * KVH * HD] = to_dev(torch, kc[b]).flatten()
        big_v[b * stride:b * stride + slots * KVH * HD] = to_dev(torch, vc[b]).flatten()
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   batch_stride_elems=stride))
    out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
    ctx.decode_attention(to_dev(torch, q), big_k, big_v, out, to_dev(torch, totals), 0.1)
    assert ctx.device_status() == 0
    assert_close(oracle, out.cpu().numpy(), ref, "strided batch")
    ctx.close()
    # engine contract: one sequence, scalar device total
    one = torch.zeros(1, H, HD, dtype=torch.float16, device="cuda")
    hkv.launch_attention_cached_fp16_dp(to_dev(torch, q[1:2]), to_dev(torch, kc[1:2]), to_dev(torch, vc[1:2]),
                                        one, 1, to_dev(torch, totals[1:2]), H, KVH, HD, slots, 0.1, 0)
    torch.cuda.synchronize()
    assert_close(oracle, one.cpu().numpy(), ref[1:2], "batch-1 scalar position")


def test_prefill_matches_oracle(hkv, cuda, oracle):
    torch = cuda
    rng = np.random.default_rng(8)
    for (H, KVH, HD, slots, past, S_new, window) in [(28, 4, 128, 512, 100, 64, 0), (16, 8, 256, 256, 0, 40, 32),
                                                     (32, 32, 96, 300, 250, 50, 0)]:
        k = normal_f16(rng, 1, slots, KVH, HD)
        v = normal_f16(rng, 1, slots, KVH, HD)
        q = normal_f16(rng, S_new, H, HD)
        scale = 1.0 / math.sqrt(HD)
        ref = oracle.prefill(q, k[0], v[0], past, scale, window=window, threads=8)
        out = torch.zeros(S_new, H, HD, dtype=torch.float16, device="cuda")
        hkv.launch_attention_prefill_cached_fp16(to_dev(torch, q), to_dev(torch, k), to_dev(torch, v), out,
                                                 S_new, past, H, KVH, HD, slots, scale, window)
        torch.cuda.synchronize()
        assert_close(oracle, out.cpu().numpy(), ref, f"prefill HD={HD}")


def test_synthetic_fill_matches_cpu_generator(hkv, cuda, oracle):
    torch = cuda
    n = 1 << 16
    buf = torch.zeros(n, dtype=torch.float16, device="cuda")
    hkv.fill_synthetic(buf, 0x48454B56, 12345)
    torch.cuda.synchronize()
    assert np.array_equal(buf.cpu().numpy().view(np.uint16), oracle.fill(0x48454B56, 12345, n).view(np.uint16))


def test_runtime_argument_errors(hkv, cuda):
    torch = cuda
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=4, num_kv_heads=2, head_dim=64, slots=64))
    t = torch.zeros(4 * 64 * 64, dtype=torch.float16, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(hkv.HkvError) as e:
        ctx.decode_attention(None, t, t, t, pos)
    assert e.value.status == 1
    with pytest.raises(hkv.HkvError) as e:
        ctx.decode_attention(t.data_ptr() + 1, t, t, t, pos)
    assert e.value.status == 3
    with pytest.raises(hkv.HkvError) as e:
        ctx.decode_attention(t, t, t, t, pos, scale=float("nan"))
    assert e.value.status == 1
    with pytest.raises(hkv.HkvError) as e:
        ctx.append(t, t, t, t, None)
    assert e.value.status == 1
    assert ctx.device_status() == 0  # nothing ran, nothing faulted
    ctx.close()


# ---------------------------------------------------------------------------
# position conventions of the boundary
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", [GENERIC, TMA], ids=["generic", "tma"])
def test_host_length_calls_back_to_back_without_sync(hkv, cuda, oracle, kernel):
    """Successive host-length calls (launch_attention_cached_fp16's contract: seq_len by value) with
    DIFFERENT lengths and no synchronisation between them: each must attend its own length. The
    length travels as a kernel argument, so nothing the second call does can reach the first."""
    torch = cuda
    B, H, KVH, HD, slots = 2, 28, 4, 128, 1024
    lens = [1000, 37, 512, 1, 801, 64]
    q, _, _, kc, vc = make_case(321, B, H, KVH, HD, slots, fill="garbage")
    scale = 1.0 / math.sqrt(HD)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   kernel_select=kernel))
    dq, dk, dv = to_dev(torch, q), to_dev(torch, kc), to_dev(torch, vc)
    outs = [torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda") for _ in lens]
    torch.cuda.synchronize()
    for n, out in zip(lens, outs):          # enqueued back to back on one stream
        ctx.decode_attention_len(dq, dk, dv, out, n, scale)
    assert ctx.device_status() == 0
    for n, out in zip(lens, outs):
        ref = oracle.decode(q, kc, vc, np.full(B, n, np.int32), scale, threads=8)
        assert_close(oracle, out.cpu().numpy(), ref, f"host length {n}")
    ctx.close()


@pytest.mark.parametrize("kernel", [GENERIC, TMA], ids=["generic", "tma"])
def test_scalar_position_is_shared_by_the_whole_batch(hkv, cuda, oracle, kernel):
    """The reference's kernels read ONE device int32 for every sequence of the batch
    (kernels/attention.cu:351, :1129). FLAG_SCALAR_POSITION keeps that convention: a 4-byte
    position buffer serves batch 3 in the append, the attention and the fused op."""
    torch = cuda
    B, H, KVH, HD, slots, pos = 3, 8, 2, 64, 256, 130
    q, nk, nv, kc, vc = make_case(77, B, H, KVH, HD, slots, np.full(B, pos, np.int32))
    scale = 1.0 / math.sqrt(HD)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, np.full(B, pos, np.int32))
    ref = oracle.decode(q, ref_k, ref_v, np.full(B, pos + 1, np.int32), scale)
    d_pos = to_dev(torch, np.array([pos], np.int32))            # ONE int32 on the device
    d_tot = to_dev(torch, np.array([pos + 1], np.int32))
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   kernel_select=kernel, flags=hkv.FLAG_SCALAR_POSITION))
    # separate ops
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.append(to_dev(torch, nk), to_dev(torch, nv), dk, dv, d_pos, 1)
    ctx.decode_attention(to_dev(torch, q), dk, dv, out, d_tot, scale)
    assert ctx.device_status() == 0
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    assert_close(oracle, out.cpu().numpy(), ref, "scalar position, separate ops")
    # fused op
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out, d_pos, scale)
    assert ctx.device_status() == 0
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert_close(oracle, out.cpu().numpy(), ref, "scalar position, fused op")
    ctx.close()
    # the reference-named launchers use this convention too
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    hkv.launch_kv_cache_update_dp(to_dev(torch, nk), to_dev(torch, nv), dk, dv, B, 1, KVH, HD, slots, d_pos)
    hkv.launch_attention_cached_fp16_dp(to_dev(torch, q), dk, dv, out, B, d_tot, H, KVH, HD, slots, scale, 0)
    torch.cuda.synchronize()
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert_close(oracle, out.cpu().numpy(), ref, "scalar position, reference-named launchers")


def test_append_only_context_allocates_no_attention_workspace(hkv, cuda, oracle):
    """An append-only context (what the KV_CACHE_UPDATE and QK_NORM_ROPE ops create) appends like any
    other but refuses attention with HKV_ERR_WORKSPACE instead of touching a workspace it never made."""
    torch = cuda
    B, KVH, HD, slots = 2, 4, 128, 4096
    geo = hkv.Geometry(batch=B, num_heads=KVH, num_kv_heads=KVH, head_dim=HD, slots=slots, max_seq_new=512,
                       flags=hkv.FLAG_APPEND_ONLY)
    free0, _ = torch.cuda.mem_get_info()
    ctx = hkv.Context(geo)
    free1, _ = torch.cuda.mem_get_info()
    assert free0 - free1 <= (2 << 20), "an append-only context must not allocate attention workspaces"
    rng = np.random.default_rng(5)
    nk, nv = normal_f16(rng, B, 1, KVH, HD), normal_f16(rng, B, 1, KVH, HD)
    kc, vc = normal_f16(rng, B, slots, KVH, HD), normal_f16(rng, B, slots, KVH, HD)
    pos = np.array([17, 4095], np.int32)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos)
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    ctx.append(to_dev(torch, nk), to_dev(torch, nv), dk, dv, to_dev(torch, pos), 1)
    torch.cuda.synchronize()
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    out = torch.zeros(B, KVH, HD, dtype=torch.float16, device="cuda")
    with pytest.raises(hkv.HkvError) as e:
        ctx.decode_attention(out, dk, dv, out, to_dev(torch, pos), 1.0)
    assert e.value.status == 6   # HKV_ERR_WORKSPACE
    ctx.close()


def test_prefill_refuses_a_batched_context(hkv, cuda):
    """The prefill op has no batch dimension (kernels/attention.cu:709): a context of batch > 1 is
    refused instead of silently processing sequence 0 only."""
    torch = cuda
    ctx = hkv.Context(hkv.Geometry(batch=2, num_heads=4, num_kv_heads=4, head_dim=64, slots=128))
    t = torch.zeros(2 * 128 * 4 * 64, dtype=torch.float16, device="cuda")
    with pytest.raises(hkv.HkvError) as e:
        ctx.prefill_attention(t, t, t, t, 4, 0, 1.0)
    assert e.value.status == 2   # HKV_ERR_GEOMETRY
    ctx.close()


@pytest.mark.parametrize("groups", [1, 2, 3], ids=["two_ctas_per_sm", "one_cta_two_groups", "one_cta_one_group"])
@pytest.mark.parametrize("shape", [
    # B, H, KVH, HD, slots, window, layout
    (5, 28, 4, 128, 4096, 0, 0),     # config 2 shape, ragged lengths
    (3, 14, 2, 64, 2048, 0, 0),      # config 1 shape
    (4, 32, 32, 96, 1024, 0, 0),     # config 3 shape (MHA, head_dim 96)
    (3, 16, 8, 256, 1024, 1024, 1),  # config 4 local layer: ring (256-wide tiles need the whole SM: falls back)
    (70, 8, 2, 128, 640, 200, 0),    # more sequences than a warp scans at once, sliding window
], ids=lambda s: "B%d_H%d_KVH%d_HD%d_%d_w%d_l%d" % s)
def test_both_shapes_of_the_tma_decode_kernel(hkv, cuda, oracle, shape, groups):
    """The TMA decode kernel runs as two CTAs per SM with one consumer group each, or as one CTA per SM
    with two groups or with one (chosen by the host; forced here through tune_tma_groups). All give
    the oracle's result for the fused append + attention, with ragged and empty sequences."""
    torch = cuda
    B, H, KVH, HD, slots, window, layout = shape
    rng = np.random.default_rng(B * 131 + HD + groups)
    hi = 3 * slots if layout == 1 else slots
    pos = rng.integers(0, hi, size=B).astype(np.int32)
    pos[0] = hi - 1
    if B > 2:
        pos[1], pos[2] = 0, -1            # first token of a sequence; a free batch slot
    q, nk, nv, _, _ = make_case(int(rng.integers(1 << 30)), B, H, KVH, HD, 1)
    lin = int(pos.max()) + 1               # linear reference planes hold every position
    kc, vc = normal_f16(rng, B, lin, KVH, HD), normal_f16(rng, B, lin, KVH, HD)
    ref_k, ref_v = kc.copy(), vc.copy()
    live = pos >= 0
    for b in np.nonzero(live)[0]:          # the reference's append: the new row at its position
        ref_k[b, pos[b]], ref_v[b, pos[b]] = nk[b, 0], nv[b, 0]
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.decode(q, ref_k, ref_v, np.maximum(pos + 1, 0), scale, window=window, threads=8)
    # device planes: the rows below each position (ring: the last `slots` of them), garbage elsewhere
    dk_h = np.full((B, slots, KVH, HD), np.nan, np.float16)
    dv_h = np.full((B, slots, KVH, HD), np.inf, np.float16)
    for b in range(B):
        for p in range(max(0, int(pos[b]) - slots) if layout == 1 else 0, max(int(pos[b]), 0)):
            r = p % slots if layout == 1 else p
            dk_h[b, r], dv_h[b, r] = kc[b, p], vc[b, p]
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, window_size=window,
                                   layout=layout, kernel_select=TMA, tune_tma_groups=groups))
    dk, dv = to_dev(torch, dk_h), to_dev(torch, dv_h)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    for _ in range(2):      # the second call re-appends the same rows: same result
        ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out,
                                    to_dev(torch, pos), scale)
    assert ctx.device_status() == 0
    got = out.cpu().numpy()
    assert_close(oracle, got, ref, f"fused decode, groups={groups}")
    assert not got[~live].any(), "a free slot gives a zero row"
    for b in np.nonzero(live)[0]:
        r = int(pos[b]) % slots if layout == 1 else int(pos[b])
        assert np.array_equal(dk[b, r].cpu().numpy().view(np.uint16), nk[b, 0].view(np.uint16))
        assert np.array_equal(dv[b, r].cpu().numpy().view(np.uint16), nv[b, 0].view(np.uint16))
    ctx.close()


@pytest.mark.parametrize("totals", [
    [1], [64], [65], [0, 1, 0], [1, 64, 65, 0, 128, 129], [4096, 1, 4095, 0, 2049],
    list(range(0, 70)),                      # 70 sequences of 0..69 rows: fewer tiles than spans
    [4096] * 3 + [0] * 30 + [17] * 4,        # a few long sequences among many empty ones
], ids=lambda t: f"{len(t)}seq_max{max(t)}")
def test_equal_span_schedule_edges(hkv, cuda, oracle, totals):
    """The TMA decode kernel cuts the line of all 64-row tiles of a launch into equal spans, one per
    gang of CTAs, with the lengths read on the device: launches with fewer tiles than spans, empty
    sequences, sequences that end exactly on a tile or span boundary, and one sequence that takes every
    span must all give the oracle's result (decode and fused append + decode)."""
    torch = cuda
    B, H, KVH, HD, slots = len(totals), 28, 4, 128, 4096
    totals = np.asarray(totals, np.int32)
    q, nk, nv, kc, vc = make_case(B * 7 + int(totals.sum()), B, H, KVH, HD, slots, fill="garbage")
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.decode(q, kc, vc, totals, scale, threads=8)
    for groups in (1, 2):
        got, kern = run_decode(hkv, torch, q, kc, vc, totals, scale, H=H, KVH=KVH, HD=HD, kernel=TMA)
        assert kern == TMA
        assert_close(oracle, got, ref, f"decode, totals={totals.tolist()[:8]}")
    # fused: append at position total (sequences with total == slots are full: the reference drops the row)
    pos = np.minimum(totals, slots - 1).astype(np.int32)
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos)
    ref2 = oracle.decode(q, ref_k, ref_v, pos + 1, scale, threads=8)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, kernel_select=TMA))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
    ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out, to_dev(torch, pos), scale)
    assert ctx.device_status() == 0
    assert_close(oracle, out.cpu().numpy(), ref2, "fused append + decode")
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), ref_k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ref_v.view(np.uint16))
    ctx.close()


@pytest.mark.parametrize("kernel", [1, 2], ids=["generic", "tma"])
def test_decode_reads_q_k_v_out_of_a_fused_qkv_activation(hkv, cuda, oracle, kernel):
    """The zero-copy QKV split (reference kernels/register_kernels.cpp:587-593, batch 1 only there):
    q, k_new and v_new are views into one [batch][q | k | v] activation, described to the context by
    the two sequence strides. Results must equal the dense call bit for bit — outputs and planes."""
    torch = cuda
    B, H, KVH, HD, slots = 3, 28, 4, 128, 512
    pos = np.array([5, 300, 511], np.int32)
    q, nk, nv, kc, vc = make_case(77, B, H, KVH, HD, slots, fill="garbage")
    scale = 1.0 / math.sqrt(HD)
    row = (H + 2 * KVH) * HD
    fused = torch.zeros(B, row, dtype=torch.float16, device="cuda")
    fused[:, :H * HD] = to_dev(torch, q).reshape(B, -1)
    fused[:, H * HD:(H + KVH) * HD] = to_dev(torch, nk).reshape(B, -1)
    fused[:, (H + KVH) * HD:] = to_dev(torch, nv).reshape(B, -1)
    qp = fused.data_ptr()
    kp, vp = qp + H * HD * 2, qp + (H + KVH) * HD * 2
    geo = dict(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, kernel_select=kernel)
    dense = hkv.Context(hkv.Geometry(**geo))
    strided = hkv.Context(hkv.Geometry(**geo, q_seq_stride_elems=row, new_kv_seq_stride_elems=row))
    dpos = to_dev(torch, pos)
    outs, planes = [], []
    for ctx, args in ((dense, (to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv))), (strided, (qp, kp, vp))):
        dk, dv = to_dev(torch, kc), to_dev(torch, vc)
        out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
        ctx.append_decode_attention(args[0], args[1], args[2], dk, dv, out, dpos, scale)
        assert ctx.device_status() == 0
        # the two-call form through the same views
        dk2, dv2 = to_dev(torch, kc), to_dev(torch, vc)
        out2 = torch.zeros_like(out)
        ctx.append(args[1], args[2], dk2, dv2, dpos, seq_new=1)
        ctx.decode_attention(args[0], dk2, dv2, out2, to_dev(torch, pos + 1), scale)
        torch.cuda.synchronize()
        assert np.array_equal(dk2.cpu().numpy().view(np.uint16), dk.cpu().numpy().view(np.uint16))
        outs.append((out.cpu().numpy(), out2.cpu().numpy()))
        planes.append((dk.cpu().numpy(), dv.cpu().numpy()))
    for i in range(2):
        assert np.array_equal(outs[0][i].view(np.uint16), outs[1][i].view(np.uint16)), "outputs differ from the dense call"
        assert np.array_equal(planes[0][i].view(np.uint16), planes[1][i].view(np.uint16)), "planes differ from the dense call"
    ref_k, ref_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, ref_k, ref_v, pos)
    assert np.array_equal(planes[1][0].view(np.uint16), ref_k.view(np.uint16))
    assert_close(oracle, outs[1][0], oracle.decode(q, ref_k, ref_v, pos + 1, scale, threads=8), "fused QKV views")
    # several new tokens per sequence are not described by the one-token strides
    with pytest.raises(hkv.HkvError):
        strided.append(kp, vp, to_dev(torch, kc), to_dev(torch, vc), dpos, seq_new=2)
    # a stride smaller than a sequence's row is refused when the context is created
    with pytest.raises(hkv.HkvError):
        hkv.Context(hkv.Geometry(**geo, q_seq_stride_elems=H * HD - 8))
    dense.close()
    strided.close()
