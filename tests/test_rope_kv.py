"""The step in front of the append: per-head RMSNorm(q, k) + RoPE with the rotated K and the V
row written straight into the cache (reference kernels/attention.cu:800-973). CPU: oracle
properties and golden vectors from the reference's own kernel; GPU: libhkv vs oracle and vs the
reference's golden vectors. q/K tolerance as for attention outputs; the V copy is bit-exact."""
import os
import sys
import zlib

import numpy as np
import pytest

from _util import assert_close, normal_f16, to_dev

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_golden as gen  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "ref_golden.npz"))
HAVE_ROPE_GOLD = (gen.ROPE_CASES[0][0] + "/q") in GOLD.files


def test_oracle_rope_properties(oracle):
    rng = np.random.default_rng(1)
    B, S, H, KVH, HD = 2, 3, 4, 2, 64
    q, k, v = normal_f16(rng, B, S, H, HD), normal_f16(rng, B, S, KVH, HD), normal_f16(rng, B, S, KVH, HD)
    ones = np.ones(HD, np.float16)
    q0, k0 = q.copy(), k.copy()
    oracle.qk_norm_rope(q, k, v, ones, ones, [0, 5])
    # unit RMS per head (rotation preserves the norm)
    assert np.allclose(np.sqrt((q.astype(np.float32) ** 2).mean(-1)), 1.0, atol=2e-3)
    # position 0: no rotation, plain RMSNorm
    x = q0[0, 0, 1].astype(np.float32)
    assert np.allclose(q[0, 0, 1].astype(np.float32), x / np.sqrt((x * x).mean() + 1e-6), atol=1e-3)
    # partial rotary: dims >= rotary_dim are only normalised
    q2, k2 = q0.copy(), k0.copy()
    oracle.qk_norm_rope(q2, k2, v, ones, ones, [7, 9], rotary_dim=32)
    x = q0[1, 2, 3].astype(np.float32)
    assert np.allclose(q2[1, 2, 3, 32:].astype(np.float32), (x / np.sqrt((x * x).mean() + 1e-6))[32:], atol=1e-3)
    # cache write: K rows land at pos + s, V is copied bit-exact, k itself untouched, rows past the plane dropped
    slots = 8
    kc = np.zeros((B, slots, KVH, HD), np.float16)
    vc = np.zeros_like(kc)
    q3, k3 = q0.copy(), k0.copy()
    oracle.qk_norm_rope(q3, k3, v, ones, ones, [1, 6], k_cache=kc, v_cache=vc)
    assert np.array_equal(k3, k0)
    assert np.array_equal(vc[0, 1:4], v[0]) and np.array_equal(vc[1, 6:8], v[1, :2])
    k4 = k0.copy()
    oracle.qk_norm_rope(q0.copy(), k4, None, ones, ones, [1, 6])
    assert np.array_equal(kc[0, 1:4].view(np.uint16), k4[0].view(np.uint16))
    assert not kc[0, 4:].any() and not kc[1, :6].any()


@pytest.mark.skipif(not HAVE_ROPE_GOLD, reason="golden file predates the rope cases")
@pytest.mark.parametrize("case", gen.ROPE_CASES, ids=lambda c: c[0])
def test_oracle_matches_reference_rope_kernel(oracle, case):
    name, S, H, KVH, HD, rot, slots, position, theta, scaling = case
    q, k, v, qw, kw, kc, vc = gen.rope_inputs(name, S, H, KVH, HD, slots)
    k_before = k.copy()
    oracle.qk_norm_rope(q, k, v, qw, kw, [position], k_cache=kc, v_cache=vc, rotary_dim=rot, theta=theta,
                        scaling=scaling)
    assert int(GOLD[name + "/k_untouched"][0]) == 1 and np.array_equal(k, k_before)
    assert zlib.crc32(vc.tobytes()) == int(GOLD[name + "/v_crc"][0])          # V copy: bit-exact
    assert_close(oracle, GOLD[name + "/q"].view(np.float16), q, name + " q")
    assert_close(oracle, GOLD[name + "/k_cache"].view(np.float16), kc, name + " k_cache")
    k2 = k_before.copy()
    oracle.qk_norm_rope(q.copy(), k2, None, qw, kw, [position], rotary_dim=rot, theta=theta, scaling=scaling)
    assert_close(oracle, GOLD[name + "/k_inplace"].view(np.float16), k2, name + " k in place")


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [0, 1], ids=["linear", "ring"])
def test_rope_kv_matches_oracle_batched(hkv, cuda, oracle, layout):
    torch = cuda
    rng = np.random.default_rng(5 + layout)
    B, S, H, KVH, HD, slots = 3, 4, 28, 4, 128, 64
    q, k, v = normal_f16(rng, B, S, H, HD), normal_f16(rng, B, S, KVH, HD), normal_f16(rng, B, S, KVH, HD)
    qw = (1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)).astype(np.float16)
    kw = (1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)).astype(np.float16)
    kc, vc = normal_f16(rng, B, slots, KVH, HD), normal_f16(rng, B, slots, KVH, HD)
    pos = np.array([0, 61, 200 if layout else 30], np.int32)   # seq 1 runs off a linear plane / wraps a ring
    rq, rk, rkc, rvc = q.copy(), k.copy(), kc.copy(), vc.copy()
    oracle.qk_norm_rope(rq, rk, v, qw, kw, pos, k_cache=rkc, v_cache=rvc, layout=layout, theta=1e6)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, layout=layout,
                                   window_size=slots if layout else 0))
    dq, dk, dkc, dvc = to_dev(torch, q), to_dev(torch, k), to_dev(torch, kc), to_dev(torch, vc)
    ctx.qk_norm_rope_kv(dq, dk, to_dev(torch, v), to_dev(torch, qw), to_dev(torch, kw), dkc, dvc, to_dev(torch, pos),
                        seq_new=S, theta=1e6)
    torch.cuda.synchronize()
    assert np.array_equal(dvc.cpu().numpy().view(np.uint16), rvc.view(np.uint16)), "V rows must be bit-exact"
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), k.view(np.uint16)), "k must stay untouched"
    assert_close(oracle, dq.cpu().numpy(), rq, "q")
    assert_close(oracle, dkc.cpu().numpy(), rkc, "k_cache")
    # no-cache form, host position
    rq2, rk2 = q.copy(), k.copy()
    oracle.qk_norm_rope(rq2, rk2, None, qw, kw, [9, 9, 9], rotary_dim=64)
    dq2, dk2 = to_dev(torch, q), to_dev(torch, k)
    ctx.qk_norm_rope_kv(dq2, dk2, None, to_dev(torch, qw), to_dev(torch, kw), position=9, seq_new=S, rotary_dim=64)
    torch.cuda.synchronize()
    assert_close(oracle, dq2.cpu().numpy(), rq2, "q (no cache)")
    assert_close(oracle, dk2.cpu().numpy(), rk2, "k in place")
    ctx.close()


@pytest.mark.gpu
@pytest.mark.skipif(not HAVE_ROPE_GOLD, reason="golden file predates the rope cases")
@pytest.mark.parametrize("case", gen.ROPE_CASES, ids=lambda c: c[0])
def test_rope_kv_reproduces_reference_kernel(hkv, cuda, oracle, case):
    torch = cuda
    name, S, H, KVH, HD, rot, slots, position, theta, scaling = case
    q, k, v, qw, kw, kc, vc = gen.rope_inputs(name, S, H, KVH, HD, slots)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots))
    dq, dkc, dvc = to_dev(torch, q), to_dev(torch, kc), to_dev(torch, vc)
    ctx.qk_norm_rope_kv(dq, to_dev(torch, k), to_dev(torch, v), to_dev(torch, qw), to_dev(torch, kw), dkc, dvc,
                        to_dev(torch, np.array([position], np.int32)), seq_new=S, rotary_dim=rot, theta=theta,
                        scaling_factor=scaling)
    torch.cuda.synchronize()
    assert zlib.crc32(dvc.cpu().numpy().tobytes()) == int(GOLD[name + "/v_crc"][0])
    assert_close(oracle, dq.cpu().numpy(), GOLD[name + "/q"].view(np.float16), name + " q vs reference")
    assert_close(oracle, dkc.cpu().numpy(), GOLD[name + "/k_cache"].view(np.float16), name + " k_cache vs reference")
    ctx.close()


ROPE_SHAPES = [
    # name, B, S, H, KVH, HD, rotary_dim, slots, layout
    ("phi3_chunk_ranges_of_tokens", 1, 700, 6, 2, 96, 96, 1024, 0),       # 12 pieces on 16 lanes; CTAs own token ranges
    ("gemma_hd256_ring", 2, 200, 4, 2, 256, 256, 256, 1),                 # one head per warp; chunk wraps the ring
    ("hd64_four_heads_per_warp", 3, 130, 14, 2, 64, 64, 256, 0),           # the last sequences run off the plane
    ("hd128_partial_rotary_odd_units", 2, 2, 9, 3, 128, 64, 512, 0),      # 15 units: a half-empty warp slot
    ("element_path_hd72_rot36", 1, 5, 3, 1, 72, 36, 256, 0),              # rotary_dim/2 not in 8-element pieces
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", ROPE_SHAPES, ids=lambda c: c[0])
def test_rope_kv_shapes(hkv, cuda, oracle, case):
    torch = cuda
    name, B, S, H, KVH, HD, rot, slots, layout = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    q, k, v = normal_f16(rng, B, S, H, HD), normal_f16(rng, B, S, KVH, HD), normal_f16(rng, B, S, KVH, HD)
    qw = (1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)).astype(np.float16)
    kw = (1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)).astype(np.float16)
    kc, vc = normal_f16(rng, B, slots, KVH, HD), normal_f16(rng, B, slots, KVH, HD)
    pos = (np.arange(B, dtype=np.int32) * 37 + 211).astype(np.int32)
    rq, rk, rkc, rvc = q.copy(), k.copy(), kc.copy(), vc.copy()
    oracle.qk_norm_rope(rq, rk, v, qw, kw, pos, k_cache=rkc, v_cache=rvc, layout=layout, rotary_dim=rot, theta=1e4)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, layout=layout,
                                   window_size=slots if layout else 0, flags=hkv.FLAG_APPEND_ONLY))
    dq, dk, dkc, dvc = to_dev(torch, q), to_dev(torch, k), to_dev(torch, kc), to_dev(torch, vc)
    ctx.qk_norm_rope_kv(dq, dk, to_dev(torch, v), to_dev(torch, qw), to_dev(torch, kw), dkc, dvc, to_dev(torch, pos),
                        seq_new=S, rotary_dim=rot, theta=1e4)
    torch.cuda.synchronize()
    assert np.array_equal(dvc.cpu().numpy().view(np.uint16), rvc.view(np.uint16)), "V rows must be bit-exact"
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), k.view(np.uint16)), "k must stay untouched"
    assert_close(oracle, dq.cpu().numpy(), rq, name + " q")
    assert_close(oracle, dkc.cpu().numpy(), rkc, name + " k_cache")
    # the in-place form on the same shapes
    rq2, rk2 = q.copy(), k.copy()
    oracle.qk_norm_rope(rq2, rk2, None, qw, kw, pos, rotary_dim=rot, theta=1e4)
    dq2, dk2 = to_dev(torch, q), to_dev(torch, k)
    ctx.qk_norm_rope_kv(dq2, dk2, None, to_dev(torch, qw), to_dev(torch, kw), None, None, to_dev(torch, pos),
                        seq_new=S, rotary_dim=rot, theta=1e4)
    torch.cuda.synchronize()
    assert_close(oracle, dq2.cpu().numpy(), rq2, name + " q (in place)")
    assert_close(oracle, dk2.cpu().numpy(), rk2, name + " k (in place)")
    ctx.close()
