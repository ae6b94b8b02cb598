"""Golden vectors produced by the REFERENCE's own kernels (kernels/attention.cu of the
reference, unmodified, rebuilt for sm_100a and run on a B200 by
tests/golden/make_reference_golden.py). CPU suite: they pin the oracle. GPU suite: libhkv
reproduces them."""
import math
import os
import sys
import zlib

import numpy as np
import pytest

from _util import assert_close, to_dev

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_reference_golden as gen  # noqa: E402  (only its case tables and input recipe)

GOLD = np.load(os.path.join(HERE, "golden", "ref_golden.npz"))


def _scale(scale, HD):
    return 1.0 / math.sqrt(HD) if scale == "default" else float(scale)


@pytest.mark.parametrize("case", gen.CASES, ids=lambda c: c[0])
def test_oracle_matches_reference_kernels(oracle, case):
    name, B, H, KVH, HD, slots, window, scale, totals = case
    q, nk, nv, kc, vc = gen.case_inputs(name, B, H, KVH, HD, slots)
    pos = np.asarray(totals, np.int32) - 1
    oracle.append(nk, nv, kc, vc, pos)
    # append: bit-exact against what the reference's kv_cache_update left in its planes
    assert zlib.crc32(kc.tobytes()) == int(GOLD[name + "/k_crc"][0])
    assert zlib.crc32(vc.tobytes()) == int(GOLD[name + "/v_crc"][0])
    ref_out = GOLD[name + "/out"].view(np.float16)
    for mode in (0, 1):
        mine = oracle.decode(q, kc, vc, totals, _scale(scale, HD), window=window, mode=mode)
        assert_close(oracle, ref_out, mine, f"{name} oracle mode {mode} vs reference kernel")
    # the reference's host-length and device-position variants agree with each other
    assert_close(oracle, GOLD[name + "/out_hostlen"].view(np.float16), ref_out, "host-length variant")


@pytest.mark.parametrize("case", gen.PREFILL_CASES, ids=lambda c: c[0])
def test_oracle_prefill_matches_reference_kernel(oracle, case):
    name, H, KVH, HD, slots, past, S_new, window = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    f16 = lambda *s: rng.standard_normal(s, dtype=np.float32).astype(np.float16)
    k, v, q = f16(slots, KVH, HD), f16(slots, KVH, HD), f16(S_new, H, HD)
    mine = oracle.prefill(q, k, v, past, 1.0 / math.sqrt(HD), window=window)
    assert_close(oracle, GOLD[name + "/out"].view(np.float16), mine, name)


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [1, 2], ids=["generic", "tma"])
@pytest.mark.parametrize("case", gen.CASES, ids=lambda c: c[0])
def test_libhkv_reproduces_reference_kernels(hkv, cuda, oracle, case, kernel):
    torch = cuda
    name, B, H, KVH, HD, slots, window, scale, totals = case
    q, nk, nv, kc, vc = gen.case_inputs(name, B, H, KVH, HD, slots)
    pos = np.asarray(totals, np.int32) - 1
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   window_size=window, kernel_select=kernel))
    dk, dv = to_dev(torch, kc), to_dev(torch, vc)
    out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
    ctx.append_decode_attention(to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), dk, dv, out,
                                to_dev(torch, pos), _scale(scale, HD))
    assert ctx.device_status() == 0
    assert zlib.crc32(dk.cpu().numpy().tobytes()) == int(GOLD[name + "/k_crc"][0])
    assert zlib.crc32(dv.cpu().numpy().tobytes()) == int(GOLD[name + "/v_crc"][0])
    assert_close(oracle, out.cpu().numpy(), GOLD[name + "/out"].view(np.float16), f"{name} vs reference kernel")
    ctx.close()
