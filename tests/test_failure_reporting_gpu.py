"""Failure detection without a GPU fault: a device-side wait that nothing satisfies must run
out after its limit, report through the status word, and leave the context usable. (Host-side
failures — bad arguments, missing device — are covered in test_capi_cpu.py and
test_parity_gpu.py::test_runtime_argument_errors.)"""
import math
import time

import numpy as np
import pytest

from _util import assert_close, make_case, to_dev

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_context_survives(hkv, cuda, oracle):
    torch = cuda
    B, H, KVH, HD, slots = 2, 28, 4, 128, 512
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots))
    assert ctx.device_status() == 0
    t0 = time.perf_counter()
    ctx.selftest_bounded_wait(limit_ms=100)
    status = ctx.device_status()          # synchronises: returns once the wait has given up
    elapsed = time.perf_counter() - t0
    assert status == 1, "the expired wait must set bit 1 of the status word"
    assert 0.05 < elapsed < 5.0, f"wait should give up after ~0.1 s, took {elapsed:.2f} s"
    assert ctx.device_status() == 0, "reading the status clears it"
    # the context and the device are fine afterwards: a normal decode still matches the oracle
    totals = np.array([512, 300], np.int32)
    q, _, _, kc, vc = make_case(3, B, H, KVH, HD, slots, totals, fill="garbage")
    out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
    scale = 1.0 / math.sqrt(HD)
    ctx.decode_attention(to_dev(torch, q), to_dev(torch, kc), to_dev(torch, vc), out, to_dev(torch, totals), scale)
    assert ctx.device_status() == 0
    assert_close(oracle, out.cpu().numpy(), oracle.decode(q, kc, vc, totals, scale, threads=4), "decode after self-test")
    with pytest.raises(hkv.HkvError):
        ctx.selftest_bounded_wait(limit_ms=0)      # limits outside 1..1000 ms are refused on the host
    ctx.close()
