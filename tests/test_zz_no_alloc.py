"""GPU test of hkv_decode_attention_static, the decode-attention entry point for callers that
cannot allocate device memory when they need attention (fixed memory plans, sandboxes that
forbid allocation after start-up, serving threads that cannot take an allocation's
synchronisation). Its split-K partials live in a fixed 8 MiB array inside the library, shared
by every call, so the test makes two calls in a row with different inputs and checks each
against the context-based entry point: stale partials from the first call must not leak into
the second. This file is collected last on purpose."""
import math

import numpy as np
import pytest

from _util import assert_close, make_case, to_dev

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_context_decode_twice(hkv, cuda, oracle):
    torch = cuda
    B, H, KVH, HD, slots = 3, 28, 4, 128, 2048
    geo = hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots)
    ctx = hkv.Context(geo)
    scale = 1.0 / math.sqrt(HD)
    # second call: shorter sequences and other data, so it uses FEWER partial rows than the first
    for call, totals in enumerate(([2048, 1500, 1033], [700, 64, 1])):
        totals = np.asarray(totals, np.int32)
        q, _, _, kc, vc = make_case(100 + call, B, H, KVH, HD, slots, totals, fill="garbage")
        dq, dk, dv, dt = to_dev(torch, q), to_dev(torch, kc), to_dev(torch, vc), to_dev(torch, totals)
        want = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
        ctx.decode_attention(dq, dk, dv, want, dt, scale)
        got = torch.full((B, H, HD), float("nan"), dtype=torch.float16, device="cuda")
        # Free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counters
        # it sees a cudaMalloc made inside the library. The first call's one-time set-up (module
        # load, symbol lookup) is allowed to move it; the second call must not.
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        hkv.decode_attention_static(geo, dq, dk, dv, got, dt, scale)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:
            assert free_after == free_before, "hkv_decode_attention_static changed the device's free memory"
        assert_close(oracle, got.cpu().numpy(), want.cpu().numpy(), f"static vs context, call {call}")
        ref = oracle.decode(q, kc, vc, totals, scale, threads=8)
        assert_close(oracle, got.cpu().numpy(), ref, f"static vs oracle, call {call}")
    assert ctx.device_status() == 0
    ctx.close()


def test_static_scratch_rejects_oversized_geometry(hkv, cuda):
    torch = cuda
    # one partial per (sequence, head) already needs 64*64*514*4 B = 8.03 MiB > 8 MiB
    geo = hkv.Geometry(batch=64, num_heads=64, num_kv_heads=64, head_dim=512, slots=64)
    assert geo.batch * geo.num_heads * (geo.head_dim + 2) * 4 > hkv.ops.STATIC_SCRATCH_BYTES
    t = torch.zeros(16, dtype=torch.float16, device="cuda")
    pos = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(hkv.HkvError) as e:
        hkv.decode_attention_static(geo, t, t, t, t, pos)  # refused before any launch
    assert e.value.status == 7  # HKV_ERR_TOO_LARGE
    torch.cuda.synchronize()
