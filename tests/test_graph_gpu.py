"""CUDA-graph single-capture contract through the C ABI from Python: a whole multi-layer
decode step (fused append + attention per layer) is captured ONCE; it is then replayed while
only the device position array (and the contents of q / k_new / v_new at fixed addresses)
change. Every replayed step is compared with the oracle, and the cache planes must end up
bit-identical to the oracle's mirror."""
import math

import numpy as np
import pytest

from _util import assert_close, normal_f16, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(3, 28, 4, 128, 512), (2, 16, 8, 256, 256)], ids=["qwen7b", "gemma"])
def test_capture_once_replay_many(hkv, cuda, oracle, shape):
    torch = cuda
    B, H, KVH, HD, slots = shape
    L, steps = 3, 12
    rng = np.random.default_rng(B * HD)
    scale = 1.0 / math.sqrt(HD)
    pos = rng.integers(40, slots - steps - 1, size=B).astype(np.int32)
    hk = [normal_f16(rng, B, slots, KVH, HD) for _ in range(L)]
    hv = [normal_f16(rng, B, slots, KVH, HD) for _ in range(L)]
    dk = [to_dev(torch, a) for a in hk]
    dv = [to_dev(torch, a) for a in hv]
    dq = torch.zeros(L, B, H, HD, dtype=torch.float16, device="cuda")
    dkn = torch.zeros(L, B, 1, KVH, HD, dtype=torch.float16, device="cuda")
    dvn = torch.zeros(L, B, 1, KVH, HD, dtype=torch.float16, device="cuda")
    out = torch.zeros(L, B, H, HD, dtype=torch.float16, device="cuda")
    dpos = to_dev(torch, pos)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots))

    def enqueue():
        for l in range(L):
            ctx.append_decode_attention(dq[l], dkn[l], dvn[l], dk[l], dv[l], out[l], dpos, scale)

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for s in range(steps):
        q = normal_f16(rng, L, B, H, HD)
        kn = normal_f16(rng, L, B, 1, KVH, HD)
        vn = normal_f16(rng, L, B, 1, KVH, HD)
        with torch.cuda.stream(side):
            dq.copy_(to_dev(torch, q)); dkn.copy_(to_dev(torch, kn)); dvn.copy_(to_dev(torch, vn))
            dpos.copy_(to_dev(torch, pos))
            if s == 0:
                # global-mode capture: a cudaMalloc or a synchronisation inside the library
                # would invalidate the capture and raise here
                with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
                    enqueue()
            graph.replay()
        side.synchronize()
        got = out.cpu().numpy()
        for l in range(L):
            oracle.append(kn[l], vn[l], hk[l], hv[l], pos)
            ref = oracle.decode(q[l], hk[l], hv[l], pos + 1, scale, threads=8)
            assert_close(oracle, got[l], ref, f"step {s} layer {l}")
        pos = pos + 1
    for l in range(L):
        assert np.array_equal(dk[l].cpu().numpy().view(np.uint16), hk[l].view(np.uint16))
        assert np.array_equal(dv[l].cpu().numpy().view(np.uint16), hv[l].view(np.uint16))
    assert ctx.device_status() == 0
    ctx.close()


@pytest.mark.parametrize("splits", [0, 3], ids=["auto", "3"])
def test_prefill_chunk_captured_and_replayed(hkv, cuda, oracle, splits):
    """A prefill chunk (append of its rows + the tensor-core attention, incl. the reset of the
    kernel's work counter and the merge of key splits) is captured once and replayed with new
    contents at the same addresses: every replay must match the oracle. The chunk geometry
    (seq_new, past_len) is frozen in the graph, as an engine replaying a fixed-shape chunk would."""
    torch = cuda
    H, KVH, HD, slots, past, S_new = 28, 4, 128, 1024, 600, 150
    rng = np.random.default_rng(7)
    scale = 1.0 / math.sqrt(HD)
    hk, hv = normal_f16(rng, 1, slots, KVH, HD), normal_f16(rng, 1, slots, KVH, HD)
    dk, dv = to_dev(torch, hk), to_dev(torch, hv)
    dq = torch.zeros(S_new, H, HD, dtype=torch.float16, device="cuda")
    dkn = torch.zeros(1, S_new, KVH, HD, dtype=torch.float16, device="cuda")
    dvn = torch.zeros(1, S_new, KVH, HD, dtype=torch.float16, device="cuda")
    out = torch.zeros(S_new, H, HD, dtype=torch.float16, device="cuda")
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   max_seq_new=S_new, tune_prefill_splits=splits))
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for s in range(4):
        q = normal_f16(rng, S_new, H, HD)
        kn, vn = normal_f16(rng, 1, S_new, KVH, HD), normal_f16(rng, 1, S_new, KVH, HD)
        with torch.cuda.stream(side):
            dq.copy_(to_dev(torch, q)); dkn.copy_(to_dev(torch, kn)); dvn.copy_(to_dev(torch, vn))
            if s == 0:
                with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
                    ctx.append_at(dkn, dvn, dk, dv, past, S_new)
                    ctx.prefill_attention(dq, dk, dv, out, S_new, past, scale)
            graph.replay()
        side.synchronize()
        hk[0, past:past + S_new] = kn[0]
        hv[0, past:past + S_new] = vn[0]
        ref = oracle.prefill(q, hk[0], hv[0], past, scale, threads=8)
        assert_close(oracle, out.cpu().numpy(), ref, f"replay {s}")
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), hk.view(np.uint16))
    assert ctx.device_status() == 0
    ctx.close()
