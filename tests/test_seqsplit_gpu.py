"""GPU tests of the sequence-split path: hkv_decode_partials over block-cyclic shards of one
logical cache, then hkv_combine_partials over the gathered partials, against the oracle on
the full cache. On one GPU the ranks are run one after another (no kernel here waits on
another rank, so this is the same computation); with >= 2 GPUs a real NCCL all-gather runs."""
import importlib
import math
import os
import sys

import numpy as np
import pytest

from _util import assert_close, make_case, to_dev

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)


def build_shards(hkv, world, BLK, kc, vc, totals, append_pos):
    """Deal the logical planes to `world` local planes (rows of position p for p < total,
    except the position being appended, which the kernel must write itself)."""
    B, ctx, KVH, HD = kc.shape
    shards = [hkv.dist.SeqShard(r, world, BLK) for r in range(world)]
    slots = shards[0].slots_for(ctx)
    lk = [np.zeros((B, slots, KVH, HD), np.float16) for _ in range(world)]
    lv = [np.zeros((B, slots, KVH, HD), np.float16) for _ in range(world)]
    for b in range(B):
        for p in range(int(totals[b])):
            if p == append_pos[b]:
                continue
            r = shards[0].owner(p)
            row = shards[r].local_row(p)
            lk[r][b, row], lv[r][b, row] = kc[b, p], vc[b, p]
    return shards, slots, lk, lv


@pytest.mark.parametrize("kernel", [1, 2], ids=["generic", "tma"])
@pytest.mark.parametrize("world,BLK", [(2, 64), (4, 128), (8, 64)])
def test_sequence_split_single_gpu_emulation(hkv, cuda, oracle, world, BLK, kernel):
    torch = cuda
    B, H, KVH, HD, ctx = 3, 28, 4, 128, 2048
    totals = np.array([2048, 1000, 65], np.int32)
    pos = totals - 1
    q, nk, nv, kc, vc = make_case(world * 31 + BLK, B, H, KVH, HD, ctx, fill="garbage")
    full_k, full_v = kc.copy(), vc.copy()
    oracle.append(nk, nv, full_k, full_v, pos)
    scale = 1.0 / math.sqrt(HD)
    ref = oracle.decode(q, full_k, full_v, totals, scale, threads=8)

    shards, slots, lk, lv = build_shards(hkv, world, BLK, kc, vc, totals, pos)
    dq, dnk, dnv, dtot = to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv), to_dev(torch, totals)
    parts = torch.zeros(world, B, H, HD + 2, dtype=torch.float32, device="cuda")
    ctxs = []
    for r in range(world):
        ctx_r = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                         shard_rank=r, shard_count=world, shard_block=BLK,
                                         kernel_select=kernel))
        dk, dv = to_dev(torch, lk[r]), to_dev(torch, lv[r])
        ctx_r.decode_partials(dq, dnk, dnv, dk, dv, parts[r], dtot, scale)
        assert ctx_r.device_status() == 0
        # the appended row landed on its owner only, bit-exact; other planes are untouched
        gk, gv = dk.cpu().numpy(), dv.cpu().numpy()
        want_k, want_v = lk[r].copy(), lv[r].copy()
        for b in range(B):
            row = shards[r].local_row(int(pos[b]))
            if row >= 0:
                want_k[b, row], want_v[b, row] = nk[b, 0], nv[b, 0]
        assert np.array_equal(gk.view(np.uint16), want_k.view(np.uint16))
        assert np.array_equal(gv.view(np.uint16), want_v.view(np.uint16))
        ctxs.append(ctx_r)
    out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
    ctxs[0].combine_partials(parts, world, out)
    torch.cuda.synchronize()
    assert_close(oracle, out.cpu().numpy(), ref, f"sequence split over {world} ranks")
    for c in ctxs:
        c.close()


@pytest.mark.parametrize("world,BLK,batch", [(2, 64, 3), (4, 128, 3), (8, 64, 1)])
def test_peer_exchange_single_gpu_emulation(hkv, cuda, oracle, world, BLK, batch):
    """The mailbox exchange with every rank on one GPU. A rank's merge kernel releases its own epoch
    flag and then waits for the others', which on one GPU would be later launches of the same
    stream — so here the test itself stores the epoch into every flag word between the publishing
    launches and the merges (what the peers' merge kernels do on their own GPUs; the real handshake
    runs in the multi-GPU tests). Three steps exercise both parities of the mailboxes; every rank's
    merged output must match the oracle on the full logical cache."""
    torch = cuda
    B, H, KVH, HD, ctx = batch, 28, 4, 128, 2048
    totals0 = np.array([2040, 1000, 65][:B], np.int32)
    q, nk, nv, kc, vc = make_case(world * 17 + BLK, B, H, KVH, HD, ctx, fill="garbage")
    scale = 1.0 / math.sqrt(HD)
    shards, slots, lk, lv = build_shards(hkv, world, BLK, kc, vc, totals0 - 1, np.full(B, -1))
    ctxs, planes, boxes = [], [], []
    for r in range(world):
        c = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                     shard_rank=r, shard_count=world, shard_block=BLK))
        ctxs.append(c)
        planes.append((to_dev(torch, lk[r]), to_dev(torch, lv[r])))
        boxes.append(torch.zeros(c.exchange_bytes(world), dtype=torch.uint8, device="cuda"))
    assert boxes[0].numel() == 512 + 2 * B * H * (HD + 2) * 4
    xs = [hkv.Context.make_exchange(r, boxes, wait_limit_ms=200) for r in range(world)]
    full_k, full_v = kc.copy(), vc.copy()
    dq, dnk, dnv = to_dev(torch, q), to_dev(torch, nk), to_dev(torch, nv)
    outs = [torch.zeros(B, H, HD, dtype=torch.float16, device="cuda") for _ in range(world)]
    for step in range(3):
        totals = totals0 + step
        oracle.append(nk, nv, full_k, full_v, totals - 1)
        ref = oracle.decode(q, full_k, full_v, totals, scale, threads=8)
        dtot = to_dev(torch, totals)
        for r in range(world):
            ctxs[r].decode_partials_publish(dq, dnk, dnv, planes[r][0], planes[r][1], xs[r], dtot, scale)
        for b in boxes:
            b[:4 * world].view(torch.int32).fill_(step + 1)
        for r in range(world):
            ctxs[r].merge_published(xs[r], outs[r])
        torch.cuda.synchronize()
        for r in range(world):
            assert ctxs[r].device_status() == 0
            assert_close(oracle, outs[r].cpu().numpy(), ref, f"step {step}, rank {r} of {world}")
        epochs = [int(b[256:260].view(torch.int32)[0]) for b in boxes]
        assert epochs == [step + 1] * world
    for c in ctxs:
        c.close()


def test_peer_exchange_wait_runs_out_as_a_status(hkv, cuda):
    """A peer that never publishes: the merge kernel's wait gives up after its limit, leaves the output
    rows alone, reports through the status word and returns; the context keeps working."""
    torch = cuda
    B, H, KVH, HD, slots = 2, 8, 2, 64, 128
    c = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                 shard_rank=0, shard_count=2, shard_block=64))
    boxes = [torch.zeros(c.exchange_bytes(2), dtype=torch.uint8, device="cuda") for _ in range(2)]
    x = hkv.Context.make_exchange(0, boxes, wait_limit_ms=50)
    rng = np.random.default_rng(3)
    f16 = lambda *s: to_dev(torch, rng.standard_normal(s, dtype=np.float32).astype(np.float16))
    q, k, v = f16(B, 1, H, HD), f16(B, slots, KVH, HD), f16(B, slots, KVH, HD)
    tot = to_dev(torch, np.array([100, 7], np.int32))
    out = torch.full((B, H, HD), 7.0, dtype=torch.float16, device="cuda")
    c.decode_partials_publish(q, None, None, k, v, x, tot)
    c.merge_published(x, out)                       # rank 1 never publishes
    torch.cuda.synchronize()
    assert c.device_status() == 1                # the wait ran out; reading clears the word
    assert bool((out == 7.0).all())
    assert c.device_status() == 0
    # the epoch has advanced all the same; the next exchange works once "rank 1" releases its flag
    assert int(boxes[0][256:260].view(torch.int32)[0]) == 1
    c.decode_partials_publish(q, None, None, k, v, x, tot)
    boxes[0][4:8].view(torch.int32)[0] = 2       # flag word of rank 1 in rank 0's mailbox
    c.merge_published(x, out)
    torch.cuda.synchronize()
    assert c.device_status() == 0
    assert not bool((out == 7.0).all())
    assert [int(b[0:4].view(torch.int32)[0]) for b in boxes] == [2, 2]   # rank 0 released epoch 2 in both mailboxes
    with pytest.raises(hkv.HkvError):
        c.merge_published(hkv.Context.make_exchange(1, boxes), out)      # not this context's rank
    c.close()


def _nccl_rank(rank, world, port, result_dir):
    sys.path[:0] = [REPO, os.path.join(REPO, "oracle"), HERE]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import hkv_oracle as oracle
        hkv = importlib.import_module("hector-engine_b200")
        B, H, KVH, HD, ctx, BLK = 4, 28, 4, 128, 4096, 256
        totals = np.array([4096, 3000, 257, 1], np.int32)
        pos = totals - 1
        q, nk, nv, kc, vc = make_case(5, B, H, KVH, HD, ctx, fill="garbage")
        full_k, full_v = kc.copy(), vc.copy()
        oracle.append(nk, nv, full_k, full_v, pos)
        scale = 1.0 / math.sqrt(HD)
        ref = oracle.decode(q, full_k, full_v, totals, scale, threads=4)
        shards, slots, lk, lv = build_shards(hkv, world, BLK, kc, vc, totals, pos)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        stream = torch.cuda.Stream()
        for exchange in ("nccl", "peer"):   # the collective, then the mailboxes (plain peer stores)
            dec = hkv.dist.SeqSplitDecoder(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots),
                                           shards[rank], layers=1, scale=scale, stream=stream, exchange=exchange,
                                           peer_wait_ms=5000)
            assert dec.exchange == exchange
            out = torch.zeros(B, H, HD, dtype=torch.float16, device="cuda")
            dk, dv, dq, dnk, dnv, dtot = dev(lk[rank]), dev(lv[rank]), dev(q), dev(nk), dev(nv), dev(totals)
            torch.cuda.synchronize()
            dec.bind(dq, dnk, dnv, out, dk, dv, dk.numel(), dtot)
            replays = 0
            for _ in range(4):  # un-captured, captured + launched, replayed twice: every call re-appends the same row and must agree
                replays += dec.step()
                dec.wait(30000)
                ok, err = oracle.within_tolerance(out.cpu().numpy(), ref)
                assert ok, f"rank {rank} ({exchange}): {err}"
            assert replays == 3
            d_ms, g_ms, m_ms = dec.step_profiled()
            assert d_ms > 0 and m_ms > 0 and (g_ms > 0 or exchange == "peer")
            assert dec.device_status() == 0
            ok, err = oracle.within_tolerance(out.cpu().numpy(), ref)
            assert ok, f"rank {rank} ({exchange}): {err}"
            dec.close()
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_sequence_split_nccl_ranks(cuda, tmp_path):
    torch = cuda
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs >= 2 GPUs (covered on one GPU by the emulation test and on CPU by gloo ranks)")
    world = 2 if n < 4 else 4
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_nccl_rank, args=(world, 29700 + os.getpid() % 200, str(tmp_path)), nprocs=world, join=True)
    assert len(os.listdir(tmp_path)) == world


def test_context_refuses_a_call_made_on_another_device(hkv, cuda):
    """A context's workspace, status word, tensor maps and shared-memory opt-ins live on the device it
    was created on: a launch entry point called with another device current is refused on the host
    (HKV_ERR_INVALID_ARG, 'context belongs to device N') instead of launching there."""
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs >= 2 GPUs")
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=4, num_kv_heads=4, head_dim=64, slots=128))
    t = torch.zeros(128 * 4 * 64, dtype=torch.float16, device="cuda:0")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    try:
        torch.cuda.set_device(1)
        with pytest.raises(hkv.HkvError) as e:
            ctx.append(t, t, t, t, pos, 1, stream=0)
        assert e.value.status == 1 and "belongs to device 0" in str(e.value)
    finally:
        torch.cuda.set_device(0)
    ctx.append(t, t, t, t, pos, 1)       # and it still works where it belongs
    torch.cuda.synchronize()
    ctx.close()
