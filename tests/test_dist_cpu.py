"""CPU suite for the multi-GPU decomposition: world_size-2 gloo ranks exercise the
sequence-split protocol (block-cyclic ownership, partial format, all-gather layout, merge)
with a numpy stand-in for the per-rank kernel, checked against the oracle on the full cache;
plus the batch-sharding arithmetic. The kernels themselves are covered by the GPU suite."""
import ctypes as C
import importlib
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)

LOG2E = 1.4426950408889634


def numpy_partial(q, k_rows, v_rows, valid, scale, G):
    """One rank's partial per (sequence, head): o[HD] un-normalised, m (log2 domain), l —
    the format hkv_decode_partials writes."""
    B, H, HD = q.shape
    out = np.zeros((B, H, HD + 2), np.float32)
    out[:, :, HD] = -1.0e30
    for b in range(B):
        rows = np.nonzero(valid[b])[0]
        if rows.size == 0:
            continue
        for h in range(H):
            kv = h // G
            s = (k_rows[b, rows, kv].astype(np.float32) @ q[b, h].astype(np.float32)) * (scale * LOG2E)
            m = s.max()
            p = np.exp2(s - m)
            out[b, h, :HD] = p @ v_rows[b, rows, kv].astype(np.float32)
            out[b, h, HD] = m
            out[b, h, HD + 1] = p.sum()
    return out


def merge_partials(parts):
    """[N, B, H, HD+2] -> fp16 [B, H, HD], the arithmetic of hkv_combine_partials."""
    HD = parts.shape[-1] - 2
    m = parts[..., HD]
    M = m.max(axis=0)
    w = np.exp2(m - M)
    L = (parts[..., HD + 1] * w).sum(axis=0)
    o = (parts[..., :HD] * w[..., None]).sum(axis=0)
    inv = np.where(L > 0, 1.0 / np.where(L > 0, L, 1.0), 0.0)
    return (o * inv[..., None]).astype(np.float16)


def _rank_main(rank, world, port, result_dir):
    sys.path[:0] = [REPO, os.path.join(REPO, "oracle"), HERE]
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import hkv_oracle as oracle
        from _util import make_case
        hkv = importlib.import_module("hector-engine_b200")
        B, H, KVH, HD, ctx, BLK = 3, 8, 2, 32, 700, 64
        totals = np.array([700, 321, 64], np.int32)
        q, nk, nv, kc, vc = make_case(77, B, H, KVH, HD, ctx, fill="garbage")
        shard = hkv.dist.SeqShard(rank, world, BLK)
        # the new row of each sequence sits at position total-1; only its owner stores it
        new_pos = totals - 1
        full_k, full_v = kc.copy(), vc.copy()
        oracle.append(nk, nv, full_k, full_v, new_pos)           # what the logical cache must hold
        slots = shard.slots_for(ctx)
        lk = np.zeros((B, slots, KVH, HD), np.float16)
        lv = np.zeros_like(lk)
        valid = np.zeros((B, slots), bool)
        for b in range(B):
            for p in range(int(totals[b])):
                r = shard.local_row(p)
                if r < 0:
                    continue
                src_k, src_v = (nk[b, 0], nv[b, 0]) if p == new_pos[b] else (kc[b, p], vc[b, p])
                lk[b, r], lv[b, r], valid[b, r] = src_k, src_v, True
            assert valid[b].sum() == shard.local_rows(int(totals[b]))
            assert not valid[b, shard.local_rows(int(totals[b])):].any()   # rows are dense from 0
        scale = 0.2
        part = torch.from_numpy(numpy_partial(q, lk, lv, valid, scale, H // KVH))
        gathered = torch.empty((world * B, H, HD + 2), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, part)              # rank-major: [num_parts, B, H, HD+2]
        merged = merge_partials(gathered.view(world, B, H, HD + 2).numpy())
        ref = oracle.decode(q, full_k, full_v, totals, scale)
        ok, err = oracle.within_tolerance(merged, ref)
        assert ok, f"rank {rank}: sequence-split result differs from the oracle ({err:.3e})"
        # every rank derives the same answer (output is replicated)
        chk = torch.tensor([float(np.abs(merged.astype(np.float32)).sum())], dtype=torch.float64)
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert lo.item() == hi.item()
        # the library's own planning arithmetic agrees with the Python mirror
        lib = hkv._capi.load()
        g = hkv.Geometry(num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots, shard_rank=rank,
                         shard_count=world, shard_block=BLK).to_c()
        for p in range(ctx):
            assert lib.hkv_slot_of_position(C.byref(g), p) == shard.local_row(p)
        for r in range(slots):
            assert lib.hkv_position_of_slot(C.byref(g), r, ctx) == shard.position_of_row(r)
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_sequence_split_protocol_two_gloo_ranks(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_batch_sharding_is_a_balanced_partition(hkv):
    for B in (1, 7, 8, 64, 65):
        for world in (1, 2, 4, 8):
            parts = [hkv.dist.shard_batch(B, world, r) for r in range(world)]
            flat = [i for p in parts for i in p]
            assert flat == list(range(B))
            sizes = [len(p) for p in parts]
            assert max(sizes) - min(sizes) <= 1


def test_seq_shard_arithmetic(hkv):
    S = hkv.dist.SeqShard
    with pytest.raises(ValueError):
        S(0, 2, 100)
    with pytest.raises(ValueError):
        S(2, 2, 64)
    for world in (1, 2, 8):
        shards = [S(r, world, 128) for r in range(world)]
        for total in (0, 1, 127, 128, 129, 5000, 131072):
            assert sum(s.local_rows(total) for s in shards) == total
        owners = [shards[0].owner(p) for p in range(0, 128 * world * 2, 128)]
        assert owners == list(range(world)) * 2
        assert all(s.slots_for(131072) == 131072 // world for s in shards)
