"""Multi-GPU decomposition of the path: one process per GPU, torch.distributed for plumbing.

Two ways the path shards (the reference is single-GPU and has neither):

* batch sharding — sequences are independent units; rank r owns sequences
  [r*B/N, (r+1)*B/N). No data-path collective at all.
* sequence split — ONE logical cache per sequence is dealt block-cyclically over the ranks
  (logical block j of `shard_block` positions lives on rank j % N as local block j // N).
  Every rank attends over its own rows with `hkv_decode_partials`, which yields one fp32
  partial (o[HD], m, l) per (sequence, head); one all-gather of B*H*(HD+2)*4 bytes per layer
  delivers all partials into local memory, and `hkv_combine_partials` merges them. The new
  K/V row is stored only by the rank that owns its position.

The arithmetic here (ownership, local row indices, buffer layout) is plain Python so that it
can be tested with gloo ranks on CPU; the compute is in libhkv's kernels.
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_batch(batch: int, world: int, rank: int) -> range:
    """Contiguous, balanced split of `batch` sequences: the first batch % world ranks get one more."""
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


@dataclass(frozen=True)
class SeqShard:
    """Block-cyclic sequence split: geometry of one rank's share of a logical cache."""
    rank: int
    world: int
    block: int = 1024  # positions per block; a multiple of 64 (the kernels' tile height)

    def __post_init__(self):
        if self.world < 1 or not 0 <= self.rank < self.world:
            raise ValueError("rank/world out of range")
        if self.block <= 0 or self.block % 64:
            raise ValueError("block must be a positive multiple of 64")

    def owner(self, pos: int) -> int:
        return (pos // self.block) % self.world

    def local_row(self, pos: int) -> int:
        """Row of this rank's plane that stores `pos`, or -1 if another rank owns it."""
        blk = pos // self.block
        if blk % self.world != self.rank:
            return -1
        return (blk // self.world) * self.block + pos % self.block

    def position_of_row(self, row: int) -> int:
        return ((row // self.block) * self.world + self.rank) * self.block + row % self.block

    def local_rows(self, total: int) -> int:
        """Number of this rank's rows that hold positions < total (they are rows [0, n))."""
        full, rem = divmod(total, self.block)
        n = ((full + self.world - 1 - self.rank) // self.world) * self.block
        if full % self.world == self.rank:
            n += rem
        return n

    def slots_for(self, max_total: int) -> int:
        """Rows per sequence this rank must allocate for sequences of up to `max_total` positions."""
        blocks = -(-max_total // self.block)
        return -(-blocks // self.world) * self.block


class SeqSplitDecoder:
    """One layer-geometry's sequence-split decode step on this rank.

    step(q, k_new, v_new, k_cache, v_cache, out, d_total_seq):
        local partials -> all_gather -> merge. `out` is replicated on every rank.
    """

    def __init__(self, hkv, geometry, shard: SeqShard, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group, self.shard = torch, dist, group, shard
        geometry.shard_rank, geometry.shard_count, geometry.shard_block = shard.rank, shard.world, shard.block
        self.ctx = hkv.Context(geometry)
        g = geometry
        kvh = g.num_heads if g.num_kv_heads is None else g.num_kv_heads
        del kvh
        self.part = torch.empty((g.batch, g.num_heads, g.head_dim + 2), dtype=torch.float32, device="cuda")
        # rank-major concatenation = [num_parts, batch, heads, head_dim + 2]
        self.gathered = torch.empty((shard.world * g.batch, g.num_heads, g.head_dim + 2), dtype=torch.float32,
                                    device="cuda")

    def step(self, q, k_new, v_new, k_cache, v_cache, out, d_total_seq, scale=None):
        self.ctx.decode_partials(q, k_new, v_new, k_cache, v_cache, self.part, d_total_seq, scale)
        if self.shard.world > 1:
            self.dist.all_gather_into_tensor(self.gathered, self.part, group=self.group)
            self.ctx.combine_partials(self.gathered, self.shard.world, out)
        else:
            self.ctx.combine_partials(self.part, 1, out)

    def close(self):
        self.ctx.close()
