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
can be tested with gloo ranks on CPU; the compute is in libhkv's kernels and the step's host
(context, NCCL communicator, graph capture, failure detection) is C++ (libhkv_dist.so), of which
SeqSplitDecoder below is only a binding.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

from . import _capi


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


# ---------------------------------------------------------------------------
# libhkv_dist: the C++ host of the sequence-split step (include/hkv_dist.h)
# ---------------------------------------------------------------------------
DIST_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libhkv_dist.so")
UNIQUE_ID_BYTES = 128
ERR_PEER, ERR_TIMEOUT, ERR_ROSTER, ERR_HOST = 101, 102, 103, 104
_dist_lib = None


def load_dist() -> C.CDLL:
    """Loads libhkv_dist.so (once); raises if it was not built. It links libhkv and NCCL."""
    global _dist_lib
    if _dist_lib is not None:
        return _dist_lib
    if not os.path.exists(DIST_LIB_PATH):
        raise ImportError(f"{DIST_LIB_PATH} is missing. Build it with `python hector-engine_b200/build.py`.")
    _capi.load()
    # Order matters in a process that also uses PyTorch: torch ships its own libnccl.so.2 and must be
    # the one to load it; libhkv_dist then binds to that copy (same SONAME). Loaded the other way
    # round, torch would find an older system NCCL already mapped and fail to import.
    import torch  # noqa: F401
    lib = C.CDLL(DIST_LIB_PATH)
    vp, i32, f32p, i32p = C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int32)
    sigs = {
        "hkvd_unique_id": (C.c_int, [vp]),
        "hkvd_create": (C.c_int, [C.POINTER(vp), C.POINTER(_capi.HkvGeometry), i32, vp, C.c_float, vp]),
        "hkvd_create_with": (C.c_int, [C.POINTER(vp), C.POINTER(_capi.HkvGeometry), i32, vp, C.c_float, vp, i32, i32]),
        "hkvd_exchange": (C.c_int, [vp, i32p]),
        "hkvd_destroy": (C.c_int, [vp]),
        "hkvd_last_error": (C.c_char_p, [vp]),
        "hkvd_bind": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, C.c_uint64, vp]),
        "hkvd_step": (C.c_int, [vp, i32, i32p]),
        "hkvd_step_profiled": (C.c_int, [vp, f32p, f32p, f32p]),
        "hkvd_wait": (C.c_int, [vp, i32]),
        "hkvd_device_status": (C.c_int, [vp, i32p]),
        "hkvd_attach_roster": (C.c_int, [vp, C.c_char_p, i32, i32]),
        "hkvd_leave": (C.c_int, [vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)   # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    lib._hkvd_symbols = tuple(sigs)
    _dist_lib = lib
    return lib


class SeqSplitError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"hkvd status {status}: {message}")
        self.status = status


def _ptr(x) -> int:
    return 0 if x is None else (x if isinstance(x, int) else x.data_ptr())


class SeqSplitDecoder:
    """Binding of the C++ sequence-split decoder (host/hkv_seqsplit.hpp behind include/hkv_dist.h):
    per layer  local split-K partials -> NCCL all-gather -> merge  (or, `exchange="peer"`, partials
    stored straight into every rank's mailbox over NVLink and merged after a bounded flag wait: no
    collective launch), all layers captured once into a CUDA graph and replayed. The communicator is
    the C++ object's own; torch.distributed is used only to hand rank 0's communicator id to the
    other ranks. `exchange`: "auto" (peer stores when every rank can map every mailbox, else NCCL),
    "nccl", "peer"; `.exchange` says what is in use.

        dec = SeqSplitDecoder(geometry, shard, layers, stream=s)
        dec.bind(q, k_new, v_new, out, k_planes, v_planes, layer_stride_elems, d_total_seq)
        dec.step()            # enqueue one token (graph replay from the third call on)
        dec.wait(5000)        # host-side wait with a deadline; raises on a stuck or failed peer
    """

    EXCHANGES = {"auto": 0, "nccl": 1, "peer": 2}

    def __init__(self, geometry, shard: SeqShard, layers: int, scale: float = 0.0, stream=None, group=None,
                 exchange: str = "auto", peer_wait_ms: int = 0):
        import torch
        self.lib = load_dist()
        self.shard = shard
        geometry.shard_rank, geometry.shard_count, geometry.shard_block = shard.rank, shard.world, shard.block
        self.geometry = geometry
        self._g = geometry.to_c()
        uid = None
        if shard.world > 1:
            import torch.distributed as dist
            box = [None]
            if dist.get_rank(group) == 0:
                buf = C.create_string_buffer(UNIQUE_ID_BYTES)
                st = self.lib.hkvd_unique_id(buf)
                if st:
                    raise SeqSplitError(st, "hkvd_unique_id")
                box[0] = buf.raw
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            uid = C.create_string_buffer(box[0], UNIQUE_ID_BYTES)
        self.stream = stream if stream is not None else torch.cuda.current_stream()
        handle = C.c_void_p()
        st = self.lib.hkvd_create_with(C.byref(handle), C.byref(self._g), layers, uid, scale, self.stream.cuda_stream,
                                       self.EXCHANGES[exchange], peer_wait_ms)
        self._h = handle
        if st:
            msg = self.lib.hkvd_last_error(handle).decode() if handle else "allocation failed"
            self.close()
            raise SeqSplitError(st, msg)

    def _check(self, st: int):
        if st:
            raise SeqSplitError(st, self.lib.hkvd_last_error(self._h).decode())

    @property
    def exchange(self) -> str:
        mode = C.c_int32(0)
        self._check(self.lib.hkvd_exchange(self._h, C.byref(mode)))
        return {1: "nccl", 2: "peer"}[mode.value]

    def bind(self, q, k_new, v_new, out, k_planes, v_planes, layer_stride_elems: int, d_total_seq):
        self._check(self.lib.hkvd_bind(self._h, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(out), _ptr(k_planes),
                                       _ptr(v_planes), layer_stride_elems, _ptr(d_total_seq)))

    def step(self, eager: bool = False) -> bool:
        """Enqueues one step on the decoder's stream; True when it was a graph replay."""
        r = C.c_int32(0)
        self._check(self.lib.hkvd_step(self._h, 1 if eager else 0, C.byref(r)))
        return bool(r.value)

    def step_profiled(self):
        """One step with CUDA events around every phase -> (decode, all-gather, merge) ms summed over layers."""
        d, g, m = C.c_float(0), C.c_float(0), C.c_float(0)
        self._check(self.lib.hkvd_step_profiled(self._h, C.byref(d), C.byref(g), C.byref(m)))
        return d.value, g.value, m.value

    def wait(self, timeout_ms: int = 10000):
        self._check(self.lib.hkvd_wait(self._h, timeout_ms))

    def device_status(self) -> int:
        w = C.c_int32(0)
        st = self.lib.hkvd_device_status(self._h, C.byref(w))
        if st not in (0, 8):
            self._check(st)
        return w.value

    def attach_roster(self, name: str, fresh: bool, grace_ms: int = 1000):
        self._check(self.lib.hkvd_attach_roster(self._h, name.encode(), 1 if fresh else 0, grace_ms))

    def leave(self):
        self._check(self.lib.hkvd_leave(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self.lib.hkvd_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
