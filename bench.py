#!/usr/bin/env python
"""Benchmark of the KV-append + cached decode-attention path.

A step = one decode step of the workload: every sequence of the batch advances one
position through ALL layers (per layer: append the new K/V row at the device-side cache
position, then grouped-query attention over the cache). Default workload: the
Qwen2-7B-shaped 28-layer config at context 32768 with the largest batch of {64,32,8,1}
that fits this GPU. Inputs are synthetic (seeded, approximately N(0,1) fp16), positions
uniform in [ctx/2, ctx).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl hkv|reference]

Prints ONE JSON line (rank 0). `value` is whole-job tokens/s with everything resident in
HBM; `e2e` is the same metric through the host-buffer C-ABI call (H2D of q/k_new/v_new and
D2H of the attention output inside the timed region); `roofline` is the split-K decode
kernel's algorithmic HBM bytes / its CUDA-event duration; `cpu_baseline` is the scalar CPU
oracle timed on a bounded sample.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

SEED = 0x48454B56
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.0172
WORKLOADS = {
    # name: layers, H, KVH, HD, window pattern (None = all global)
    "qwen2-7b": dict(layers=28, H=28, KVH=4, HD=128),
    "qwen2-0.5b": dict(layers=1, H=14, KVH=2, HD=64, batch=1, ctx=2048),
    "phi3-mini": dict(layers=32, H=32, KVH=32, HD=96, batch=16, ctx=4096),
    # 5 sliding-window layers (window 1024) per global layer
    "gemma-local-global": dict(layers=12, H=16, KVH=8, HD=256, window=1024, local_every=6, pos_rule="ctx-1-b",
                               batch=8, ctx=32768),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hkv", choices=["hkv", "reference"])
    ap.add_argument("--workload", default="qwen2-7b", choices=sorted(WORKLOADS))
    ap.add_argument("--ctx", type=int, default=0, help="context (0 = the workload's own, 32768 for qwen2-7b)")
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (0 = largest that fits)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (parity/debug runs)")
    ap.add_argument("--kernel", type=int, default=0, help="0 auto, 1 generic, 2 tma")
    ap.add_argument("--chunk-tiles", type=int, default=0)
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ref-layers", type=int, default=2, help="layers the reference arm runs per step")
    ap.add_argument("--past", type=int, default=30720, help="prefill mode: cache rows before the chunk")
    ap.add_argument("--chunk", type=int, default=2048, help="prefill mode: new queries per chunk")
    ap.add_argument("--mode", default="batch", choices=["batch", "seqsplit", "prefill"],
                    help="batch: sequences sharded over GPUs, no collective (default). seqsplit: every "
                         "sequence's cache split block-cyclically over the GPUs, partials all-gathered "
                         "over NCCL; --ctx is then the rows per sequence PER GPU")
    ap.add_argument("--shard-block", type=int, default=1024)
    ap.add_argument("--graph", action="store_true",
                    help="also time the step as ONE captured CUDA graph replayed --steps times (adds graph_replay)")
    ap.add_argument("--linear-window", action="store_true",
                    help="window layers keep a linear plane + mask (the reference's layout) instead of a ring")
    return ap.parse_args()


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs.

    The query process is started before warm-up (it needs ~0.1 s to come up) and streams a sample
    every 20 ms; a reader thread stamps each line on receipt and only the samples received between
    begin() and end() count. A region too short to catch three samples is followed by extra,
    untimed steps of the same work (`keep_loaded`) until three have been taken; the record says so."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_id: str):
        self.gpu_id = gpu_id
        self.proc = None
        self.samples = []   # (receipt time, [fields])
        self.t0 = self.t1 = None
        self.thread = None

    def start(self):
        import threading
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except Exception:
            self.proc = None
            return

        def reader():
            try:
                for line in self.proc.stdout:
                    self.samples.append((time.monotonic(), [p.strip() for p in line.split(",")]))
            except Exception:
                pass
        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def begin(self):
        self.t0 = time.monotonic()

    def end(self):
        self.t1 = time.monotonic()

    def _in_region(self):
        if self.t0 is None:
            return list(self.samples)
        t1 = self.t1 if self.t1 is not None else time.monotonic()
        return [f for (t, f) in list(self.samples) if self.t0 <= t <= t1 and len(f) >= 7]

    def stop(self, keep_loaded=None) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        if self.t1 is None:
            self.end()
        if keep_loaded is not None and len(self._in_region()) < 3:
            # the timed region was shorter than the sampling period: same load, untimed
            out["sampled_under"] = "extra untimed steps of the same work after the timed region"
            self.t0 = time.monotonic()
            self.t1 = None
            deadline = time.monotonic() + 2.0
            while len(self._in_region()) < 3 and time.monotonic() < deadline:
                keep_loaded()
            self.end()
        rows = self._in_region()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for parts in rows:
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(self.NAMES, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)), samples=len(sm),
                       power_w_max=float(max(power)))
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------
def pick_batch(torch, cfg, ctx, requested):
    per_seq = 2 * cfg["layers"] * ctx * cfg["KVH"] * cfg["HD"] * 2
    free, _ = torch.cuda.mem_get_info()
    if requested:
        return requested
    if cfg.get("batch"):
        return cfg["batch"]
    for b in (64, 32, 8, 1):
        if b * per_seq + (6 << 30) < free:
            return b
    raise SystemExit("not enough free device memory for batch 1")


def layer_specs(cfg, ctx, linear_window=False):
    """Per layer: (rows per sequence, window, layout). Window layers use a ring plane of
    `window` rows unless linear_window asks for the reference's layout (linear plane + mask)."""
    specs = []
    for l in range(cfg["layers"]):
        w = cfg.get("window", 0) if cfg.get("local_every") and (l % cfg["local_every"]) != cfg["local_every"] - 1 else 0
        if w and not linear_window:
            specs.append((w, w, 1))
        else:
            specs.append((ctx, w, 0))
    return specs


class Workload:
    def __init__(self, torch, hkv, cfg, ctx, B, rank, kernel=0, chunk_tiles=0, linear_window=False):
        self.torch, self.hkv, self.cfg, self.ctx_len, self.B, self.rank = torch, hkv, cfg, ctx, B, rank
        L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
        self.scale = 1.0 / math.sqrt(HD)
        self.specs = layer_specs(cfg, ctx, linear_window)
        dev = "cuda"
        self.k = [torch.empty((B, s, KVH, HD), dtype=torch.float16, device=dev) for s, _, _ in self.specs]
        self.v = [torch.empty((B, s, KVH, HD), dtype=torch.float16, device=dev) for s, _, _ in self.specs]
        self.q = torch.empty((L, B, H, HD), dtype=torch.float16, device=dev)
        self.kn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
        self.vn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
        self.out = torch.zeros((L, B, H, HD), dtype=torch.float16, device=dev)
        self.seeds = {n: SEED ^ (rank * 0x10001) ^ (i << 20) for i, n in enumerate(("k", "v", "q", "kn", "vn"))}
        for l in range(L):   # plane l is its own stream: element i of layer l = value(seed ^ (l << 8), i)
            hkv.fill_synthetic(self.k[l], self.seeds["k"] ^ (l << 8))
            hkv.fill_synthetic(self.v[l], self.seeds["v"] ^ (l << 8))
        for n, t in (("q", self.q), ("kn", self.kn), ("vn", self.vn)):
            hkv.fill_synthetic(t, self.seeds[n])
        if cfg.get("pos_rule") == "ctx-1-b":      # distinct ring phases
            self.pos0 = (ctx - 1 - np.arange(B)).astype(np.int32)
        else:
            self.pos0 = np.random.default_rng(SEED + rank).integers(ctx // 2, ctx, size=B).astype(np.int32)
        self.h_pos = torch.from_numpy(self.pos0.copy()).pin_memory()
        self.d_pos = torch.from_numpy(self.pos0.copy()).to(dev)
        self.ctxs = {}
        for spec in dict.fromkeys(self.specs):
            self.ctxs[spec] = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD,
                                                       slots=spec[0], window_size=spec[1], layout=spec[2],
                                                       kernel_select=kernel, chunk_tiles=chunk_tiles))
        self.hctx = self.ctxs[self.specs[0]]
        torch.cuda.synchronize()

    def ctx_of(self, layer):
        return self.ctxs[self.specs[layer]]

    def positions_at(self, step):
        return np.minimum(self.pos0 + step, self.ctx_len - 1)

    def reset_positions(self):
        self.d_pos.copy_(self.h_pos, non_blocking=True)

    def advance(self):
        self.d_pos.add_(1).clamp_(max=self.ctx_len - 1)

    def step_device(self):
        for l in range(self.cfg["layers"]):
            self.ctx_of(l).append_decode_attention(self.q[l], self.kn[l], self.vn[l], self.k[l], self.v[l],
                                                   self.out[l], self.d_pos, self.scale)
        self.advance()

    def device_status(self):
        return max(c.device_status() for c in self.ctxs.values())

    def algorithmic_bytes_per_layer(self, step, layer=None):
        """Sum over sequences of 4*L*KVH*HD (read K and V) + 8*KVH*HD (new row in, row out)
        + 4*H*HD (q in, out); L = attended rows (window-limited on window layers). With
        layer=None: mean over the layers."""
        H, KVH, HD = self.cfg["H"], self.cfg["KVH"], self.cfg["HD"]
        layers = range(self.cfg["layers"]) if layer is None else [layer]
        tot = 0
        for l in layers:
            Ls = self.positions_at(step).astype(np.int64) + 1
            if self.specs[l][1]:
                Ls = np.minimum(Ls, self.specs[l][1])
            tot += int((4 * Ls * KVH * HD).sum() + self.B * (8 * KVH * HD + 4 * H * HD))
        return tot / len(layers)


def _host_plane(w, oracle, name, layer, b, rows):
    """Rows [0, rows) of sequence b of a layer's plane, regenerated on the CPU from the seed."""
    KVH, HD = w.cfg["KVH"], w.cfg["HD"]
    row = KVH * HD
    slots = w.specs[layer][0]
    return oracle.fill(w.seeds[name] ^ (layer << 8), (b * slots) * row, rows * row).reshape(1, rows, KVH, HD).copy()


def verify(w: Workload, oracle, layer, seqs):
    """Full-size parity: regenerate the cache rows of (layer, b) on the CPU from the seed,
    append the new row, attend with the oracle, compare with the GPU's output."""
    cfg = w.cfg
    H, KVH, HD, B = cfg["H"], cfg["KVH"], cfg["HD"], w.B
    slots, window, layout = w.specs[layer]
    w.reset_positions()
    w.ctx_of(layer).append_decode_attention(w.q[layer], w.kn[layer], w.vn[layer], w.k[layer], w.v[layer],
                                            w.out[layer], w.d_pos, w.scale)
    status = w.ctx_of(layer).device_status()
    assert status == 0, f"device status word {status}"
    worst = 0.0
    row = KVH * HD
    for b in seqs:
        pos = int(w.pos0[b])
        rows = slots if layout == 1 else pos + 1
        kc, vc = _host_plane(w, oracle, "k", layer, b, rows), _host_plane(w, oracle, "v", layer, b, rows)
        nb = (layer * B + b) * row
        at = pos % slots if layout == 1 else pos
        kc[0, at] = oracle.fill(w.seeds["kn"], nb, row).reshape(KVH, HD)
        vc[0, at] = oracle.fill(w.seeds["vn"], nb, row).reshape(KVH, HD)
        q = oracle.fill(w.seeds["q"], (layer * B + b) * H * HD, H * HD).reshape(1, H, HD)
        ref = oracle.decode(q, kc, vc, [pos + 1], w.scale, window=window, layout=layout,
                            threads=oracle.hardware_threads())
        got = w.out[layer, b].cpu().numpy()
        ok, err = oracle.within_tolerance(got, ref[0])
        assert ok, f"parity failed at layer {layer} seq {b}: max abs err {err:.3e}"
        # the appended row must be in the cache, bit-exact
        assert np.array_equal(w.k[layer][b, at].cpu().numpy().view(np.uint16), kc[0, at].view(np.uint16))
        assert np.array_equal(w.v[layer][b, at].cpu().numpy().view(np.uint16), vc[0, at].view(np.uint16))
        worst = max(worst, err)
    return worst


def cpu_baseline(w: Workload, oracle, budget_s=12.0):
    """Scalar CPU oracle on a bounded sample: whole (sequence, layer) units, all heads, all
    host threads; tokens/s = units / (seconds * layers)."""
    cfg = w.cfg
    H, B = cfg["H"], w.B
    threads = oracle.hardware_threads()
    done, secs, wall0 = 0, 0.0, time.perf_counter()
    for i in range(B * cfg["layers"]):
        l, b = divmod(i, B)
        slots, window, layout = w.specs[l]
        pos = int(w.pos0[b])
        rows = slots if layout == 1 else pos + 1
        kc, vc = _host_plane(w, oracle, "k", l, b, rows), _host_plane(w, oracle, "v", l, b, rows)
        q = oracle.fill(w.seeds["q"], (l * B + b) * H * cfg["HD"], H * cfg["HD"]).reshape(1, H, cfg["HD"])
        t0 = time.perf_counter()
        oracle.decode(q, kc, vc, [pos + 1], w.scale, window=window, layout=layout, threads=threads)
        secs += time.perf_counter() - t0
        done += 1
        if secs > budget_s or time.perf_counter() - wall0 > 6 * budget_s:
            break
    tok_s = done / (secs * cfg["layers"])  # a token = one sequence through all layers
    return {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{done} (sequence, layer) units x {H} heads of the same workload "
                      f"({secs:.1f} s of CPU attention time), scaled to {cfg['layers']} layers per token"}


# ---------------------------------------------------------------------------
# reference arm: the reference's own kernels rebuilt for sm_100a (GPU only)
# ---------------------------------------------------------------------------
def run_reference(args, torch, hkv, oracle, cfg, ctx, B, rank):
    ref = oracle.load_reference()
    if ref is None:
        return None
    w = Workload(torch, hkv, cfg, ctx, B, rank, linear_window=True)  # the reference has no ring layout
    L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
    nl = max(1, min(args.ref_layers, L))
    d_total = (w.d_pos + 1).contiguous()
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        # The reference op is batch 1 with one scalar device position
        # (kernels/register_kernels.cpp:870): one launch pair per sequence, serially.
        for l in range(nl):
            for b in range(B):
                ref.hector_ref_kv_cache_update_dp(w.kn[l, b].data_ptr(), w.vn[l, b].data_ptr(),
                                                  w.k[l][b].data_ptr(), w.v[l][b].data_ptr(), 1, 1, KVH, HD,
                                                  ctx, w.d_pos.data_ptr() + 4 * b, stream)
                ref.hector_ref_attention_cached_dp(w.q[l, b].data_ptr(), w.k[l][b].data_ptr(),
                                                   w.v[l][b].data_ptr(), w.out[l, b].data_ptr(), 1,
                                                   d_total.data_ptr() + 4 * b, H, KVH, HD, ctx, w.scale,
                                                   w.specs[l][1], stream)
        w.advance()
        torch.add(w.d_pos, 1, out=d_total)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps * (L / nl)  # scaled from nl layers to all layers
    return w, ms, nl


def run_seqsplit(args, torch, hkv, dist, cfg, ctx_local, B, rank, world, base, gpu_id):
    """Long-context mode: one logical cache of ctx_local*world rows per sequence, dealt
    block-cyclically over the ranks; per layer: local split-K decode to one partial per
    (sequence, head), NCCL all-gather of the partials, merge. Output replicated on all ranks."""
    L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
    logical = ctx_local * world
    shard = hkv.dist.SeqShard(rank, world, args.shard_block)
    assert shard.slots_for(logical) == ctx_local, "ctx per GPU must be a multiple of the shard block"
    dev = "cuda"
    k = torch.empty((L, B, ctx_local, KVH, HD), dtype=torch.float16, device=dev)
    v = torch.empty((L, B, ctx_local, KVH, HD), dtype=torch.float16, device=dev)
    q = torch.empty((L, B, H, HD), dtype=torch.float16, device=dev)
    kn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
    vn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
    out = torch.zeros((L, B, H, HD), dtype=torch.float16, device=dev)
    for i, t in enumerate((k, v)):
        hkv.fill_synthetic(t, SEED ^ (rank * 0x10001) ^ (i << 20))
    for i, t in enumerate((q, kn, vn)):      # replicated inputs: same seed on every rank
        hkv.fill_synthetic(t, SEED ^ ((i + 2) << 20))
    pos0 = np.random.default_rng(SEED).integers(logical // 2, logical, size=B).astype(np.int32)
    d_tot = torch.from_numpy(pos0 + 1).to(dev)
    h_tot = torch.from_numpy(pos0 + 1).pin_memory()
    dec = hkv.dist.SeqSplitDecoder(hkv, hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD,
                                                     slots=ctx_local, kernel_select=args.kernel,
                                                     chunk_tiles=args.chunk_tiles), shard)
    scale = 1.0 / math.sqrt(HD)

    def step():
        for l in range(L):
            dec.step(q[l], kn[l], vn[l], k[l], v[l], out[l], d_tot, scale)
        d_tot.add_(1).clamp_(max=logical)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(gpu_id)
    sampler.start()
    for _ in range(args.warmup):
        step()
    d_tot.copy_(h_tot)
    barrier()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.end()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    extended = None
    if float(ms.item()) < 150.0:
        # shorter than a few sampling periods: every rank runs the same number of extra, untimed
        # steps (the step holds a collective) and the clocks are sampled under that same load
        sampler.begin()
        for _ in range(int(math.ceil(150.0 / max(ms_per_step, 1e-3)))):
            step()
        barrier()
        sampler.end()
        extended = "extra untimed steps of the same work after the timed region"
    clocks = sampler.stop()
    if extended:
        clocks["sampled_under"] = extended
    assert dec.ctx.device_status() == 0
    # algorithmic bytes over ALL ranks: the K/V rows of every sequence once, + new rows + q/out per rank
    Ls = np.stack([np.minimum(pos0 + 1 + s, logical) for s in range(args.steps)]).astype(np.int64)
    alg = float((4 * Ls * KVH * HD).sum(axis=1).mean() + world * B * (8 * KVH * HD + 4 * H * HD)) * L
    if rank == 0:
        cfgd = dict(base["config"], workload=f"{args.workload}-shaped long-context decode: {L} layers, logical ctx "
                    f"{logical} split block-cyclically ({args.shard_block}) over {world} GPU(s) = {ctx_local} rows per "
                    f"GPU, batch {B}", parallelism=f"sequence-split x{world}, NCCL all-gather of "
                    f"{B * H * (HD + 2) * 4} B partials per layer", global_batch=B, ctx=logical)
        line = dict(base, config=cfgd, impl="hkv", mode="seqsplit", value=B / (ms_per_step / 1e3),
                    ms_per_step=ms_per_step, clocks=clocks, gpu_launches=args.steps * L * 4,
                    hbm_gbs_step=alg / (ms_per_step * 1e-3) / 1e9,
                    hbm_gbs_per_gpu=alg / world / (ms_per_step * 1e-3) / 1e9,
                    hbm_frac_of_8TBs_per_gpu=alg / world / (ms_per_step * 1e-3) / 1e9 / 8000.0,
                    e2e=None, roofline=None, cpu_baseline=None)
        print(json.dumps(line))
    dec.close()


def run_prefill_reference(args, torch, oracle, cfg, base, gpu_id, q, k, v, out, S, past, slots, scale, ctx):
    """Reference arm of the prefill metric: the reference's own attention_prefill_cached kernel
    (kernels/attention.cu:664-788, rebuilt for sm_100a in oracle/_ref) on the same chunk. Its grid is
    one CTA per (query, head), each streaming its whole key range, so time is additive over queries:
    three slices of 32 queries (start, middle, end of the chunk) are timed and scaled to the chunk.
    The slices are also compared with this library's output for the same queries."""
    ref = oracle.load_reference()
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "oracle/_ref/libhector_ref_attention.so not built (reference checkout absent at build time)"}))
        ctx.close()
        return
    H, KVH, HD = cfg["H"], cfg["KVH"], cfg["HD"]
    n = min(32, S)
    los = sorted({0, max(0, S // 2 - n // 2), S - n})
    rout = torch.zeros((n, H, HD), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def ref_slice(lo):
        st = ref.hector_ref_attention_prefill_cached(q[lo:].data_ptr(), k.data_ptr(), v.data_ptr(), rout.data_ptr(), n,
                                                     past + lo, H, KVH, HD, slots, scale, 0, stream)
        assert st == 0, f"reference prefill kernel failed: {st}"

    worst = 0.0
    for lo in los:   # warm-up + agreement with this library (both within tolerance of the oracle)
        ref_slice(lo)
        torch.cuda.synchronize()
        ok, e = oracle.within_tolerance(out[lo:lo + n].cpu().numpy(), rout.cpu().numpy())
        assert ok, f"reference and hkv prefill disagree at query {lo}: {e:.3e}"
        worst = max(worst, e)
    sampler = ClockSampler(gpu_id)
    sampler.start()
    for _ in range(max(args.warmup, 1)):
        ref_slice(los[-1])
    torch.cuda.synchronize()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        for lo in los:
            ref_slice(lo)
    e1.record()
    torch.cuda.synchronize()
    sampler.end()
    clocks = sampler.stop(keep_loaded=lambda: (ref_slice(los[-1]), torch.cuda.synchronize()))
    ms = e0.elapsed_time(e1) / args.steps * (S / float(n * len(los)))
    flops = 4.0 * H * HD * sum(past + i + 1 for i in range(S))
    cfgd = {"workload": f"{args.workload}-shaped chunked prefill over the cache: chunk {S} queries, {past} rows "
                        f"already cached, {H}q/{KVH}kv heads, head_dim {HD}, one layer per step, batch 1",
            "chunk": S, "past_len": past}
    sample = (f"the reference's attention_prefill_cached kernel rebuilt for sm_100a, run on the GPU: {len(los)} slices of "
              f"{n} queries of the chunk per step, time scaled to {S} queries (one CTA per (query, head): additive)")
    val = S / (ms * 1e-3)
    line = dict(base, config=cfgd, impl="reference", mode="prefill", metric="prefill attention tokens/s (one layer)",
                value=val, ms_per_step=ms, clocks=clocks, gpu_launches=args.steps * len(los),
                tflops=flops / (ms * 1e-3) / 1e12, agreement_max_abs_err=worst,
                e2e={"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                cpu_baseline={"value": val, "unit": "tokens/s", "cores": 0, "kind": "reference", "sample": sample})
    print(json.dumps(line))
    ctx.close()


def run_prefill(args, torch, hkv, oracle, cfg, rank, base, gpu_id):
    """Chunked prefill over the cache (batch 1, one layer per call): append the chunk's K/V,
    then attention of its --chunk queries over rows [0, past + chunk). Tensor-bound:
    flops = 4*H*HD*sum_q(past + q + 1)."""
    H, KVH, HD = cfg["H"], cfg["KVH"], cfg["HD"]
    S, past = args.chunk, args.past
    slots = past + S
    dev = "cuda"
    k = torch.empty((slots, KVH, HD), dtype=torch.float16, device=dev)
    v = torch.empty((slots, KVH, HD), dtype=torch.float16, device=dev)
    q = torch.empty((S, H, HD), dtype=torch.float16, device=dev)
    kn = torch.empty((S, KVH, HD), dtype=torch.float16, device=dev)
    vn = torch.empty((S, KVH, HD), dtype=torch.float16, device=dev)
    out = torch.zeros((S, H, HD), dtype=torch.float16, device=dev)
    for i, t in enumerate((k, v, q, kn, vn)):
        hkv.fill_synthetic(t, SEED ^ (i << 20))
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   kernel_select=args.kernel, max_seq_new=S))
    scale = 1.0 / math.sqrt(HD)

    def step():
        ctx.append_at(kn, vn, k, v, past, S)
        ctx.prefill_attention(q, k, v, out, S, past, scale)

    step()
    assert ctx.device_status() == 0
    if args.impl == "reference":
        return run_prefill_reference(args, torch, oracle, cfg, base, gpu_id, q, k, v, out, S, past, slots, scale, ctx)
    err = None
    if not args.no_verify:  # sampled queries against the oracle
        hk, hv, hq = k.cpu().numpy(), v.cpu().numpy(), q.cpu().numpy()
        got = out.cpu().numpy()
        err = 0.0
        for lo in (0, S // 2, S - 4):
            ref = oracle.prefill(hq, hk, hv, past, scale, q_begin=lo, q_end=lo + 4, threads=oracle.hardware_threads())
            ok, e = oracle.within_tolerance(got[lo:lo + 4], ref[lo:lo + 4])
            assert ok, f"prefill parity failed at query {lo}: {e:.3e}"
            err = max(err, e)
    sampler = ClockSampler(gpu_id)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.begin()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    attn_ms = 0.0
    evs = []
    for _ in range(args.steps):
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record(); ctx.append_at(kn, vn, k, v, past, S)
        b.record(); ctx.prefill_attention(q, k, v, out, S, past, scale)
        c.record(); evs.append((a, b, c))
    torch.cuda.synchronize()
    sampler.end()
    clocks = sampler.stop(keep_loaded=lambda: (step(), torch.cuda.synchronize()))
    tot_ms = sum(a.elapsed_time(c) for a, b, c in evs) / args.steps
    attn_ms = sum(b.elapsed_time(c) for a, b, c in evs) / args.steps
    flops = 4.0 * H * HD * sum(past + i + 1 for i in range(S))
    peaks_path = os.path.join(REPO, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["bf16_tflops"]) if os.path.exists(peaks_path) else 1590.0
    achieved = flops / (attn_ms * 1e-3) / 1e12
    cfgd = {"workload": f"{args.workload}-shaped chunked prefill over the cache: chunk {S} queries, {past} rows "
                        f"already cached, {H}q/{KVH}kv heads, head_dim {HD}, one layer per step, batch 1",
            "chunk": S, "past_len": past, "l2": "K/V planes of %.0f MB, re-read per query tile" % (slots * KVH * HD * 4 / 1e6)}
    line = dict(base, config=cfgd, impl="hkv", mode="prefill", metric="prefill attention tokens/s (one layer)",
                value=S / (tot_ms * 1e-3), ms_per_step=tot_ms, clocks=clocks, gpu_launches=args.steps * 2,
                roofline={"bound": "tensor", "kernel": "hkv_prefill_tc_kernel", "achieved": achieved, "peak": peak,
                          "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": "measured burst bf16 GEMM",
                          "traffic": None, "algorithmic_flops_per_launch": flops, "avg_launch_ms": attn_ms},
                e2e=None, cpu_baseline=None, parity_max_abs_err=err)
    print(json.dumps(line))
    ctx.close()


def main():
    args = parse_args()
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0  # the reference has no multi-GPU path: rank 0 alone measures it
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path exists)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1 and args.impl != "reference":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    hkv = importlib.import_module("hector-engine_b200")
    hkv._capi.load()  # fail loudly if the native library is missing
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import hkv_oracle as oracle

    cfg = dict(WORKLOADS[args.workload])
    if args.layers:
        cfg["layers"] = args.layers
    ctx = args.ctx or cfg.get("ctx", 32768)
    B = 1 if args.mode == "prefill" else pick_batch(torch, cfg, ctx, args.batch)
    n_gpus = world if args.impl != "reference" else 1
    try:
        gpu_id = str(torch.cuda.get_device_properties(local).uuid)
        gpu_id = gpu_id if gpu_id.startswith("GPU-") else "GPU-" + gpu_id
    except Exception:
        gpu_id = str(local)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    workload_name = (f"{args.workload}-shaped decode: {cfg['layers']} layers, {cfg['H']}q/{cfg['KVH']}kv heads, "
                     f"head_dim {cfg['HD']}, ctx {ctx}, batch {B} per GPU, cache_pos ~ U[ctx/2, ctx)")
    config = {"workload": workload_name, "batch_per_gpu": B, "global_batch": B * n_gpus, "ctx": ctx,
              "layers": cfg["layers"], "parallelism": f"batch-sharded x{n_gpus} (no data-path collective)",
              "l2": "inputs larger than L2 (K/V read per step >> 126 MB)", "fp16_kv": True}
    base = {"metric": "decode attn+KV-append tokens/s", "unit": "tokens/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 storage / fp32 accumulate", "data": "synthetic",
            "config": config}

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference" and args.mode == "prefill":
        run_prefill(args, torch, hkv, oracle, cfg, rank, base, gpu_id)
        return 0
    if args.impl == "reference":
        sampler = ClockSampler(gpu_id)
        sampler.start()
        sampler.begin()
        res = run_reference(args, torch, hkv, oracle, cfg, ctx, B, rank)
        sampler.end()
        clocks = sampler.stop()
        if res is None:
            print(json.dumps({"impl": "reference", "unavailable":
                              "oracle/_ref/libhector_ref_attention.so not built (reference checkout absent at build time)"}))
            return 0
        w, ms, nl = res
        tok_s = B / (ms / 1e3)
        line = dict(base, impl="reference", value=tok_s, ms_per_step=ms, clocks=clocks,
                    gpu_launches=args.steps * nl * B * 3,
                    e2e={"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    cpu_baseline={"value": tok_s, "unit": "tokens/s", "cores": 0, "kind": "reference",
                                  "sample": f"the reference's own attention.cu + kv_cache_update kernels rebuilt for "
                                            f"sm_100a, run on the GPU (the reference has no CPU implementation of "
                                            f"this path): {nl} of {cfg['layers']} layers per step, one launch pair "
                                            f"per sequence as its batch-1 op does, time scaled to all layers"})
        print(json.dumps(line))
        return 0

    if args.mode == "prefill":
        if rank == 0:
            run_prefill(args, torch, hkv, oracle, cfg, rank, base, gpu_id)
        if dist is not None:
            dist.destroy_process_group()
        return 0
    if args.mode == "seqsplit":
        run_seqsplit(args, torch, hkv, dist, cfg, ctx, B, rank, n_gpus, base, gpu_id)
        if dist is not None:
            dist.destroy_process_group()
        return 0

    # ------------------------------------------------------------------ this library
    w = Workload(torch, hkv, cfg, ctx, B, rank, args.kernel, args.chunk_tiles, args.linear_window)
    L = cfg["layers"]
    verify_err = None
    if not args.no_verify:
        verify_err = verify(w, oracle, layer=L // 2, seqs=sorted({0, B // 2, B - 1}))

    # device-resident timing
    sampler = ClockSampler(gpu_id)
    sampler.start()
    w.reset_positions()
    for _ in range(args.warmup):
        w.step_device()
    w.reset_positions()
    barrier()
    for c in w.ctxs.values():
        c.profile_begin(args.steps * L)
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        w.step_device()
    e1.record()
    barrier()
    sampler.end()
    dec_ms = comb_ms = 0.0
    calls = 0
    for c in w.ctxs.values():
        d_, m_, n_ = c.profile_end()
        dec_ms, comb_ms, calls = dec_ms + d_, comb_ms + m_, calls + n_
    # (no collective inside the extra steps: every rank extends its own load independently)
    clocks = sampler.stop(keep_loaded=lambda: (w.step_device(), torch.cuda.synchronize()))
    graph_ms = None
    if args.graph:
        # The engine's own contract: the whole step captured ONCE, then replayed while only the
        # device positions change (src/engine.cpp:151-269 of the reference). Timed separately:
        # per-kernel events cannot be recorded inside a captured graph.
        w.reset_positions()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
                w.step_device()
            for _ in range(args.warmup):
                graph.replay()
            side.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(side)
            for _ in range(args.steps):
                graph.replay()
            g1.record(side)
            side.synchronize()
        graph_ms = g0.elapsed_time(g1) / args.steps
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    status = w.device_status()
    assert status == 0, f"device status word {status}"
    tok_s = B * n_gpus / (ms_per_step / 1e3)

    alg_bytes = float(np.mean([w.algorithmic_bytes_per_layer(s) for s in range(args.steps)]))
    peaks_path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    dec_avg_ms = dec_ms / max(calls, 1)
    achieved = alg_bytes / (dec_avg_ms * 1e-3) / 1e9
    # DRAM bytes (read + write) per algorithmic byte of the TMA decode kernel, from one ncu
    # capture of a batch-8 launch of this workload (profiles/decode_tma_qwen2-7b_b8_ctx32k_ncu_full.md);
    # the traffic is the K/V rows themselves, so it scales with the rows a launch reads.
    traffic = DRAM_BYTES_PER_ALGORITHMIC_BYTE * alg_bytes if w.hctx.kernel == 2 else None
    roofline = {"bound": "hbm", "kernel": "hkv_decode_tma_kernel" if w.hctx.kernel == 2 else "hkv_decode_generic_kernel",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_8TBs": achieved / 8000.0, "peak_source": peak_src, "traffic": traffic,
                "algorithmic_bytes_per_launch": alg_bytes, "avg_launch_ms": dec_avg_ms,
                "combine_avg_ms": comb_ms / max(calls, 1), "launches_timed": calls}
    step_gbs = alg_bytes * L / (ms_per_step * 1e-3) / 1e9

    # end to end through the host-buffer entry point
    e2e = None
    if not args.no_e2e:
        H, KVH, HD = cfg["H"], cfg["KVH"], cfg["HD"]
        hq = w.q.cpu().pin_memory()
        hk = w.kn.cpu().pin_memory()
        hv = w.vn.cpu().pin_memory()
        ho = torch.zeros((L, B, H, HD), dtype=torch.float16).pin_memory()
        w.reset_positions()

        def e2e_step():
            w.d_pos.copy_(w.h_pos, non_blocking=True)  # this step's positions, host -> device
            for l in range(L):
                w.ctx_of(l).append_decode_attention_host(hq[l], hk[l], hv[l], w.k[l], w.v[l], ho[l], w.d_pos, w.scale)
            torch.cuda.current_stream().synchronize()   # the step's result is now readable on the host
            w.h_pos.add_(1).clamp_(max=ctx - 1)

        for _ in range(min(args.warmup, 2)):
            e2e_step()
        barrier()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            e2e_step()
        t1.record()
        barrier()
        ems = torch.tensor([t0.elapsed_time(t1)], device="cuda")
        if dist is not None:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e_ms = float(ems.item()) / args.steps
        e2e = {"value": B * n_gpus / (e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": int(L * (B * H * HD + 2 * B * KVH * HD) * 2 + B * 4),
               "d2h_bytes_per_step": int(L * B * H * HD * 2)}

    cpu = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w, oracle)

    if rank == 0:
        line = dict(base, impl="hkv", value=tok_s, ms_per_step=ms_per_step, clocks=clocks, e2e=e2e,
                    gpu_launches=args.steps * L * w.hctx.launches_per_decode, roofline=roofline,
                    cpu_baseline=cpu, hbm_gbs_step=step_gbs, hbm_frac_of_8TBs_step=step_gbs / 8000.0,
                    parity_max_abs_err=verify_err)
        if graph_ms is not None:
            line["graph_replay"] = {"ms_per_step": graph_ms, "value": B * n_gpus / (graph_ms / 1e3), "unit": "tokens/s",
                                    "hbm_gbs_step": alg_bytes * L / (graph_ms * 1e-3) / 1e9}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
