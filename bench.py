#!/usr/bin/env python
"""Benchmark of the KV-append + cached decode-attention path.

A step = one decode step of the workload: every sequence of the batch advances one
position through ALL layers (per layer: append the new K/V row at the device-side cache
position, then grouped-query attention over the cache). Default workload: the
Qwen2-7B-shaped 28-layer config at context 32768 with the largest batch of {64,32,8,1}
that fits this GPU. Inputs are synthetic (seeded, approximately N(0,1) fp16), positions
uniform in [ctx/2, ctx).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl hkv|reference]

Prints ONE JSON line (rank 0).
  value        whole-job tokens/s with everything resident in HBM, the step captured ONCE as a
               CUDA graph and replayed K times (the engine's own execution mode); mean, median
               and minimum step times are all given, `eager` is the same step issued as one
               C-ABI call per layer
  e2e          the same metric through the host-buffer C-ABI call (H2D of q/k_new/v_new and D2H
               of the attention output inside the timed region)
  roofline     the split-K decode kernel's algorithmic HBM bytes / its CUDA-event duration,
               taken in a separate pass so that no event sits inside the timed region
  cpu_baseline the scalar CPU oracle timed on a bounded sample
  extras       (1 GPU) compact, parity-checked records of the other model shapes and batch
               sizes, of the tensor-core prefill chunk and of the fused norm+RoPE+cache write
  seqsplit     the sequence-split path (one logical cache dealt over the GPUs, NCCL all-gather
               of the partials, hosted in C++): strong scaling of batch 64 / ctx 32768, and on
               8 GPUs the 131072-token decode of the long-context config

--impl reference times the reference's own kernels (rebuilt for sm_100a under oracle/_ref) on the
same workload and never loads this repository's library.
"""
from __future__ import annotations

import argparse
import gc
import importlib
import json
import math
import os
import subprocess
import sys
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "oracle"))

SEED = 0x48454B56
# DRAM bytes (read + write) per algorithmic byte of the TMA decode kernel, from an ncu capture of a
# batch-8 launch of the default workload; the traffic is the K/V rows themselves, so it scales with
# the rows a launch reads.
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.012
WORKLOADS = {
    # name: layers, H, KVH, HD, window pattern (None = all global)
    "qwen2-7b": dict(layers=28, H=28, KVH=4, HD=128),
    "qwen2-0.5b": dict(layers=1, H=14, KVH=2, HD=64, batch=1, ctx=2048, pos_rule="fixed-511"),
    "phi3-mini": dict(layers=32, H=32, KVH=32, HD=96, batch=16, ctx=4096),
    # 5 sliding-window layers (window 1024) per global layer
    "gemma-local-global": dict(layers=12, H=16, KVH=8, HD=256, window=1024, local_every=6, pos_rule="ctx-1-b",
                               batch=8, ctx=32768),
}


# The one JSON line goes to the process's ORIGINAL standard output; everything else that writes to file
# descriptor 1 meanwhile (NCCL announces its version there when a communicator is first created) goes to stderr.
_REAL_STDOUT = None


def claim_stdout():
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    sys.stdout.flush()
    data = (json.dumps(obj) + "\n").encode()
    os.write(_REAL_STDOUT if _REAL_STDOUT is not None else 1, data)


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
    ap.add_argument("--tma-groups", type=int, default=0, help="decode kernel shape: 0 auto, 1 two CTAs per SM, 2 one CTA per SM")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra records of the 1-GPU line")
    ap.add_argument("--no-seqsplit", action="store_true", help="skip the sequence-split legs")
    ap.add_argument("--past", type=int, default=30720, help="prefill mode: cache rows before the chunk")
    ap.add_argument("--chunk", type=int, default=2048, help="prefill / rope mode: new queries per chunk")
    ap.add_argument("--mode", default="batch", choices=["batch", "seqsplit", "prefill", "rope"],
                    help="batch: sequences sharded over GPUs, no collective (default; adds the extras and the "
                         "sequence-split legs). seqsplit: only the sequence-split leg; --ctx is then the LOGICAL "
                         "context, split over the GPUs. prefill / rope: one kernel's own figure")
    ap.add_argument("--shard-block", type=int, default=256,
                    help="sequence split: positions per dealt block (256 balances the ranks' rows better than 1024: +3 %% at 4 GPUs)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "peer"],
                    help="sequence split: how partials travel between the ranks")
    ap.add_argument("--ring-extra", type=int, default=0,
                    help="rows a window layer's ring plane has beyond its window (a plane sized for chunked prefill)")
    ap.add_argument("--linear-window", action="store_true",
                    help="window layers keep a linear plane + mask (the reference's layout) instead of a ring")
    return ap.parse_args()


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs.

    The query process is started before warm-up (it needs a moment to come up) and streams a sample
    every 20 ms; a reader thread stamps each line on receipt and only the samples received between
    begin() and end() count. A region too short to catch three samples is followed by extra,
    untimed steps of the same work until three have been taken; the record says so."""
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
        self.note = None

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
        self.t0, self.t1 = time.monotonic(), None

    def end(self):
        self.t1 = time.monotonic()

    def in_region(self):
        if self.t0 is None:
            return list(self.samples)
        t1 = self.t1 if self.t1 is not None else time.monotonic()
        return [f for (t, f) in list(self.samples) if self.t0 <= t <= t1 and len(f) >= 7]

    def extend(self, keep_loaded, agree=None, want=3, limit_s=4.0):
        """The timed region was shorter than a few sampling periods: run the same work again,
        untimed, and sample under it. `agree(n)` (multi-rank work with a collective inside) maps this
        rank's sample count to the minimum over the ranks, so that every rank runs the same number of
        extra rounds."""
        count = lambda: len(self.in_region())
        n = agree(count()) if agree else count()
        if n >= want:
            return
        self.note = "extra untimed steps of the same work after the timed region"
        self.begin()
        deadline = time.monotonic() + limit_s
        while True:
            keep_loaded()
            n = agree(count()) if agree else count()
            late = time.monotonic() >= deadline
            if agree:
                late = agree(0 if late else 1) == 0   # stop together
            if n >= want or late:
                break
        self.end()

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        if self.t1 is None:
            self.end()
        rows = self.in_region()
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
        if self.note:
            out["sampled_under"] = self.note
        return out


def gpu_uuid(torch, local):
    try:
        gpu_id = str(torch.cuda.get_device_properties(local).uuid)
        return gpu_id if gpu_id.startswith("GPU-") else "GPU-" + gpu_id
    except Exception:
        return str(local)


def step_stats(ms_list):
    a = np.asarray(ms_list, dtype=np.float64)
    return {"ms_per_step": float(a.mean()), "ms_per_step_median": float(np.median(a)), "ms_per_step_min": float(a.min())}


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


def layer_specs(cfg, ctx, linear_window=False, ring_extra=0):
    """Per layer: (rows per sequence, window, layout). Window layers use a ring plane of
    `window` (+ ring_extra: a plane sized for chunked prefill) rows unless linear_window asks for the
    reference's layout (linear plane + mask)."""
    specs = []
    for l in range(cfg["layers"]):
        w = cfg.get("window", 0) if cfg.get("local_every") and (l % cfg["local_every"]) != cfg["local_every"] - 1 else 0
        if w and not linear_window:
            specs.append((w + ring_extra, w, 1))
        else:
            specs.append((ctx, w, 0))
    return specs


def start_positions(cfg, ctx, B, rank):
    if cfg.get("pos_rule") == "ctx-1-b":      # distinct ring phases
        return (ctx - 1 - np.arange(B)).astype(np.int32)
    if cfg.get("pos_rule") == "fixed-511":    # the single-layer correctness config: append at 511
        return np.full(B, 511, np.int32)
    return np.random.default_rng(SEED + rank).integers(ctx // 2, ctx, size=B).astype(np.int32)


class Workload:
    def __init__(self, torch, hkv, cfg, ctx, B, rank, kernel=0, chunk_tiles=0, linear_window=False, tma_groups=0,
                 ring_extra=0):
        self.torch, self.hkv, self.cfg, self.ctx_len, self.B, self.rank = torch, hkv, cfg, ctx, B, rank
        L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
        self.scale = 1.0 / math.sqrt(HD)
        self.specs = layer_specs(cfg, ctx, linear_window, ring_extra)
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
        self.pos0 = start_positions(cfg, ctx, B, rank)
        self.h_pos = torch.from_numpy(self.pos0.copy()).pin_memory()
        self.d_pos = torch.from_numpy(self.pos0.copy()).to(dev)
        self.ctxs = {}
        for spec in dict.fromkeys(self.specs):
            self.ctxs[spec] = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD,
                                                       slots=spec[0], window_size=spec[1], layout=spec[2],
                                                       kernel_select=kernel, chunk_tiles=chunk_tiles,
                                                       tune_tma_groups=tma_groups))
        self.hctx = self.ctxs[self.specs[0]]
        torch.cuda.synchronize()

    def close(self):
        for c in self.ctxs.values():
            c.close()
        self.ctxs = {}
        self.k = self.v = self.q = self.kn = self.vn = self.out = None

    def ctx_of(self, layer):
        return self.ctxs[self.specs[layer]]

    def contexts(self):
        return list(self.ctxs.values())

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


def verify(w: Workload, oracle, layers, seqs):
    """Full-size parity: regenerate the cache rows of (layer, b) on the CPU from the seed,
    append the new row, attend with the oracle, compare with the GPU's output."""
    cfg = w.cfg
    H, KVH, HD, B = cfg["H"], cfg["KVH"], cfg["HD"], w.B
    worst = 0.0
    row = KVH * HD
    for layer in layers:
        slots, window, layout = w.specs[layer]
        w.reset_positions()
        w.ctx_of(layer).append_decode_attention(w.q[layer], w.kn[layer], w.vn[layer], w.k[layer], w.v[layer],
                                                w.out[layer], w.d_pos, w.scale)
        status = w.ctx_of(layer).device_status()
        assert status == 0, f"device status word {status}"
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


def time_graph(torch, w: Workload, steps, warmup, sampler=None, barrier=None):
    """The engine's own contract: the whole step captured ONCE, then replayed while only the device
    positions change (src/engine.cpp:151-269 of the reference). Returns the per-step times (ms)."""
    w.reset_positions()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
            w.step_device()
        for _ in range(warmup):
            graph.replay()
        w.reset_positions()
        side.synchronize()
        if barrier:
            barrier()
        if sampler:
            sampler.begin()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record(side)
        for i in range(steps):
            graph.replay()
            evs[i + 1].record(side)
        side.synchronize()
        if barrier:
            barrier()
        if sampler:
            sampler.end()
    torch.cuda.current_stream().wait_stream(side)
    per_step = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return per_step, evs[0].elapsed_time(evs[steps]), graph, side


def decode_record(torch, hkv, oracle, name, cfg, ctx, B, steps, warmup, verify_layers, note=None):
    """A compact, parity-checked record of one decode workload under graph replay."""
    w = Workload(torch, hkv, cfg, ctx, B, 0)
    L = cfg["layers"]
    err = verify(w, oracle, layers=verify_layers, seqs=sorted({0, B - 1}))
    per_step, total, graph, side = time_graph(torch, w, steps, warmup)
    assert w.device_status() == 0
    st = step_stats(per_step)
    alg = float(np.mean([w.algorithmic_bytes_per_layer(s) for s in range(steps)])) * L
    gbs = alg / (st["ms_per_step_median"] * 1e-3) / 1e9
    footprint = sum(t.numel() * 2 for t in w.k) * 2
    rec = {"workload": name, "batch": B, "ctx": ctx, "layers": L, "value": B / (st["ms_per_step_median"] / 1e3),
           "unit": "tokens/s", **st, "hbm_gbs_step": gbs, "hbm_frac_of_8TBs_step": gbs / 8000.0,
           "parity_max_abs_err": err, "kernel": "tma" if w.hctx.kernel == 2 else "generic",
           "l2": "cache planes of %.2f GB, all read every step" % (footprint / 1e9) if footprint > 4 * (126 << 20)
                 else "cache planes of %.1f MB stay L2-resident: a latency figure, not a bandwidth one" % (footprint / 1e6)}
    if note:
        rec["note"] = note
    del graph
    w.close()
    del w
    gc.collect()
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------
# prefill and rope figures
# ---------------------------------------------------------------------------
def measured_peak(key, fallback):
    peaks_path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))[key]), f"measured (MEASURED_PEAKS.json {key})"
    return fallback, "fallback"


def prefill_record(args, torch, hkv, oracle, cfg, name, S, past, steps, warmup, gpu_id=None, window=0, ring_slots=0,
                   attend_first=False):
    """Chunked prefill over the cache (batch 1, one layer per call): append the chunk's K/V,
    then attention of its S queries over rows [0, past + S). Tensor-bound:
    flops = 4*H*HD*sum_q(attended rows of q). `attend_first`: the one-call form for a ring of exactly
    `window` rows (hkv_prefill_append_attention: attends the cached rows and the chunk's own rows, then
    appends)."""
    H, KVH, HD = cfg["H"], cfg["KVH"], cfg["HD"]
    ring = ring_slots > 0
    slots = ring_slots if ring else past + S
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
                                   window_size=window, layout=1 if ring else 0,
                                   kernel_select=args.kernel, max_seq_new=S if S <= 4096 else 0))
    scale = 1.0 / math.sqrt(HD)

    def step():
        if attend_first:
            ctx.prefill_append_attention(q, kn, vn, k, v, out, S, past, scale)
        else:
            ctx.append_at(kn, vn, k, v, past, S)
            ctx.prefill_attention(q, k, v, out, S, past, scale)

    before = (k.cpu().numpy(), v.cpu().numpy()) if attend_first and not args.no_verify else None
    step()
    assert ctx.device_status() == 0
    err = None
    if not args.no_verify:  # sampled queries against the oracle (linear planes + window mask semantics)
        hq = q.cpu().numpy()
        if attend_first:   # the ring as it was BEFORE the call held positions [past - slots, past); then the chunk
            hk = np.zeros((past + S, KVH, HD), np.float16); hv = np.zeros_like(hk)
            pos = np.arange(max(0, past - slots), past)
            hk[pos], hv[pos] = before[0][pos % slots], before[1][pos % slots]
            hk[past:], hv[past:] = kn.cpu().numpy(), vn.cpu().numpy()
        elif ring:    # logical view of the ring: position p lives in row p % slots
            first = max(0, past + S - slots)
            pos = np.arange(first, past + S)
            hk = np.zeros((past + S, KVH, HD), np.float16); hv = np.zeros_like(hk)
            hk[pos], hv[pos] = k.cpu().numpy()[pos % slots], v.cpu().numpy()[pos % slots]
        else:
            hk, hv = k.cpu().numpy(), v.cpu().numpy()
        got = out.cpu().numpy()
        err = 0.0
        for lo in (0, S // 2, S - 4):
            ref = oracle.prefill(hq, hk, hv, past, scale, window=window, q_begin=lo, q_end=lo + 4,
                                 threads=oracle.hardware_threads())
            ok, e = oracle.within_tolerance(got[lo:lo + 4], ref[lo:lo + 4])
            assert ok, f"prefill parity failed at query {lo}: {e:.3e}"
            err = max(err, e)
    sampler = ClockSampler(gpu_id) if gpu_id else None
    if sampler:
        sampler.start()
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if sampler:
        sampler.begin()
    evs = []
    for _ in range(steps):
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        if attend_first:   # one call: both passes, the merge and the append
            a.record(); b.record(); ctx.prefill_append_attention(q, kn, vn, k, v, out, S, past, scale)
        else:
            a.record(); ctx.append_at(kn, vn, k, v, past, S)
            b.record(); ctx.prefill_attention(q, k, v, out, S, past, scale)
        c.record(); evs.append((a, b, c))
    torch.cuda.synchronize()
    clocks = None
    if sampler:
        sampler.end()
        sampler.extend(lambda: (step(), torch.cuda.synchronize()))
        clocks = sampler.stop()
    tot = step_stats([a.elapsed_time(c) for a, b, c in evs])
    attn = step_stats([b.elapsed_time(c) for a, b, c in evs])
    attended = [min(past + i + 1, window) if window else past + i + 1 for i in range(S)]
    flops = 4.0 * H * HD * sum(attended)
    peak, peak_src = measured_peak("bf16_tflops", 1590.0)
    achieved = flops / (attn["ms_per_step_median"] * 1e-3) / 1e12
    plan = ctx.plan_prefill(S, past)
    rec = {"workload": f"{name}-shaped chunked prefill over the cache: chunk {S} queries, {past} rows already cached, "
                       f"{H}q/{KVH}kv heads, head_dim {HD}" + (f", window {window}" if window else "") +
                       (f", ring plane of {slots} rows" if ring else "") +
                       (", attend-then-append in one call (hkv_prefill_append_attention)" if attend_first else "") +
                       ", one layer per step, batch 1",
           "chunk": S, "past_len": past, "value": S / (tot["ms_per_step_median"] * 1e-3), "unit": "tokens/s", **tot,
           "attention_ms_median": attn["ms_per_step_median"], "attention_ms_min": attn["ms_per_step_min"],
           "roofline": {"bound": "tensor", "kernel": "tcgen05 prefill (hkv_prefill_tc*_kernel)" if plan[0]
                        else "hkv_prefill_generic_kernel (SIMT)",
                        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "peak_source": peak_src + " burst bf16 GEMM", "traffic": None,
                        "algorithmic_flops_per_launch": flops, "avg_launch_ms": attn["ms_per_step"]},
           "l2": "K/V planes of %.0f MB, re-read per query tile" % (slots * KVH * HD * 4 / 1e6),
           "parity_max_abs_err": err}
    rec["plan"] = {"tiles_in_flight": plan[0], "items": plan[1], "key_splits": plan[2]}
    if clocks is not None:
        rec["clocks"] = clocks
    ctx.close()
    return rec


def prefill_sequence_record(args, torch, hkv, oracle, dist, cfg, name, total_tokens, chunk, rank, world):
    """The long-context config's prefill as stated: every GPU prefills ONE sequence of `total_tokens`
    tokens (sequences sharded by batch, no collective) in chunks of `chunk` queries through all layers:
    per chunk and layer, append the chunk's K/V rows, then attention of its queries over the cache so
    far. One pass is timed (seconds of GPU work); max over ranks."""
    L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
    dev = "cuda"
    k = torch.zeros((L, total_tokens, KVH, HD), dtype=torch.float16, device=dev)
    v = torch.zeros((L, total_tokens, KVH, HD), dtype=torch.float16, device=dev)
    q = torch.empty((chunk, H, HD), dtype=torch.float16, device=dev)
    kn = torch.empty((chunk, KVH, HD), dtype=torch.float16, device=dev)
    vn = torch.empty((chunk, KVH, HD), dtype=torch.float16, device=dev)
    out = torch.zeros((chunk, H, HD), dtype=torch.float16, device=dev)
    seeds = [SEED ^ 0xF11 ^ (rank * 0x10001) ^ (i << 20) for i in range(3)]
    for t, sd in zip((q, kn, vn), seeds):
        hkv.fill_synthetic(t, sd)
    ctx = hkv.Context(hkv.Geometry(batch=1, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=total_tokens,
                                   kernel_select=args.kernel, max_seq_new=chunk))
    scale = 1.0 / math.sqrt(HD)
    n_chunks = total_tokens // chunk

    def one_pass(layers):
        for c in range(n_chunks):
            for l in layers:
                ctx.append_at(kn, vn, k[l], v[l], c * chunk, chunk)
                ctx.prefill_attention(q, k[l], v[l], out, chunk, c * chunk, scale)

    one_pass([0])                      # warm-up on one layer (also fills its plane)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    one_pass(range(L))
    e1.record()
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    err = None
    if rank == 0 and not args.no_verify:
        # the last chunk of the last layer, four queries, against the oracle: every chunk wrote the same
        # rows, so the plane is the chunk's K/V repeated
        hkn, hvn = oracle.fill(seeds[1], 0, chunk * KVH * HD).reshape(chunk, KVH, HD), oracle.fill(seeds[2], 0, chunk * KVH * HD).reshape(chunk, KVH, HD)
        hk, hv = np.tile(hkn, (n_chunks, 1, 1)), np.tile(hvn, (n_chunks, 1, 1))
        hq = oracle.fill(seeds[0], 0, chunk * H * HD).reshape(chunk, H, HD)
        past = (n_chunks - 1) * chunk
        ref = oracle.prefill(hq, hk, hv, past, scale, q_begin=chunk - 4, q_end=chunk, threads=oracle.hardware_threads())
        ok, err = oracle.within_tolerance(out[chunk - 4:].cpu().numpy(), ref[chunk - 4:])
        assert ok, f"full-sequence prefill parity failed: {err:.3e}"
    flops = 4.0 * H * HD * (total_tokens * (total_tokens + 1) / 2.0) * L
    peak, peak_src = measured_peak("bf16_tflops_sustained", 1400.0)
    ach = flops / (ms * 1e-3) / 1e12
    rec = {"workload": f"{name}-shaped prefill of {world} sequence(s) of {total_tokens} tokens, one per GPU, in chunks of "
                       f"{chunk} queries through {L} layers (append + attention over the cache per chunk and layer)",
           "n_gpus": world, "value": world * total_tokens / (ms * 1e-3), "unit": "tokens/s", "seconds_per_sequence": ms / 1e3,
           "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                        "peak_source": peak_src + " (a seconds-long run: the sustained figure)",
                        "algorithmic_flops": flops},
           "gpu_launches": n_chunks * L * 2, "parity_max_abs_err": err}
    ctx.close()
    del k, v
    gc.collect()
    torch.cuda.empty_cache()
    return rec if rank == 0 else None


def rope_record(args, torch, hkv, oracle, cfg, name, B, S, slots, steps, warmup):
    """The step in front of the append: per-head RMSNorm of q and k + rotary embedding with K and V
    written straight into the cache (hkv_qk_norm_rope_kv). HBM-bound:
    bytes = q in + q out + k in + v in + K row out + V row out (+ two weight rows)."""
    H, KVH, HD = cfg["H"], cfg["KVH"], cfg["HD"]
    dev = "cuda"
    q = torch.empty((B, S, H, HD), dtype=torch.float16, device=dev)
    k = torch.empty((B, S, KVH, HD), dtype=torch.float16, device=dev)
    v = torch.empty((B, S, KVH, HD), dtype=torch.float16, device=dev)
    kc = torch.zeros((B, slots, KVH, HD), dtype=torch.float16, device=dev)
    vc = torch.zeros((B, slots, KVH, HD), dtype=torch.float16, device=dev)
    qw = torch.empty((HD,), dtype=torch.float16, device=dev)
    kw = torch.empty((HD,), dtype=torch.float16, device=dev)
    for i, t in enumerate((q, k, v, qw, kw)):
        hkv.fill_synthetic(t, SEED ^ ((i + 9) << 20))
    q0 = q.clone()
    pos = torch.from_numpy(np.arange(B, dtype=np.int32) * 3 + 5).to(dev)
    ctx = hkv.Context(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=slots,
                                   flags=hkv.FLAG_APPEND_ONLY))
    err = None
    if not args.no_verify:   # one sequence against the oracle
        ctx.qk_norm_rope_kv(q, k, v, qw, kw, kc, vc, pos, 0, S, 0, 1e-6, 10000.0, 1.0)
        torch.cuda.synchronize()
        b = B - 1
        hq, hk, hv = q0[b:b + 1].cpu().numpy().copy(), k[b:b + 1].cpu().numpy().copy(), v[b:b + 1].cpu().numpy()
        rk = np.zeros((1, slots, KVH, HD), np.float16); rv = np.zeros_like(rk)
        oracle.qk_norm_rope(hq, hk, hv, qw.cpu().numpy(), kw.cpu().numpy(), np.array([int(pos[b])], np.int32),
                            k_cache=rk, v_cache=rv, eps=1e-6, theta=10000.0)
        ok, err = oracle.within_tolerance(q[b:b + 1].cpu().numpy().reshape(-1, HD), hq.reshape(-1, HD))
        assert ok, f"rope parity (q) failed: {err:.3e}"
        ok, e2 = oracle.within_tolerance(kc[b:b + 1].cpu().numpy().reshape(-1, HD), rk.reshape(-1, HD))
        assert ok, f"rope parity (K rows in the cache) failed: {e2:.3e}"
        assert np.array_equal(vc[b:b + 1].cpu().numpy().view(np.uint16), rv.view(np.uint16)), "V rows not bit-exact"
        err = max(err, e2)
        q.copy_(q0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than L2

    def step():
        flush.zero_()
        ctx.qk_norm_rope_kv(q, k, v, qw, kw, kc, vc, pos, 0, S, 0, 1e-6, 10000.0, 1.0)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush.zero_()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); ctx.qk_norm_rope_kv(q, k, v, qw, kw, kc, vc, pos, 0, S, 0, 1e-6, 10000.0, 1.0); b_.record()
        evs.append((a, b_))
    torch.cuda.synchronize()
    st = step_stats([a.elapsed_time(b_) for a, b_ in evs])
    # the same launch warm and back to back, as it runs inside a decode loop: 20 launches captured as one graph
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
            for _ in range(20):
                ctx.qk_norm_rope_kv(q, k, v, qw, kw, kc, vc, pos, 0, S, 0, 1e-6, 10000.0, 1.0)
        graph.replay()
        side.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(side)
        for _ in range(5):
            graph.replay()
        g1.record(side)
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    warm_ms = g0.elapsed_time(g1) / 100.0
    alg = B * S * (2 * H * HD + 4 * KVH * HD) * 2 + 4 * HD
    peak, peak_src = measured_peak("hbm_gbs", 6650.0)
    achieved = alg / (st["ms_per_step_median"] * 1e-3) / 1e9
    rec = {"workload": f"{name}-shaped fused per-head RMSNorm + RoPE + K/V cache write: batch {B}, {S} new tokens per "
                       f"sequence, {H}q/{KVH}kv heads, head_dim {HD}", "value": B * S / (st["ms_per_step_median"] * 1e-3),
           "unit": "tokens/s", **st,
           "roofline": {"bound": "hbm", "kernel": "hkv_qk_norm_rope_kernel", "achieved": achieved, "peak": peak,
                        "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "traffic": None,
                        "algorithmic_bytes_per_launch": alg},
           "l2": "256 MB written between timed launches (L2 flush)", "parity_max_abs_err": err,
           "warm_back_to_back_ms": warm_ms,
           "warm_note": "100 launches replayed from a graph, inputs resident in L2 where they fit: the launch as a decode "
                        "loop sees it; the cold figure above pays instruction, constant and TLB misses after the flush"}
    ctx.close()
    return rec


# ---------------------------------------------------------------------------
# sequence split (C++ host: libhkv_dist)
# ---------------------------------------------------------------------------
def seqsplit_leg(args, torch, hkv, oracle, dist, cfg, logical_ctx, B, rank, world, gpu_id, steps, warmup, label):
    """One logical cache of `logical_ctx` rows per sequence, dealt block-cyclically over the ranks.
    Per layer: local split-K decode with the append fused in -> one partial per (sequence, head) to every
    rank (stored into the ranks' mailboxes over NVLink by the kernel that merges the local partials; or an
    NCCL all-gather, timed beside it) -> merge; all layers captured once as a CUDA graph by the C++ decoder
    and replayed. Output replicated on all ranks. Returns the record (rank 0) or None."""
    L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
    shard = hkv.dist.SeqShard(rank, world, args.shard_block)
    ctx_local = shard.slots_for(logical_ctx)
    assert ctx_local * world == logical_ctx, "logical context must be a multiple of world * shard block"
    dev = "cuda"
    row = KVH * HD
    k = torch.empty((L, B, ctx_local, KVH, HD), dtype=torch.float16, device=dev)
    v = torch.empty((L, B, ctx_local, KVH, HD), dtype=torch.float16, device=dev)
    q = torch.empty((L, B, H, HD), dtype=torch.float16, device=dev)
    kn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
    vn = torch.empty((L, B, KVH, HD), dtype=torch.float16, device=dev)
    out = torch.zeros((L, B, H, HD), dtype=torch.float16, device=dev)
    plane_seed = lambda i, r: SEED ^ 0x5E9 ^ (r * 0x10001) ^ (i << 20)
    for i, t in enumerate((k, v)):
        hkv.fill_synthetic(t, plane_seed(i, rank))
    rep_seed = lambda i: SEED ^ 0x5E9 ^ ((i + 2) << 20)
    for i, t in enumerate((q, kn, vn)):      # replicated inputs: same seed on every rank
        hkv.fill_synthetic(t, rep_seed(i))
    pos0 = np.random.default_rng(SEED).integers(logical_ctx // 2, logical_ctx, size=B).astype(np.int32)
    h_tot = torch.from_numpy(pos0 + 1).pin_memory()
    stream = torch.cuda.Stream()
    scale = 1.0 / math.sqrt(HD)
    d_tot = torch.from_numpy(pos0 + 1).to(dev)
    torch.cuda.synchronize()
    # NCCL announces its version on stdout when a communicator is first created (with NCCL_DEBUG set):
    # stdout carries the one JSON line, so the descriptor points at stderr while the decoder is built
    def make_decoder(exchange):
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            d = hkv.dist.SeqSplitDecoder(hkv.Geometry(batch=B, num_heads=H, num_kv_heads=KVH, head_dim=HD, slots=ctx_local,
                                                      kernel_select=args.kernel, chunk_tiles=args.chunk_tiles),
                                         shard, layers=L, scale=scale, stream=stream, exchange=exchange)
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
        d.bind(q, kn, vn, out, k, v, B * ctx_local * row, d_tot)
        return d

    dec = make_decoder(args.exchange)
    exchange = dec.exchange if world > 1 else "none"

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def agree(n):   # minimum over the ranks
        if dist is None:
            return n
        t = torch.tensor([n], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t.item())

    def step():
        with torch.cuda.stream(stream):
            dec.step()
            d_tot.add_(1).clamp_(max=logical_ctx)

    # ---- parity: one un-captured step at the start positions, sampled (layer, sequence) pairs vs the oracle
    err = None
    with torch.cuda.stream(stream):
        dec.step(eager=True)
    dec.wait(60000)
    assert dec.device_status() == 0
    if rank == 0 and not args.no_verify:
        err = 0.0
        layer = L // 2
        for b in sorted({0, B - 1}):
            total = int(pos0[b]) + 1
            hk = np.empty((total, KVH, HD), np.float16); hv = np.empty_like(hk)
            for r in range(world):     # regenerate rank r's rows of (layer, b) from its seed, deal them back
                sh = hkv.dist.SeqShard(r, world, args.shard_block)
                n = sh.local_rows(total)
                first = ((layer * B + b) * ctx_local) * row
                lk = oracle.fill(plane_seed(0, r) & 0xFFFFFFFFFFFFFFFF, first, n * row).reshape(n, KVH, HD)
                lv = oracle.fill(plane_seed(1, r) & 0xFFFFFFFFFFFFFFFF, first, n * row).reshape(n, KVH, HD)
                for lb in range(0, n, args.shard_block):
                    p0 = ((lb // args.shard_block) * world + r) * args.shard_block
                    m = min(args.shard_block, n - lb)
                    hk[p0:p0 + m], hv[p0:p0 + m] = lk[lb:lb + m], lv[lb:lb + m]
            nb = (layer * B + b) * row
            hk[total - 1] = oracle.fill(rep_seed(1), nb, row).reshape(KVH, HD)
            hv[total - 1] = oracle.fill(rep_seed(2), nb, row).reshape(KVH, HD)
            hq = oracle.fill(rep_seed(0), (layer * B + b) * H * HD, H * HD).reshape(1, H, HD)
            ref = oracle.decode(hq, hk[None], hv[None], [total], scale, threads=oracle.hardware_threads())
            ok, e = oracle.within_tolerance(out[layer, b].cpu().numpy(), ref[0])
            assert ok, f"sequence-split parity failed at layer {layer} seq {b}: max abs err {e:.3e}"
            assert float(np.abs(ref[0].astype(np.float32)).max()) > 0.0, "the oracle's output is all zero: nothing was checked"
            err = max(err, e)
    barrier()

    sampler = ClockSampler(gpu_id)
    sampler.start()
    for _ in range(max(warmup, 2)):     # the second call captures the graph
        step()
    with torch.cuda.stream(stream):
        d_tot.copy_(h_tot, non_blocking=True)
    barrier()
    sampler.begin()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record(stream)
    for i in range(steps):
        step()
        evs[i + 1].record(stream)
    dec.wait(120000)
    barrier()
    sampler.end()
    per_step = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    ms = torch.tensor([evs[0].elapsed_time(evs[steps])], device=dev)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / steps
    sampler.extend(lambda: ([step() for _ in range(4)], dec.wait(120000)), agree=agree if dist is not None else None)
    clocks = sampler.stop()
    # the all-gather's share: events around every phase of every layer, a few un-captured steps
    prof = []
    for _ in range(3):
        with torch.cuda.stream(stream):
            prof.append(dec.step_profiled())
    barrier()
    assert dec.device_status() == 0
    dms, gms, cms = (float(np.median([p[i] for p in prof])) / L for i in range(3))
    # the same step with the other exchange (the collective), timed the same way, for comparison
    other = None
    if world > 1 and exchange == "peer":
        dec.close()
        dec = make_decoder("nccl")
        with torch.cuda.stream(stream):
            d_tot.copy_(h_tot, non_blocking=True)
        for _ in range(max(warmup, 2)):
            step()
        with torch.cuda.stream(stream):
            d_tot.copy_(h_tot, non_blocking=True)
        barrier()
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev2[0].record(stream)
        for i in range(steps):
            step()
        ev2[1].record(stream)
        dec.wait(120000)
        barrier()
        ms2 = torch.tensor([ev2[0].elapsed_time(ev2[1])], device=dev)
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        prof2 = []
        for _ in range(3):
            with torch.cuda.stream(stream):
                prof2.append(dec.step_profiled())
        barrier()
        other = {"exchange": "nccl all-gather", "ms_per_step": float(ms2.item()) / steps,
                 "value": B / (float(ms2.item()) / steps / 1e3),
                 "decode_ms_per_layer": float(np.median([p[0] for p in prof2])) / L,
                 "allgather_ms_per_layer": float(np.median([p[1] for p in prof2])) / L,
                 "combine_ms_per_layer": float(np.median([p[2] for p in prof2])) / L}
    Ls = np.stack([np.minimum(pos0 + 1 + s, logical_ctx) for s in range(steps)]).astype(np.int64)
    # algorithmic bytes over ALL ranks: the K/V rows of every sequence once, + the new row once, + q/out per rank
    alg = float((4 * Ls * KVH * HD).sum(axis=1).mean() + B * 8 * KVH * HD + world * B * 4 * H * HD) * L
    rec = None
    if rank == 0:
        st = step_stats(per_step)
        rec = {"label": label, "workload": f"qwen2-7b-shaped long-context decode: {L} layers, logical ctx {logical_ctx} "
                                           f"dealt block-cyclically ({args.shard_block}) over {world} GPU(s) = {ctx_local} rows "
                                           f"per GPU, batch {B}",
               "parallelism": f"sequence-split x{world}" + (
                   " (no exchange)" if world == 1 else
                   f", {B * H * (HD + 2) * 4} B per rank per layer stored into every rank's mailbox over NVLink by the kernel "
                   "that merges the local partials; bounded flag wait in the final merge; no collective launch"
                   if exchange == "peer" else f", NCCL all-gather of {B * H * (HD + 2) * 4} B per rank per layer"),
               "exchange": exchange,
               "host": "C++ (libhkv_dist): all layers captured once as a CUDA graph on the compute stream",
               "n_gpus": world, "batch": B, "ctx": logical_ctx, "rows_per_gpu": ctx_local, "scaling": "strong",
               "value": B / (ms_per_step / 1e3), "unit": "tokens/s", "ms_per_step": ms_per_step,
               "ms_per_step_median_rank0": st["ms_per_step_median"], "ms_per_step_min_rank0": st["ms_per_step_min"],
               "hbm_gbs_step": alg / (ms_per_step * 1e-3) / 1e9,
               "hbm_gbs_per_gpu": alg / world / (ms_per_step * 1e-3) / 1e9,
               "hbm_frac_of_8TBs_per_gpu": alg / world / (ms_per_step * 1e-3) / 1e9 / 8000.0,
               "decode_ms_per_layer": dms, "allgather_ms_per_layer": gms, "combine_ms_per_layer": cms,
               "phases": ("decode = split-K kernel + local merge that pushes; combine = flag wait + final merge"
                          if exchange == "peer" else "decode = split-K kernel + local merge; all-gather; combine = final merge"),
               "with_nccl_allgather": other,
               "parity_max_abs_err": err, "clocks": clocks, "gpu_launches": steps * L * 3}
    dec.close()
    del k, v, q, kn, vn, out, dec
    gc.collect()
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------
# reference arm: the reference's own kernels rebuilt for sm_100a (GPU only). This arm never
# imports this repository's package: tensors come from torch, kernels from oracle/_ref.
# ---------------------------------------------------------------------------
def reference_main(args):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rank != 0:
        return 0  # the reference has no multi-GPU path: rank 0 alone measures it
    import torch
    import hkv_oracle as oracle    # loader of oracle/_ref (and of the CPU port, not used here)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the reference's path is GPU-only)")
    torch.cuda.set_device(local)
    ref = oracle.load_reference()
    if ref is None:
        emit(({"impl": "reference", "unavailable":
                          "oracle/_ref/libhector_ref_attention.so not built (reference checkout absent at build time)"}))
        return 0
    cfg = dict(WORKLOADS[args.workload])
    if args.layers:
        cfg["layers"] = args.layers
    ctx = args.ctx or cfg.get("ctx", 32768)
    L, H, KVH, HD = cfg["layers"], cfg["H"], cfg["KVH"], cfg["HD"]
    gpu_id = gpu_uuid(torch, local)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(HD)
    # n_gpus echoes the launch; the reference has no multi-GPU path, so rank 0 alone runs it on one GPU
    base = {"unit": "tokens/s", "n_gpus": max(1, args.gpus), "gpus_used": 1, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 storage / fp32 accumulate",
            "data": "synthetic", "impl": "reference"}
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    normal = lambda *shape: torch.empty(shape, dtype=torch.float16, device="cuda").normal_(generator=gen)

    if args.mode == "prefill":
        # The reference's attention_prefill_cached kernel (kernels/attention.cu:664-788): one CTA per
        # (query, head), each streaming its whole key range, so time is additive over queries: three
        # slices of 32 queries (start, middle, end of the chunk) are timed and scaled to the chunk.
        S, past = args.chunk, args.past
        slots = past + S
        k, v, q = normal(slots, KVH, HD), normal(slots, KVH, HD), normal(S, H, HD)
        n = min(32, S)
        los = sorted({0, max(0, S // 2 - n // 2), S - n})
        rout = torch.zeros((n, H, HD), dtype=torch.float16, device="cuda")

        def ref_slice(lo):
            st = ref.hector_ref_attention_prefill_cached(q[lo:].data_ptr(), k.data_ptr(), v.data_ptr(), rout.data_ptr(), n,
                                                         past + lo, H, KVH, HD, slots, scale, 0, stream)
            assert st == 0, f"reference prefill kernel failed: {st}"

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
        sampler.extend(lambda: (ref_slice(los[-1]), torch.cuda.synchronize()))
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / args.steps * (S / float(n * len(los)))
        flops = 4.0 * H * HD * sum(past + i + 1 for i in range(S))
        val = S / (ms * 1e-3)
        sample = (f"the reference's attention_prefill_cached kernel rebuilt for sm_100a, run on the GPU: {len(los)} slices "
                  f"of {n} queries of the chunk per step, time scaled to {S} queries (one CTA per (query, head): additive)")
        emit((dict(base, metric="prefill attention tokens/s (one layer)", mode="prefill",
                              config={"workload": f"{args.workload}-shaped chunked prefill over the cache: chunk {S} queries, "
                                                  f"{past} rows already cached, {H}q/{KVH}kv heads, head_dim {HD}, one layer "
                                                  f"per step, batch 1", "chunk": S, "past_len": past},
                              value=val, ms_per_step=ms, extrapolated=True, queries_timed=n * len(los), clocks=clocks,
                              gpu_launches=args.steps * len(los), tflops=flops / (ms * 1e-3) / 1e12,
                              e2e={"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                              cpu_baseline={"value": val, "unit": "tokens/s", "cores": 0, "kind": "reference",
                                            "sample": sample})))
        return 0

    per_seq = 2 * L * ctx * KVH * HD * 2
    free, _ = torch.cuda.mem_get_info()
    B = args.batch or cfg.get("batch") or next(b for b in (64, 32, 8, 1) if b * per_seq + (6 << 30) < free)
    specs = layer_specs(cfg, ctx, linear_window=True)    # the reference has no ring layout: linear plane + mask
    k = [normal(B, ctx, KVH, HD) for _ in range(L)]
    v = [normal(B, ctx, KVH, HD) for _ in range(L)]
    q, kn, vn = normal(L, B, H, HD), normal(L, B, KVH, HD), normal(L, B, KVH, HD)
    out = torch.zeros((L, B, H, HD), dtype=torch.float16, device="cuda")
    pos0 = start_positions(cfg, ctx, B, 0)
    h_pos = torch.from_numpy(pos0.copy())
    d_pos = h_pos.to("cuda")
    d_total = (d_pos + 1).contiguous()
    torch.cuda.synchronize()

    def advance():
        d_pos.add_(1).clamp_(max=ctx - 1)
        torch.add(d_pos, 1, out=d_total)

    def reset(values=None):
        d_pos.copy_(h_pos if values is None else values)
        torch.add(d_pos, 1, out=d_total)

    def step_per_sequence(st=None):
        # The reference op is batch 1 with one scalar device position
        # (kernels/register_kernels.cpp:870): one launch pair per sequence, serially.
        s = stream if st is None else st
        for l in range(L):
            for b in range(B):
                ref.hector_ref_kv_cache_update_dp(kn[l, b].data_ptr(), vn[l, b].data_ptr(), k[l][b].data_ptr(),
                                                  v[l][b].data_ptr(), 1, 1, KVH, HD, ctx, d_pos.data_ptr() + 4 * b, s)
                ref.hector_ref_attention_cached_dp(q[l, b].data_ptr(), k[l][b].data_ptr(), v[l][b].data_ptr(),
                                                   out[l, b].data_ptr(), 1, d_total.data_ptr() + 4 * b, H, KVH, HD, ctx,
                                                   scale, specs[l][1], s)
        advance()

    def step_batched(st=None):
        # Upper bound the engine itself never reaches: its launchers do take a batch
        # (kernels/attention.cu:496-510, :1153-1170) but read ONE position for all of it, so the
        # whole batch sits at a common position (element 0 of the arrays).
        s = stream if st is None else st
        for l in range(L):
            ref.hector_ref_kv_cache_update_dp(kn[l].data_ptr(), vn[l].data_ptr(), k[l].data_ptr(), v[l].data_ptr(), B, 1,
                                              KVH, HD, ctx, d_pos.data_ptr(), s)
            ref.hector_ref_attention_cached_dp(q[l].data_ptr(), k[l].data_ptr(), v[l].data_ptr(), out[l].data_ptr(), B,
                                               d_total.data_ptr(), H, KVH, HD, ctx, scale, specs[l][1], s)
        advance()

    def step_batch1(st=None):
        s = stream if st is None else st
        for l in range(L):
            ref.hector_ref_kv_cache_update_dp(kn[l, 0].data_ptr(), vn[l, 0].data_ptr(), k[l][0].data_ptr(),
                                              v[l][0].data_ptr(), 1, 1, KVH, HD, ctx, d_pos.data_ptr(), s)
            ref.hector_ref_attention_cached_dp(q[l, 0].data_ptr(), k[l][0].data_ptr(), v[l][0].data_ptr(),
                                               out[l, 0].data_ptr(), 1, d_total.data_ptr(), H, KVH, HD, ctx, scale,
                                               specs[l][1], s)
        advance()

    def timed(step_fn, steps, warmup, sampler=None):
        for _ in range(warmup):
            step_fn()
        torch.cuda.synchronize()
        if sampler:
            sampler.begin()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record()
        for i in range(steps):
            step_fn()
            evs[i + 1].record()
        torch.cuda.synchronize()
        if sampler:
            sampler.end()
        return [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]

    sampler = ClockSampler(gpu_id)
    sampler.start()
    reset()
    main_stats = step_stats(timed(step_per_sequence, args.steps, args.warmup, sampler))
    clocks = sampler.stop()
    tok_s = B / (main_stats["ms_per_step"] / 1e3)

    # upper bound: one batched launch pair per layer, every sequence at the mean position
    common = torch.full((B,), int(pos0.astype(np.int64).mean()), dtype=torch.int32)
    reset(common)
    bat = step_stats(timed(step_batched, args.steps, args.warmup))
    # the engine's own mode: batch 1, the whole step captured once as a CUDA graph and replayed
    reset()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step_batch1(side.cuda_stream)          # first token un-captured, as the engine does
        with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
            step_batch1(side.cuda_stream)
        for _ in range(args.warmup):
            graph.replay()
        side.synchronize()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        evs[0].record(side)
        for i in range(args.steps):
            graph.replay()
            evs[i + 1].record(side)
        side.synchronize()
    b1 = step_stats([evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)])

    workload_name = (f"{args.workload}-shaped decode: {L} layers, {H}q/{KVH}kv heads, head_dim {HD}, ctx {ctx}, "
                     f"batch {B} per GPU, cache_pos ~ U[ctx/2, ctx)")
    config = {"workload": workload_name, "batch_per_gpu": B, "global_batch": B, "ctx": ctx, "layers": L,
              "parallelism": "batch-sharded x1 (no data-path collective)",
              "l2": "inputs larger than L2 (K/V read per step >> 126 MB)", "fp16_kv": True}
    sample = (f"the reference's own attention.cu + kv_cache_update kernels rebuilt for sm_100a, run on the GPU (the "
              f"reference has no CPU implementation of this path): all {L} layers per step, one launch pair per sequence "
              f"as its batch-1 op does")
    line = dict(base, metric="decode attn+KV-append tokens/s", config=config, value=tok_s, **main_stats, clocks=clocks,
                layers_timed=L, extrapolated=False, gpu_launches=args.steps * L * B * 2,
                e2e={"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                cpu_baseline={"value": tok_s, "unit": "tokens/s", "cores": 0, "kind": "reference", "sample": sample},
                reference_batched={"value": B / (bat["ms_per_step"] / 1e3), "unit": "tokens/s", **bat,
                                   "note": "upper bound the engine never reaches: ONE batched launch pair per layer with "
                                           "the whole batch at a common position (the mean of the workload's positions); "
                                           "the reference op itself is batch 1 (kernels/register_kernels.cpp:870)"},
                reference_batch1_graph={"value": 1.0 / (b1["ms_per_step"] / 1e3), "unit": "tokens/s", **b1,
                                        "note": "the engine's own mode: batch 1, all layers captured once as a CUDA graph "
                                                "and replayed (sequence 0 of the workload)"})
    emit((line))
    return 0


# ---------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_main(args)
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path exists)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    hkv = importlib.import_module("hector-engine_b200")
    hkv._capi.load()  # fail loudly if the native library is missing
    import hkv_oracle as oracle

    cfg = dict(WORKLOADS[args.workload])
    if args.layers:
        cfg["layers"] = args.layers
    ctx = args.ctx or cfg.get("ctx", 32768)
    n_gpus = world
    gpu_id = gpu_uuid(torch, local)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def finish(rc=0):
        if dist is not None:
            dist.destroy_process_group()
        return rc

    base = {"metric": "decode attn+KV-append tokens/s", "unit": "tokens/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 storage / fp32 accumulate", "data": "synthetic", "impl": "hkv"}

    # ------------------------------------------------------------------ single-kernel modes
    if args.mode == "prefill":
        if rank == 0:
            rec = prefill_record(args, torch, hkv, oracle, cfg, args.workload, args.chunk, args.past, args.steps, args.warmup,
                                 gpu_id, window=0)
            emit((dict(base, metric="prefill attention tokens/s (one layer)", mode="prefill", n_gpus=1,
                                  config={"workload": rec.pop("workload"), "chunk": rec.pop("chunk"),
                                          "past_len": rec.pop("past_len"), "l2": rec.pop("l2")},
                                  gpu_launches=args.steps * 2, e2e=None, cpu_baseline=None, **rec)))
        return finish()
    if args.mode == "rope":
        if rank == 0:
            B = args.batch or 1
            rec = rope_record(args, torch, hkv, oracle, cfg, args.workload, B, args.chunk, max(args.chunk + 64, 4096),
                              args.steps, args.warmup)
            emit((dict(base, metric="fused qk-norm + rope + KV write tokens/s (one layer)", mode="rope", n_gpus=1,
                                  config={"workload": rec.pop("workload"), "l2": rec.pop("l2")},
                                  gpu_launches=args.steps, e2e=None, cpu_baseline=None, **rec)))
        return finish()
    if args.mode == "seqsplit":
        B = args.batch or 64
        rec = seqsplit_leg(args, torch, hkv, oracle, dist, cfg, ctx, B, rank, n_gpus, gpu_id, args.steps, args.warmup,
                           "requested")
        if rank == 0:
            emit((dict(base, mode="seqsplit", scaling="strong",
                                  config={"workload": rec["workload"], "parallelism": rec["parallelism"], "ctx": ctx,
                                          "global_batch": B, "l2": "inputs larger than L2"},
                                  value=rec["value"], ms_per_step=rec["ms_per_step"], clocks=rec["clocks"],
                                  gpu_launches=rec["gpu_launches"], e2e=None, roofline=None, cpu_baseline=None,
                                  seqsplit=[rec])))
        return finish()

    # ------------------------------------------------------------------ batch mode (the headline)
    B = pick_batch(torch, cfg, ctx, args.batch)
    workload_name = (f"{args.workload}-shaped decode: {cfg['layers']} layers, {cfg['H']}q/{cfg['KVH']}kv heads, "
                     f"head_dim {cfg['HD']}, ctx {ctx}, batch {B} per GPU, cache_pos ~ U[ctx/2, ctx)")
    config = {"workload": workload_name, "batch_per_gpu": B, "global_batch": B * n_gpus, "ctx": ctx,
              "layers": cfg["layers"], "parallelism": f"batch-sharded x{n_gpus} (no data-path collective)",
              "l2": "inputs larger than L2 (K/V read per step >> 126 MB)", "fp16_kv": True,
              "timing": "the whole step captured once as a CUDA graph and replayed (the engine's execution mode); "
                        "CUDA events on the replay stream, max over ranks"}
    w = Workload(torch, hkv, cfg, ctx, B, rank, args.kernel, args.chunk_tiles, args.linear_window, args.tma_groups,
                 args.ring_extra)
    L = cfg["layers"]
    verify_err = None
    if not args.no_verify:
        verify_err = verify(w, oracle, layers=sorted({0, L // 2, L - 1}), seqs=sorted({0, B // 2, B - 1}))

    # ---- the timed region: K graph replays
    sampler = ClockSampler(gpu_id)
    sampler.start()
    per_step, total_ms, graph, side = time_graph(torch, w, args.steps, max(args.warmup, 3), sampler, barrier)
    sampler.extend(lambda: (graph.replay(), torch.cuda.synchronize()))   # no collective inside: each rank on its own
    clocks = sampler.stop()
    ms = torch.tensor([total_ms], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    stats = step_stats(per_step)
    tok_s = B * n_gpus / (ms_per_step / 1e3)
    del graph

    # ---- the same step issued call by call (one C-ABI call per layer from Python)
    w.reset_positions()
    for _ in range(2):
        w.step_device()
    w.reset_positions()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        w.step_device()
    e1.record()
    barrier()
    eager_ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(eager_ms, op=dist.ReduceOp.MAX)
    eager_ms = float(eager_ms.item()) / args.steps

    # ---- per-kernel durations, in a pass of their own (events between the kernels of every layer)
    w.reset_positions()
    for c in w.ctxs.values():
        c.profile_begin(args.steps * L)
    for _ in range(args.steps):
        w.step_device()
    dec_ms = comb_ms = 0.0
    calls = 0
    for c in w.ctxs.values():
        d_, m_, n_ = c.profile_end()
        dec_ms, comb_ms, calls = dec_ms + d_, comb_ms + m_, calls + n_
    status = w.device_status()
    assert status == 0, f"device status word {status}"

    alg_bytes = float(np.mean([w.algorithmic_bytes_per_layer(s) for s in range(args.steps)]))
    peak, peak_src = measured_peak("hbm_gbs", 6650.0)
    dec_avg_ms = dec_ms / max(calls, 1)
    achieved = alg_bytes / (dec_avg_ms * 1e-3) / 1e9
    traffic = DRAM_BYTES_PER_ALGORITHMIC_BYTE * alg_bytes if w.hctx.kernel == 2 else None
    roofline = {"bound": "hbm", "kernel": "hkv_decode_tma_kernel" if w.hctx.kernel == 2 else "hkv_decode_generic_kernel",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_8TBs": achieved / 8000.0, "peak_source": peak_src, "traffic": traffic,
                "algorithmic_bytes_per_launch": alg_bytes, "avg_launch_ms": dec_avg_ms,
                "combine_avg_ms": comb_ms / max(calls, 1), "launches_timed": calls}
    step_gbs = alg_bytes * L / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point
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
            for l in range(L):   # copies on the context's copy streams, overlapping the neighbouring layers' kernels
                w.ctx_of(l).append_decode_attention_host_pipelined(hq[l], hk[l], hv[l], w.k[l], w.v[l], ho[l], w.d_pos, w.scale)
            for c in w.contexts():
                c.host_flush()
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
               "call": "hkv_append_decode_attention_host_pipelined per layer + hkv_host_flush per step (pinned host q/k/v/out; "
                       "copies on the context's copy streams overlap the neighbouring layers' kernels)",
               "h2d_bytes_per_step": int(L * (B * H * HD + 2 * B * KVH * HD) * 2 + B * 4),
               "d2h_bytes_per_step": int(L * B * H * HD * 2)}
        del hq, hk, hv, ho

    cpu = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w, oracle)

    launches_per_decode = w.hctx.launches_per_decode
    kernel_is_tma = w.hctx.kernel == 2
    w.close()
    del w
    gc.collect()
    torch.cuda.empty_cache()

    # ---- extras (1 GPU): the other configs and batch sizes, prefill, rope
    extras = None
    default_workload = args.workload == "qwen2-7b" and not args.ctx and not args.batch and not args.layers
    if n_gpus == 1 and default_workload and not args.no_extras:
        q7 = WORKLOADS["qwen2-7b"]
        extras = {"decode": [], "note": "graph replay, 20 steps after 5; value = batch / median step time"}
        def guarded(fn, *a, **kw):
            try:
                return fn(*a, **kw)
            except Exception as e:   # an extra record must not take the headline line down with it
                gc.collect()
                torch.cuda.empty_cache()
                return {"workload": str(a[4] if fn is decode_record else a[5]), "error": f"{type(e).__name__}: {e}"}
        for name, c, cx, b, layers in (
                ("qwen2-0.5b single layer, append at 511 (config 1)", WORKLOADS["qwen2-0.5b"], 2048, 1, [0]),
                ("phi3-mini MHA head_dim 96 (config 3)", WORKLOADS["phi3-mini"], 4096, 16, [0, 31]),
                ("gemma local/global head_dim 256, ring planes (config 4)", WORKLOADS["gemma-local-global"], 32768, 8, [0, 5]),
                ("qwen2-7b ctx 32768 batch 8", q7, 32768, 8, [13]),
                ("qwen2-7b ctx 32768 batch 1 (the engine's own batch)", q7, 32768, 1, [13]),
                ("qwen2-7b ctx 4096 batch 64", q7, 4096, 64, [13]),
                ("qwen2-7b ctx 4096 batch 1", q7, 4096, 1, [13])):
            extras["decode"].append(guarded(decode_record, torch, hkv, oracle, name, dict(c), cx, b, 20, 5, layers))
        extras["prefill"] = [
            guarded(prefill_record, args, torch, hkv, oracle, q7, "qwen2-7b", 2048, 30720, 10, 3),
            guarded(prefill_record, args, torch, hkv, oracle, q7, "qwen2-7b", 2048, 0, 10, 3),
            guarded(prefill_record, args, torch, hkv, oracle, WORKLOADS["phi3-mini"], "phi3-mini", 2048, 2048, 10, 3),
            guarded(prefill_record, args, torch, hkv, oracle, WORKLOADS["gemma-local-global"], "gemma-local-global", 2048, 30720, 10, 3),
            guarded(prefill_record, args, torch, hkv, oracle, WORKLOADS["gemma-local-global"], "gemma-local-global (local layer)",
                           512, 30720, 10, 3, window=1024, ring_slots=2048),
            guarded(prefill_record, args, torch, hkv, oracle, WORKLOADS["gemma-local-global"], "gemma-local-global (local layer)",
                           512, 30720, 10, 3, window=1024, ring_slots=1024, attend_first=True),
        ]
        extras["rope"] = [guarded(rope_record, args, torch, hkv, oracle, q7, "qwen2-7b", 64, 1, 4096, 20, 5),
                          guarded(rope_record, args, torch, hkv, oracle, q7, "qwen2-7b", 1, 2048, 4096, 20, 5)]
        gc.collect()
        torch.cuda.empty_cache()

    # ---- sequence split: strong scaling of batch 64 / ctx 32768; on 8 GPUs also the 131072-token decode
    seqsplit = None
    if default_workload and not args.no_seqsplit:
        seqsplit = []
        legs = [("strong scaling: batch 64, logical ctx 32768", 32768)]
        if n_gpus == 8:
            legs.append(("long-context config: batch 64, logical ctx 131072 over 8 GPUs", 131072))
        for label, logical in legs:
            # a leg that fails (on every rank alike: e.g. out of memory) must not take the headline line with it
            try:
                rec = seqsplit_leg(args, torch, hkv, oracle, dist, cfg, logical, B, rank, n_gpus, gpu_id, args.steps,
                                   max(args.warmup, 3), label)
            except Exception as exc:   # noqa: BLE001 - reported in the record
                rec = {"label": label, "error": f"{type(exc).__name__}: {exc}"[:400]}
                gc.collect()
                torch.cuda.empty_cache()
            if rank == 0:
                seqsplit.append(rec)

    # ---- the long-context config's prefill: one 131 072-token sequence per GPU, 2 048-query chunks
    prefill_seq = None
    if default_workload and not args.no_extras:
        try:
            prefill_seq = prefill_sequence_record(args, torch, hkv, oracle, dist, cfg, args.workload, 131072, 2048, rank, n_gpus)
        except Exception as exc:   # noqa: BLE001 - reported in the record
            prefill_seq = {"error": f"{type(exc).__name__}: {exc}"[:400]}
            gc.collect()
            torch.cuda.empty_cache()

    if rank == 0:
        line = dict(base, config=config, value=tok_s, ms_per_step=ms_per_step,
                    ms_per_step_median=stats["ms_per_step_median"], ms_per_step_min=stats["ms_per_step_min"],
                    clocks=clocks, e2e=e2e, gpu_launches=args.steps * L * launches_per_decode, roofline=roofline,
                    cpu_baseline=cpu, hbm_gbs_step=step_gbs, hbm_frac_of_8TBs_step=step_gbs / 8000.0,
                    parity_max_abs_err=verify_err,
                    eager={"ms_per_step": eager_ms, "value": B * n_gpus / (eager_ms / 1e3), "unit": "tokens/s",
                           "note": "the same step as one C-ABI call per layer from Python, no graph"})
        if extras is not None:
            line["extras"] = extras
        if seqsplit:
            line["seqsplit"] = seqsplit
        if prefill_seq is not None:
            line["prefill_sequences"] = prefill_seq
        emit((line))
    return finish()


if __name__ == "__main__":
    claim_stdout()
    sys.exit(main())
