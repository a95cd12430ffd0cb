#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c1|c2|c3|c4|c5]

Without --workload one JSON line carries the whole metric ("attn decode KV GB/s + prefill attn TFLOP/s"):

  headline  config 2, the 35B-MoE decode attention layer — 16 q / 2 kv heads, head_dim 256, partial RoPE (64 dims,
            theta 1e7), sigmoid gate, 32768-token f16 KV context, one new token — for the model's 10 attention layers.
            A step is one decode token through those layers: RoPE + KV append + split-K decode + merge + gate per
            layer, each layer with its own caches (10 x 67 MB: no layer's K/V survives in the 126 MB L2 until its next
            use).  With N > 1 (one process per GPU) every rank holds a 32768-row chunk of an N x 32768-token context and
            the ranks merge their (m, l, o) records over NVLink (weak scaling; N = 1 is exactly config 2).
  "check"   before anything is timed: one layer step on small seeded inputs in the run's own shard layout (4096 rows
            per rank, all N ranks, the same exchange), the single-sequence and the batched path, and a small prefill
            on this rank's kv-head group, each against the float64 CPU oracle; the run fails outside max-abs 2e-3 /
            max-rel 1e-2 or when the appended row differs in any bit.
  "prefill" config 3: causal prefill of an 8192-token prompt, 24 q / 4 kv heads, head_dim 256, kv-head groups dealt to
            the ranks (N = 1, 2, 4), TFLOP/s of the causal half.
  "c5"      config 5: 8 sequences x 131072-token context, KV sequence sharded over the N ranks (strong scaling).

With --workload the named configuration alone is the line (profiling captures use this with --layers / --ctx / --cols).

value    whole-job throughput with inputs resident in HBM: CUDA events around K steps, the region repeated until
         0.5 s have been timed; median region, max over ranks
e2e      the same metric through the host-buffer C-ABI call (pinned host q/k/v/gate in, out back, every step)
roofline the dominant kernel alone: algorithmic bytes (flops) per launch / its CUDA-event duration, against the
         measured peaks of MEASURED_PEAKS.json
Inputs are seeded synthetic tensors (N(0,1) -> f16, config 2 with 4 outlier channels per head x20): the reference
measures on chat prompts through real weights, which do not exist here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c1": dict(nH=16, nKV=8, hd=128, n_rot=128, theta=1e6, ctx=4096, n_cols=1, n_seqs=1, layers=28, gate=False, outliers=False,
               desc="config 1: Qwen3-1.7B-shaped decode attention, 16q/8kv hd128 full RoPE, ctx 4096, 28 layers"),
    "c2": dict(nH=16, nKV=2, hd=256, n_rot=64, theta=1e7, ctx=32768, n_cols=1, n_seqs=1, layers=10, gate=True, outliers=True,
               desc="config 2: Qwen3.6-35B-MoE-shaped decode attention, 16q/2kv hd256 partial RoPE 64, gate, ctx 32768, 10 attention layers"),
    "c4": dict(nH=24, nKV=4, hd=256, n_rot=64, theta=1e7, ctx=16384, n_cols=5, n_seqs=1, layers=16, gate=True, outliers=False,
               desc="config 4: 27B-hybrid-shaped 5-token verify block, 24q/4kv hd256, ctx 16384, 16 attention layers"),
    "c3": dict(nH=24, nKV=4, hd=256, n_rot=64, theta=1e7, ctx=0, n_cols=8192, n_seqs=1, layers=4, gate=False, outliers=False,
               desc="config 3: 27B-hybrid-shaped causal prefill, 8192-token prompt into an empty cache, 24q/4kv hd256 partial RoPE 64, 4 layers per step"),
    "c5": dict(nH=16, nKV=2, hd=256, n_rot=64, theta=1e7, ctx=131072, n_cols=1, n_seqs=8, layers=2, gate=True, outliers=False,
               desc="config 5: 8 sequences x 131072-token context, 16q/2kv hd256, gate, KV sequence sharded across the GPUs (strong scaling), 2 layers"),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures summarised
# under profiles/ (same per-launch shape as the bench's; the captures only use fewer layers)
CAPTURED_TRAFFIC = {"c2": 67.36e6 + 0.74e6, "c4": 67.35e6 + 1.27e6}
MIN_TIMED_S = 0.5


def peaks(key="hbm_gbs", fallback=6650.0):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p[key]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return fallback, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region (a read-only query)."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


class Run:
    """Process-wide state: rank layout, device, torch.distributed."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0")); self.world = int(os.environ.get("WORLD_SIZE", "1")); self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def min_over_ranks(self, x: float) -> float:
        return -self.max_over_ranks(-x)

    def timed(self, run_step, steps: int, min_total_s: float | None = None, max_regions: int = 2000):
        """Regions of exactly `steps` steps, each bracketed by barrier + synchronize and timed with CUDA events (max over
        ranks), repeated until min_total_s have been timed.  Returns the per-region milliseconds."""
        torch = self.torch
        # shorter regions (core kernel, end to end) scale with the main one
        min_total_s = self.args.min_time if min_total_s is None else min_total_s * self.args.min_time / MIN_TIMED_S
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        regions, total = [], 0.0
        while True:
            self.barrier()
            e0.record()
            for _ in range(steps):
                run_step()
            e1.record()
            self.barrier()
            ms = self.max_over_ranks(e0.elapsed_time(e1))
            regions.append(ms); total += ms
            if total >= min_total_s * 1e3 or len(regions) >= max_regions:
                return regions

    def close(self):
        if self.world > 1:
            self.dist.barrier(); self.dist.destroy_process_group()


def _spread(regions, steps):
    med = statistics.median(regions)
    return med, {"repeats": len(regions), "ms_per_step_min": round(min(regions) / steps, 5), "ms_per_step_max": round(max(regions) / steps, 5),
                 "timed_s": round(sum(regions) / 1e3, 3)}


def decode_config(args, w, world):
    """The `config` object of a decode line: a function of the arguments only, so both arms print the same one."""
    strong = w["n_seqs"] > 1
    chunk = (w["ctx"] // world) if strong else w["ctx"]
    total_ctx = w["ctx"] if strong else w["ctx"] * world
    rows = chunk if world > 1 else w["ctx"] + w["n_cols"]
    kernel_bytes = 2 * rows * w["nKV"] * w["hd"] * 2 * w["n_seqs"]
    return {"workload": w["desc"], "kv_rows_per_gpu": chunk, "total_context": total_ctx, "layers_per_step": w["layers"],
            "l2": "each layer has its own caches; a step touches %d MB per GPU, more than the 126 MB L2, before any row is reused" % (w["layers"] * kernel_bytes // 1_000_000),
            "launch": "CUDA graph replay of the step" if (args.graph and (world == 1 or args.exchange == "peer")) else "eager C-ABI calls",
            "exchange": (args.exchange if world > 1 else None)}


# ------------------------------------------------------------------------------------------------ decode --

def run_decode(R: Run, w, headline: bool):
    """Decode / verify workloads (c1, c2, c4: one sequence, weak scaling over ranks; c5: 8 sequences, strong scaling)."""
    torch, dist, args = R.torch, R.dist, R.args
    from pooled_b200 import AttnConfig, AttnEngine
    from pooled_b200.shard import ShardPlan, ShardedDecoder
    rank, world, dev = R.rank, R.world, R.dev
    nH, nKV, hd, ctx, n_cols, n_seqs, layers = w["nH"], w["nKV"], w["hd"], w["ctx"], w["n_cols"], w["n_seqs"], w["layers"]
    qd, kvd = nH * hd, nKV * hd
    strong = n_seqs > 1
    sharded = world > 1
    chunk = (ctx // world) if strong else ctx          # rows each rank holds per sequence
    total_ctx = ctx if strong else ctx * world
    max_seq = chunk if sharded else chunk + 64         # a shard's cache is exactly its chunk
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=w["n_rot"], rope_theta=w["theta"], max_seq=max_seq, n_layers=layers,
                                n_seqs=n_seqs, act_dtype=torch.float16, max_cols=max(8, n_cols * n_seqs)), device=R.local)
    g = torch.Generator(device=dev); g.manual_seed(1234 + rank)
    for li in range(layers):
        for name in ("k", "v"):
            c = eng.cache(li, name)
            for s in range(n_seqs):
                x = torch.randn((max_seq, kvd), generator=g, device=dev, dtype=torch.float32)
                if w["outliers"] and name == "k":
                    x.view(max_seq, nKV, hd)[..., :4] *= 20.0
                c[s].copy_(x.to(torch.float16).view(torch.int16))
                del x
    T = n_cols * n_seqs
    gh = torch.Generator(); gh.manual_seed(99)
    mk = lambda n: torch.randn((layers, T, n), generator=gh).to(torch.float16)
    hq, hk, hv, hg = mk(qd), mk(kvd), mk(kvd), mk(qd)
    if w["outliers"]:
        hq.view(layers, T, nH, hd)[..., :4] *= 20.0
    hq, hk, hv, hg = (t.pin_memory() for t in (hq, hk, hv, hg))
    hout = torch.empty((layers, T, qd), dtype=torch.float16).pin_memory()
    dq, dk, dv, dg = (t.to(dev) for t in (hq, hk, hv, hg))
    dout = torch.empty((layers, T, qd), dtype=torch.float16, device=dev)
    gate = (lambda t, li: t[li]) if w["gate"] else (lambda t, li: None)

    if sharded:
        plan = ShardPlan(world, chunk)
        if args.exchange == "peer":
            eng.exchange_setup(rank, world, dist, max_rows=max(64, T * nH))
        sd = ShardedDecoder(eng, plan, rank, dist, exchange=args.exchange)
        gbuf = torch.empty((world, T * nH * (hd + 2)), dtype=torch.float32, device=dev)
        new_pos = total_ctx - 1   # the new token is the last row of the last rank's chunk
        seqs_pos = [(s, new_pos) for s in range(n_seqs)]

        def step():
            for li in range(layers):
                sd.step(li, seqs_pos, dq[li], dk[li], dv[li], gate(dg, li), dout[li], gbuf)
        bytes_per_layer_rank = [2 * min(chunk, max(0, new_pos + 1 - r * chunk)) * kvd * 2 * n_seqs for r in range(world)]
        bytes_per_step = layers * sum(bytes_per_layer_rank)
        kernel_bytes = bytes_per_layer_rank[rank]
    else:
        pos = ctx   # the cache holds rows [0, ctx); the new tokens land at ctx .. ctx + n_cols - 1
        if n_seqs == 1:
            def step():
                for li in range(layers):
                    eng.encode_layer(li, pos, dq[li], dk[li], dv[li], gate(dg, li), dout[li], mode="decode")
        else:
            items = [(s, pos, 1) for s in range(n_seqs)]

            sp = [(s, pos) for s in range(n_seqs)]

            def step():
                for li in range(layers):
                    eng.encode_items(li, sp, dq[li], dk[li], dv[li], gate(dg, li), dout[li])   # all sequences, one call per layer
        kernel_bytes = 2 * (pos + n_cols) * kvd * 2 * n_seqs
        bytes_per_step = layers * kernel_bytes

    for _ in range(max(args.warmup, 3)):
        step()
    R.barrier()
    # launch mode of the timed region: the step captured once into a CUDA graph and replayed (what pooled does with its
    # pre-encoded per-token command buffers, engine/qwen35.js:4004-4009), or eager C-ABI calls (--no-graph)
    launches_per_step = None
    run_step, graph = step, None
    if args.graph and (not sharded or args.exchange == "peer"):   # NCCL inside a captured step is left to eager launches
        cs = torch.cuda.Stream(device=dev)
        cs.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(cs):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=cs):
                s1 = eng.stats()
                step()
                launches_per_step = eng.stats()["kernel_launches"] - s1["kernel_launches"]
        torch.cuda.current_stream(dev).wait_stream(cs)
        run_step = graph.replay
        for _ in range(3):
            run_step()
    R.barrier()
    clocks = ClockSampler(R.local).start()
    st0 = eng.stats()
    regions = R.timed(run_step, args.steps)
    st1 = eng.stats()
    ms, spread = _spread(regions, args.steps)
    n_launch = launches_per_step * args.steps if launches_per_step is not None else (st1["kernel_launches"] - st0["kernel_launches"]) // len(regions)
    value = bytes_per_step * args.steps / (ms * 1e-3) / 1e9

    # The dominant kernel alone.  Single-sequence steps: the same K steps with only the core kernel of every layer
    # launched (a CUDA graph of `layers` core launches), back to back, between one CUDA-event pair (a pair around each
    # 10-20 us launch would time the launch gap as well); on a shard that leaves the cross-GPU exchange out, as it leaves
    # the merge out, so the figure is the streaming kernel's own.  Batched steps: an event pair around every core launch.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if n_seqs == 1 and (not sharded or args.exchange == "peer"):
        eng.set_core_only(True)
        cs2 = torch.cuda.Stream(device=dev)
        cs2.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(cs2):
            step()
            core_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(core_graph, stream=cs2):     # host launch cost (~15 us per eager call) would hide a 10 us kernel
                step()
        torch.cuda.current_stream(dev).wait_stream(cs2)
        for _ in range(3):
            core_graph.replay()
        core_regions = R.timed(core_graph.replay, args.steps, min_total_s=0.2)
        core_ms, core_n = statistics.median(core_regions), layers * args.steps
        eng.set_core_only(False)
        step()
    else:
        eng.set_core_only(True)      # no merge, no exchange: the launch's duration is the streaming kernel's own
        eng.timing_begin(layers * args.steps + 8)
        for _ in range(args.steps):
            step()
        core_ms, core_n = eng.timing_end()
        eng.set_core_only(False)
        step()
    eng.sync()

    # end to end: host buffers in, host result out, every step
    if not sharded and n_seqs == 1:
        # one C-ABI call per token step: pinned host q/k/v/gate of all layers up, the layers back to back, out down
        host_step = lambda: eng.encode_step_host(ctx, hq, hk, hv, hg if w["gate"] else None, hout, mode="decode")
        h2d = layers * T * (qd + 2 * kvd + (qd if w["gate"] else 0)) * 2
        call = "pa_attn_step_host (one upload per array, all layers, one download, stream drained) per step"
    else:
        # sharded / batched steps: the same step with a pinned-host upload of its inputs and a download of its result
        def host_step():
            dq.copy_(hq, non_blocking=True); dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True); dg.copy_(hg, non_blocking=True)
            step()
            hout.copy_(dout, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
        h2d = int(hq.numel() + hk.numel() + hv.numel() + hg.numel()) * 2 * world
        call = "pinned-host upload of q/k/v/gate, the step's C-ABI calls, download of out, stream drained, per step and rank"
    for _ in range(3):
        host_step()
    eregions = R.timed(host_step, args.steps, min_total_s=0.25)
    ems, espread = _spread(eregions, args.steps)
    e2e = {"value": round(bytes_per_step * args.steps / (ems * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(ems / args.steps, 5),
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(hout.numel()) * 2 * (world if sharded else 1), "call": call, **espread}
    ck = clocks.stop()

    peak, peak_src = peaks()
    achieved = kernel_bytes / (core_ms / max(core_n, 1) * 1e-3) / 1e9 if core_n else None
    verify_tc = n_seqs == 1 and n_cols * (nH // nKV) > 8
    traffic = args.traffic
    if traffic is None and args.ctx <= 0 and world == 1:
        traffic = CAPTURED_TRAFFIC.get(w["key"])
    cfg = decode_config(args, w, world)
    rec = {
        "metric": "attn decode KV GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms / args.steps, 5), **spread, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "f16 cache and activations, f32 accumulate",
        "data": "synthetic (seeded N(0,1) -> f16, outlier channels x20)" if w["outliers"] else "synthetic (seeded N(0,1) -> f16)",
        "config": cfg, "pct_of_8TBs_nominal_per_gpu": round(100 * value / world / 8000, 1),
        "roofline": {"bound": "hbm", "kernel": "pa_prefill_kernel<256,2> (split-K tcgen05 verify)" if verify_tc else "pa_decode_kernel",
                     "achieved": round(achieved, 1) if achieved else None, "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4) if achieved else None, "peak_source": peak_src, "launches_timed": int(core_n),
                     "us_per_launch": round(core_ms / max(core_n, 1) * 1e3, 2), "algorithmic_bytes_per_launch": kernel_bytes, "traffic": traffic},
        "e2e": e2e, "gpu_launches": int(n_launch), "clocks": ck,
    }
    del dq, dk, dv, dg, dout, hq, hk, hv, hg, hout
    eng.destroy()
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------------ prefill --

def run_prefill(R: Run, w):
    """Config 3: tiled causal prefill.  With N > 1 the kv-head groups are dealt to the ranks (no collective: heads
    never interact inside attention); value is the whole job's causal FLOP/s (strong scaling)."""
    torch, args = R.torch, R.args
    from pooled_b200 import AttnConfig, AttnEngine
    rank, world, dev = R.rank, R.world, R.dev
    nH, nKV, hd, T, layers = w["nH"], w["nKV"], w["hd"], w["n_cols"], w["layers"]
    if nKV % world:
        return {"metric": "prefill attn TFLOP/s", "n_gpus": world, "unavailable": f"{nKV} kv-head groups do not divide over {world} GPUs"}
    nH_r, nKV_r = nH // world, nKV // world          # this rank's heads
    qd, kvd = nH_r * hd, nKV_r * hd
    eng = AttnEngine(AttnConfig(n_heads=nH_r, n_kv_heads=nKV_r, head_dim=hd, n_rot=w["n_rot"], rope_theta=w["theta"], max_seq=T, n_layers=layers,
                                act_dtype=torch.float16, max_cols=T), device=R.local)
    gh = torch.Generator(); gh.manual_seed(7 + rank)
    mk = lambda n: torch.randn((T, n), generator=gh).to(torch.float16).pin_memory()
    hq, hk, hv = mk(qd), mk(kvd), mk(kvd)
    hout = torch.empty((T, qd), dtype=torch.float16).pin_memory()
    dq, dk, dv = hq.to(dev), hk.to(dev), hv.to(dev)
    dout = torch.empty((layers, T, qd), dtype=torch.float16, device=dev)

    def step():
        for li in range(layers):
            eng.encode_layer(li, 0, dq, dk, dv, None, dout[li], mode="prefill")

    flops_layer = 4.0 * nH * hd * T * (T + 1) / 2          # whole job, causal half only
    for _ in range(max(args.warmup, 3)):
        step()
    R.barrier()
    clocks = ClockSampler(R.local).start()
    st0 = eng.stats()
    regions = R.timed(step, args.steps)
    st1 = eng.stats()
    ms, spread = _spread(regions, args.steps)
    eng.timing_begin(layers * args.steps + 8)
    for _ in range(args.steps):
        step()
    core_ms, core_n = eng.timing_end()

    def step_host():
        dq.copy_(hq, non_blocking=True); dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True)
        step()
        hout.copy_(dout[layers - 1], non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
    step_host()
    eregions = R.timed(step_host, args.steps, min_total_s=0.25)
    ems, espread = _spread(eregions, args.steps)
    ck = clocks.stop()
    value = flops_layer * layers * args.steps / (ms * 1e-3) / 1e12
    # the burst cuBLAS figure for a short run at full clocks; the sustained one when this run itself sat under the power
    # cap (seconds of back-to-back tensor work settle near 1.2-1.3 GHz on a 1 kW part)
    capped = "sw_power_cap" in (ck.get("reasons") or []) or bool(ck.get("sm_mhz") and ck.get("sm_max_mhz") and ck["sm_mhz"] < 0.85 * ck["sm_max_mhz"])
    peak, src = peaks("bf16_tflops_sustained", 1400.0) if capped else peaks("bf16_tflops", 1590.0)
    src += ", cuBLAS bf16 sustained (this run was power-capped)" if capped else ", cuBLAS bf16 burst"
    ach = flops_layer / world / (core_ms / max(core_n, 1) * 1e-3) / 1e12
    rec = {"metric": "prefill attn TFLOP/s", "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
           "ms_per_step": round(ms / args.steps, 4), **spread, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "f16 operands, f32 accumulate", "data": "synthetic (seeded N(0,1) -> f16)",
           "config": {"workload": w["desc"], "heads_per_gpu": f"{nH_r}q/{nKV_r}kv", "flops": "4*nH*hd*T(T+1)/2 per layer (masked half not credited)",
                      "l2": "q, k, v and out of a layer are 235 MB, more than the 126 MB L2; each layer has its own caches"},
           "pct_of_2250TF_nominal_per_gpu": round(100 * value / world / 2250, 1),
           "roofline": {"bound": "tensor", "kernel": "pa_prefill_kernel<256,0>", "achieved": round(ach, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(ach / peak, 4),
                        "peak_source": src, "launches_timed": int(core_n), "us_per_launch": round(core_ms / max(core_n, 1) * 1e3, 1), "traffic": args.traffic},
           "e2e": {"value": round(flops_layer * layers * args.steps / (ems * 1e-3) / 1e12, 1), "unit": "TFLOP/s", "ms_per_step": round(ems / args.steps, 4),
                   "h2d_bytes_per_step": int(hq.numel() + hk.numel() + hv.numel()) * 2 * world, "d2h_bytes_per_step": int(hout.numel()) * 2 * world, **espread},
           "gpu_launches": int((st1["kernel_launches"] - st0["kernel_launches"]) // len(regions)), "clocks": ck}
    del dq, dk, dv, dout
    eng.destroy()
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------------------ check --

def run_check(R: Run):
    """One layer step on small seeded inputs in the run's own layout, against the float64 CPU oracle (the checker:
    nothing of it is timed).  Three paths: one sequence (the headline's calls), a batch of sequences (config 5's
    calls) and a prefill chunk on this rank's kv-head group (config 3's calls)."""
    import numpy as np
    from oracle import po
    from pooled_b200 import AttnConfig, AttnEngine
    from pooled_b200.shard import ShardPlan, ShardedDecoder
    torch, dist, args = R.torch, R.dist, R.args
    rank, world, dev = R.rank, R.world, R.dev
    MAX_ABS, MAX_REL = 2e-3, 1e-2
    nH, nKV, hd, n_rot, theta = 16, 2, 256, 64, 1e7
    qd, kvd = nH * hd, nKV * hd
    f16v = lambda seed, shape, s=1.0: po.np_h2f(po.np_f16_rne(po.normal(seed, int(np.prod(shape))) * s)).reshape(shape)
    tdev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.float16).to(dev)
    out = {"n_ranks": world, "tolerance": {"max_abs": MAX_ABS, "max_rel": MAX_REL}}
    worst_abs = worst_rel = 0.0
    ok = True

    def errs(got, ref):
        d = np.abs(got.astype(np.float64) - ref)
        return float(d.max()), float(d.max() / max(np.abs(ref).max(), 1e-30))

    def all_ranks_same(t):
        if world == 1:
            return True
        bufs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(bufs, t.contiguous())
        return all(bool(torch.equal(bufs[0].view(torch.int16), b.view(torch.int16))) for b in bufs[1:])

    for name, n_seqs, chunk in (("one_sequence", 1, 4096), ("batched", 8, 1024)):
        total = chunk * world
        pos = total - 1                                   # the new token: last row of the last rank's chunk
        eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=chunk, n_layers=1, n_seqs=n_seqs,
                                    act_dtype=torch.float16, max_cols=max(8, n_seqs)), device=R.local)
        K = [po.np_f16_rne(po.normal(100 + s, total * kvd) * 0.8).reshape(total, kvd) for s in range(n_seqs)]
        V = [po.np_f16_rne(po.normal(200 + s, total * kvd)).reshape(total, kvd) for s in range(n_seqs)]
        lo, hi = rank * chunk, min((rank + 1) * chunk, pos)
        for s in range(n_seqs):
            eng.cache(0, "k")[s, :hi - lo] = torch.from_numpy(K[s][lo:hi].view(np.int16)).to(dev)
            eng.cache(0, "v")[s, :hi - lo] = torch.from_numpy(V[s][lo:hi].view(np.int16)).to(dev)
        q, kn, vn, g = f16v(301, (n_seqs, qd)), f16v(302, (n_seqs, kvd)), f16v(303, (n_seqs, kvd)), f16v(304, (n_seqs, qd))
        dq, dk, dv, dg = tdev(q), tdev(kn), tdev(vn), tdev(g)
        dout = torch.zeros((n_seqs, qd), dtype=torch.float16, device=dev)
        seqs_pos = [(s, pos) for s in range(n_seqs)]
        rec = {}
        if world > 1:
            if args.exchange == "peer":
                eng.exchange_setup(rank, world, dist, max_rows=max(64, n_seqs * nH))
            sd = ShardedDecoder(eng, ShardPlan(world, chunk), rank, dist, exchange=args.exchange)
            sd.step(0, seqs_pos, dq, dk, dv, dg, dout)
            eng.sync()
            rec["ranks_identical"] = all_ranks_same(dout)
            ok &= rec["ranks_identical"]
            if args.exchange == "peer":
                # the same step through the other exchange (NCCL all-gather of the records + merge kernel)
                dout2 = torch.zeros_like(dout)
                ShardedDecoder(eng, ShardPlan(world, chunk), rank, dist, exchange="nccl").step(0, seqs_pos, dq, dk, dv, dg, dout2)
                eng.sync()
                rec["peer_vs_nccl_max_abs"] = R.max_over_ranks(float((dout.float() - dout2.float()).abs().max()))
                ok &= rec["peer_vs_nccl_max_abs"] <= MAX_ABS
        elif n_seqs == 1:
            eng.encode_layer(0, pos, dq, dk, dv, dg, dout, mode="decode")
        else:
            q_rot = eng.rope_append_items(0, seqs_pos, dq, dk, dv)
            eng.decode(0, [(s, pos, 1) for s in range(n_seqs)], q_rot, dg, dout)
        eng.sync()
        got = dout.float().cpu().numpy()
        bit_exact = True
        ma = mr = 0.0
        for s in range(n_seqs):
            k_row = po.f16_rne(po.rope_neox_f64(kn[s], nKV, hd, n_rot, pos, theta)); v_row = po.f16_rne(vn[s])
            if rank == world - 1:                          # the owner of the new position
                gk = eng.cache(0, "k")[s, pos - lo].cpu().numpy().view(np.uint16); gv = eng.cache(0, "v")[s, pos - lo].cpu().numpy().view(np.uint16)
                bit_exact &= bool(np.array_equal(gk, k_row) and np.array_equal(gv, v_row))
            if rank == 0 and (s == 0 or s == n_seqs - 1):  # the oracle on the first and the last sequence
                Kf = np.concatenate([K[s][:pos], k_row[None]]); Vf = np.concatenate([V[s][:pos], v_row[None]])
                ref = po.attn_f64(po.rope_neox_f64(q[s], nH, hd, n_rot, pos, theta)[None], Kf, Vf, nH, nKV, hd, pos, 1, g[s][None])
                a, r = errs(got[s][None], ref)
                ma, mr = max(ma, a), max(mr, r)
        ma, mr = R.max_over_ranks(ma), R.max_over_ranks(mr)
        bit_exact = R.min_over_ranks(1.0 if bit_exact else 0.0) > 0.5
        rec.update({"max_abs": ma, "max_rel": mr, "append_bit_exact": bit_exact, "rows_per_rank": chunk, "sequences": n_seqs})
        ok &= bool(np.isfinite(ma)) and ma <= MAX_ABS and mr <= MAX_REL and bit_exact
        worst_abs, worst_rel = max(worst_abs, ma), max(worst_rel, mr)
        out[name] = rec
        eng.destroy()

    # prefill: 512 columns into an empty cache, this rank's kv-head group (24 q / 4 kv heads over the ranks)
    pH, pKV, T = 24, 4, 512
    if pKV % world == 0:
        hH, hKV = pH // world, pKV // world
        eng = AttnEngine(AttnConfig(n_heads=hH, n_kv_heads=hKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=T, n_layers=1, act_dtype=torch.float16, max_cols=T),
                         device=R.local)
        q, kn, vn = f16v(401 + rank, (T, hH * hd)), f16v(501 + rank, (T, hKV * hd)), f16v(601 + rank, (T, hKV * hd))
        dout = eng.encode_layer(0, 0, tdev(q), tdev(kn), tdev(vn), None, mode="prefill")
        eng.sync()
        got = dout.float().cpu().numpy()
        Kf = np.stack([po.f16_rne(po.rope_neox_f64(kn[c], hKV, hd, n_rot, c, theta)) for c in range(T)]); Vf = po.f16_rne(vn)
        gk = eng.cache(0, "k")[0, :T].cpu().numpy().view(np.uint16)
        bit_exact = bool(np.array_equal(gk, Kf))
        cols = [0, 1, 63, 64, 127, 128, 300, T - 1]
        ma = mr = 0.0
        for c in cols:
            # q reaches the tensor cores as f16: the oracle sees the same rounded rotated q
            qr = po.np_h2f(po.np_f16_rne(po.rope_neox_f64(q[c], hH, hd, n_rot, c, theta)))
            ref = po.attn_f64(qr[None], Kf, Vf, hH, hKV, hd, c, 1, None)
            a, r = errs(got[c][None], ref)
            ma, mr = max(ma, a), max(mr, r)
        ma, mr = R.max_over_ranks(ma), R.max_over_ranks(mr)
        bit_exact = R.min_over_ranks(1.0 if bit_exact else 0.0) > 0.5
        out["prefill"] = {"max_abs": ma, "max_rel": mr, "append_bit_exact": bit_exact, "columns": T, "columns_checked": len(cols), "heads_per_rank": f"{hH}q/{hKV}kv"}
        ok &= bool(np.isfinite(ma)) and ma <= MAX_ABS and mr <= MAX_REL and bit_exact
        worst_abs, worst_rel = max(worst_abs, ma), max(worst_rel, mr)
        eng.destroy()
    else:
        out["prefill"] = {"unavailable": f"{pKV} kv-head groups do not divide over {world} GPUs"}
    out.update({"max_abs": worst_abs, "max_rel": worst_rel, "append_bit_exact": all(out[k].get("append_bit_exact", True) for k in ("one_sequence", "batched", "prefill")),
                "ok": bool(ok)})
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------ CPU arm --

def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_sample(w, steps: int | None, budget_s: float, warmup: int = 1):
    """The reference's CPU attention (the oracle's threaded f32 restatement of it) on one layer call of one sequence of
    the workload, on every host core this process may use (torchrun's OMP_NUM_THREADS=1 is overridden).  steps = None:
    as many repetitions as fit budget_s."""
    import numpy as np
    from oracle import po
    cores = po.set_threads(host_cores())
    nH, nKV, hd, ctx, n_cols = w["nH"], w["nKV"], w["hd"], w["ctx"], w["n_cols"]
    rows = ctx + n_cols
    K = po.np_f16_rne(po.normal(1, rows * nKV * hd)).reshape(rows, nKV * hd)
    V = po.np_f16_rne(po.normal(2, rows * nKV * hd)).reshape(rows, nKV * hd)
    q = po.normal(3, n_cols * nH * hd).astype(np.float32).reshape(n_cols, nH * hd)
    g = po.normal(4, n_cols * nH * hd).astype(np.float32).reshape(n_cols, nH * hd) if w["gate"] else None
    for _ in range(max(1, warmup)):
        po.attn_f32_fast(q, K, V, nH, nKV, hd, ctx, n_cols, g)
    t0 = time.perf_counter(); reps = 0
    while True:
        po.attn_f32_fast(q, K, V, nH, nKV, hd, ctx, n_cols, g); reps += 1
        if (steps is not None and reps >= steps) or (steps is None and (time.perf_counter() - t0 > budget_s or reps >= 400)):
            break
        if steps is not None and time.perf_counter() - t0 > 240.0:
            break
    dt = (time.perf_counter() - t0) / reps
    nbytes = 2 * rows * nKV * hd * 2
    return {"value": round(nbytes / dt / 1e9, 3), "unit": "GB/s", "cores": cores, "kind": "port", "ms_per_sample": round(dt * 1e3, 2), "reps": reps,
            "sample": f"{reps} repetitions of one layer call of one sequence ({rows} rows x {nKV} kv heads x {hd}), threaded over (column, head, sequence chunk) on {cores} host threads; {dt * 1e3:.1f} ms each"}


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_sample(w, steps=args.steps, budget_s=0.0, warmup=max(1, min(args.warmup, 3)))
    line = {"impl": "reference", "metric": "attn decode KV GB/s", "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": cb["reps"],
            "warmup": args.warmup, "ms_per_step": cb["ms_per_sample"], "higher_is_better": True, "scaling": "strong" if w["n_seqs"] > 1 else "weak", "vs_baseline": None,
            "dtype": "f32 accumulate over an f16 cache", "data": "synthetic (seeded N(0,1) -> f16)", "config": decode_config(args, w, args.gpus),
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "pooled's attention runs only as WGSL through WebGPU, which needs a graphics stack (unavailable on this box), and no "
                    "JavaScript runtime exists here; this arm times the C restatement of its CPU reference attention on the host cores, "
                    "a step being one layer call of one sequence of the workload"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ main --

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS), help="one configuration alone (default: config 2 as the headline with check, prefill and c5 sub-records)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time eager C-ABI calls instead of a CUDA-graph replay of the step")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="sharded decode (N > 1): merge inside the combine kernel over peer memory, or NCCL all-gather + merge kernel")
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count (small profiling captures)")
    ap.add_argument("--ctx", type=int, default=0, help="override the decode workloads' context length (scaling probes)")
    ap.add_argument("--cols", type=int, default=0, help="override the prompt length of the prefill workload (small profiling captures)")
    ap.add_argument("--traffic", type=float, default=None, help="ncu dram bytes per launch of the dominant kernel (default: the committed capture's figure, where one exists for the workload at its full per-launch size)")
    ap.add_argument("--min-time", type=float, default=MIN_TIMED_S, help="seconds each timed region is repeated up to (0: one region; small profiling captures)")
    ap.add_argument("--no-check", dest="check", action="store_false", help="skip the oracle check ahead of the timed regions")
    ap.add_argument("--no-sub", dest="sub", action="store_false", help="headline only: no prefill / c5 sub-records")
    args = ap.parse_args()

    def workload(key):
        w = dict(WORKLOADS[key]); w["key"] = key
        if args.workload is not None:      # overrides apply to an explicitly named workload only
            if args.layers > 0:
                w["layers"] = args.layers
            if args.ctx > 0 and key != "c3":
                w["ctx"] = args.ctx
            if args.cols > 0 and key == "c3":
                w["n_cols"] = args.cols
        return w

    head = workload(args.workload or "c2")
    if args.impl == "reference":
        run_reference(args, head if head["key"] != "c3" else workload("c2"))
        return
    R = Run(args)
    rc = 0
    if args.workload is not None:
        line = run_prefill(R, head) if head["key"] == "c3" else run_decode(R, head, True)
    else:
        check = run_check(R) if args.check else None
        line = run_decode(R, head, True)
        line["check"] = check
        if check is not None and not check["ok"]:
            rc = 3
        if args.sub:
            line["prefill"] = run_prefill(R, workload("c3"))
            line["c5"] = run_decode(R, workload("c5"), False)
    if R.rank == 0:
        if R.world == 1 and head["key"] != "c3":
            line["cpu_baseline"] = cpu_sample(head, steps=None, budget_s=args.cpu_seconds)
        print(json.dumps(line), flush=True)
        if rc:
            print("bench.py: the oracle check failed: " + json.dumps(line.get("check")), file=sys.stderr, flush=True)
    R.close()
    sys.exit(rc)


if __name__ == "__main__":
    main()
