#!/usr/bin/env python
"""Benchmark of the grouped 4-bit MoE expert GEMM: microseconds per MoE layer
(gate_up call + down call), with decode HBM GB/s or prefill TFLOP/s against the roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--config NAME] [--impl reference]

A step is one layer pass over one batch of synthetic tokens: the grouped gate_up GEMM and
the grouped down GEMM of one MoE layer (the GLU between them is not part of the op and is
left out; the down GEMM's input is a fresh bf16 N(0,1) tensor of the right shape).  Every
step uses a different layer out of ``--layers`` resident layer stacks and its own seeded
routing, so weights come from HBM, not from L2.

One JSON line is printed by rank 0:
  value       us/layer with all inputs resident in HBM, K steps captured in one CUDA graph,
              timed with CUDA events (max over ranks)
  e2e         us/layer through the public Python entry points with HOST inputs: pinned
              activations and host routing lists are copied in, the layer output is read back
  roofline    the dominant kernel (gate_up) timed alone: algorithmic bytes or flops / time
  cpu_baseline  the reference project's own CPU kernels (oracle/_ref) on the host cores

``--impl reference`` times only that CPU path with all host threads, same metric and config.
With --gpus N > 1 (under torchrun) the layer is expert-parallel: experts are sharded
across ranks, M tokens per rank are dispatched and combined over NVLink by the library's own
kernels storing into the peers' memory (NCCL all-to-all is the fallback).
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT / "grouped-nf4-gemm_b200"), str(ROOT)):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

import synth  # noqa: E402

BASELINE_US = {  # reference's published B200 numbers (fused Triton, gate_up + down), us/layer
    ("qwen3_30b_a3b", 1): 185.0 + 100.0,       # decode_bs1
    ("qwen3_30b_a3b", 2048): 1428.0 + 794.0,   # prefill_s2048
}
# DRAM traffic of one gate_up launch (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture each, summarised
# with its command under profiles/).  Other workloads: not captured, null.
NCU_TRAFFIC_BYTES = {
    ("qwen3_30b_a3b", 1): 14.22e6,                # = the algorithmic 14.21 MB: nothing re-read
    ("qwen3_30b_a3b", 4096): 360.8e6 + 85.6e6,    # weights once + activations + scales read, output written
}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, smax, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax = max(smax, float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        busy = [v for v in sm if v >= 0.5 * smax] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- workload
def algorithmic(shape, proj, rows, active):
    """Bytes and flops of one grouped call (each distinct expert's weights counted once)."""
    N, K = getattr(shape, proj)
    if shape.fmt == "nf4":
        wbytes = active * N * (K // 2 + (K // 64) * 4)
    else:
        wbytes = active * N * (K // 2 + K // 32)
    return wbytes + 2 * rows * (K + N), 2 * rows * N * K


def workload_config(shape, tokens, layers, n_gpus=1):
    """The `config` object of the JSON line; the same for both arms of a run."""
    if n_gpus > 1:
        layers = max(2, min(layers, 8))        # what the expert-parallel leg keeps resident per rank
    if n_gpus <= 1:
        workload = (f"{shape.name} {shape.fmt} MoE layer, {tokens} tokens per GPU, top-{shape.top_k} of "
                    f"{shape.experts} experts, gate_up {shape.gate_up} + down {shape.down}")
    else:
        workload = (f"{shape.name} {shape.fmt} MoE layer, expert-parallel over {n_gpus} GPUs "
                    f"({shape.experts // n_gpus} experts per GPU), {tokens} tokens per GPU, top-{shape.top_k}, "
                    f"dispatch and combine over NVLink by the library's own stores into peer memory")
    return {"workload": workload, "tokens": tokens, "layers_resident": layers,
            "l2": f"inputs larger than L2: {layers} layer stacks walked round-robin, fresh routing per step",
            "timing": "K steps in one CUDA graph, median over replays, CUDA events (GPU arm); wall clock per layer pass (CPU arm)"}


def make_steps(shape, tokens, n_steps, seed, zipf=None):
    """Per-step routing and host activations (pinned)."""
    gen = torch.Generator().manual_seed(seed)
    steps = []
    for _ in range(n_steps):
        x, idx, w = synth.routed_batch(shape, tokens, gen, zipf)
        tok, sizes, eids, _ = synth.dispatch(idx, shape.experts)
        a_cat = x[tok].contiguous()
        h = torch.randn(a_cat.shape[0], shape.inter, generator=gen).to(torch.bfloat16)
        steps.append(dict(a=a_cat.pin_memory() if torch.cuda.is_available() else a_cat,
                          h=h.pin_memory() if torch.cuda.is_available() else h,
                          sizes=sizes, eids=eids, rows=a_cat.shape[0], active=len(eids)))
    return steps


def build_layers(shape, n_layers, device, seed, random_bytes=False):
    gen = torch.Generator().manual_seed(seed)
    layers = []
    for _ in range(n_layers):
        (n1, k1), (n2, k2) = shape.gate_up, shape.down
        if shape.fmt == "nf4" and random_bytes:
            # profiling aid: uniform random codes and absmax in [0.01, 0.06] instead of quantised
            # N(0, 0.02) weights -- the kernels' timing does not depend on the values
            mk = lambda n, k: (torch.randint(0, 256, (shape.experts, n, k // 2), dtype=torch.uint8, device=device),  # noqa: E731
                               torch.rand(shape.experts, n, k // 64, device=device) * 0.05 + 0.01)
            gu, dn = mk(n1, k1), mk(n2, k2)
        elif shape.fmt == "nf4":
            gu = synth.nf4_stack(shape.experts, n1, k1, gen, device=device, fast=True)
            dn = synth.nf4_stack(shape.experts, n2, k2, gen, device=device, fast=True)
        else:
            gu = synth.mxfp4_stack(shape.experts, n1, k1, gen, device=device, fast=True)
            dn = synth.mxfp4_stack(shape.experts, n2, k2, gen, device=device, fast=True)
        layers.append((gu, dn))
    return layers


def grouped(shape):
    import mxfp4_grouped
    import nf4_grouped
    return nf4_grouped.gemm_4bit_grouped if shape.fmt == "nf4" else mxfp4_grouped.gemm_mxfp4_grouped


# --------------------------------------------------------------------------- CPU arm
def cpu_layers(shape, n_layers, seed):
    """Small random-byte stacks for the CPU arm (its speed does not depend on the values)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n_layers):
        pair = []
        for (n, k) in (shape.gate_up, shape.down):
            W = rng.integers(0, 256, size=(shape.experts, n, k // 2), dtype=np.uint8)
            if shape.fmt == "nf4":
                S = (rng.random(size=(shape.experts, n, k // 64), dtype=np.float32) * 0.05 + 0.01)
            else:
                S = rng.integers(119, 126, size=(shape.experts, n, k // 32), dtype=np.uint8)
            pair.append((W, S))
        out.append(pair)
    return out


def time_cpu(shape, tokens, steps, warmup, seed, max_rows_per_group=None, budget_s=25.0):
    """us/layer of the reference's compiled CPU kernels (oracle/_ref) with all host threads.
    Groups are cut to ``max_rows_per_group`` rows when the full problem would take too long
    and the time is scaled by rows/rows_sampled (flagged in ``sample``)."""
    import numpy as np
    from oracle import oracle as O
    L = O.load_ref()
    kind = "reference"
    if L is None:
        raise RuntimeError("oracle/_ref is not built; run `python oracle/build.py` where the reference checkout is")
    threads = O.host_threads()
    n_layers = min(4, max(2, steps))
    layers = cpu_layers(shape, n_layers, seed)
    st = make_steps(shape, tokens, warmup + steps, seed + 1)
    L.gnf4_pool_start(0)
    times, ffn_times, scale_note = [], [], "full workload"
    ffn_ok = shape.fmt == "nf4" and shape.gate_up[0] == 2 * shape.down[1]
    try:
        for i, s in enumerate(st):
            sizes, eids = list(s["sizes"]), list(s["eids"])
            rows = sum(sizes)
            if max_rows_per_group:
                sizes = [min(v, max_rows_per_group) for v in sizes]
            # the reference's CPU kernels take at most 512 groups per call
            sub_rows = sum(sizes)
            a = np.random.default_rng(i).standard_normal((sub_rows, shape.hidden), dtype=np.float32)
            h = np.random.default_rng(i + 1).standard_normal((sub_rows, shape.inter), dtype=np.float32)
            (Wg, Sg), (Wd, Sd) = layers[i % n_layers]
            t0 = time.perf_counter()
            for c0 in range(0, len(sizes), 512):
                sz, ei = sizes[c0:c0 + 512], eids[c0:c0 + 512]
                r0, r1 = sum(sizes[:c0]), sum(sizes[:c0 + 512])
                O.ref_call("gemv", shape.fmt, a[r0:r1], Wg, Sg, sz, ei, threads=0)
                O.ref_call("gemv", shape.fmt, h[r0:r1], Wd, Sd, sz, ei, threads=0)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt * (rows / max(sub_rows, 1)))
            if ffn_ok and len(sizes) <= 512 and min(sizes) >= 1:
                # the reference's fused FFN entry point (one call per layer), for the e2e_ffn comparison
                t0 = time.perf_counter()
                O.ref_ffn_call(a, Wg, Sg, Wd, Sd, sizes, eids, threads=0)
                if i >= warmup:
                    ffn_times.append((time.perf_counter() - t0) * (rows / max(sub_rows, 1)))
            if sub_rows != rows:
                scale_note = (f"groups cut to <= {max_rows_per_group} rows ({sub_rows} of {rows} rows timed), "
                              f"time extrapolated x rows/rows_timed")
            if sum(times) > budget_s and len(times) >= 3:
                break
    finally:
        L.gnf4_pool_stop()
    us = statistics.median(times) * 1e6
    extra = {"ffn_value": statistics.median(ffn_times) * 1e6} if ffn_times else {}
    return dict(extra, value=us, unit="us/layer", cores=threads, kind=kind,
                sample=f"{len(times)} layer passes, tokens={tokens}, {scale_note}; pool of {threads} threads; "
                       f"variant {L.variant}")


# --------------------------------------------------------------------------- GPU arm
def run_gpu(args, shape, rank, world):
    import nf4_grouped
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    fn = grouped(shape)
    K, W = args.steps, args.warmup
    layers = build_layers(shape, args.layers, dev, seed=1234 + rank, random_bytes=args.random_bytes)
    steps = make_steps(shape, args.tokens, K + W, seed=99 + rank)
    dsteps = []
    for s in steps:
        off = [0]
        for v in s["sizes"]:
            off.append(off[-1] + v)
        dsteps.append(dict(a=s["a"].to(dev), h=s["h"].to(dev),
                           off=torch.tensor(off, dtype=torch.int32, device=dev),
                           eids=torch.tensor(s["eids"], dtype=torch.int32, device=dev),
                           max_rows=max(s["sizes"]) if s["sizes"] else 0))
    torch.cuda.synchronize()

    # the group tables of every step were uploaded during set-up: no kernel of the timed region writes them
    kw = dict(tables_ready=True, path=args.path)

    def layer_resident(i, what="both"):
        (gu, dn), d = layers[i % args.layers], dsteps[i]
        o = None
        if what in ("both", "gate_up"):
            o = fn(d["a"], gu[0], gu[1], None, d["eids"], group_offsets=d["off"], max_rows=d["max_rows"], **kw)
        if what in ("both", "down"):
            o = fn(d["h"], dn[0], dn[1], None, d["eids"], group_offsets=d["off"], max_rows=d["max_rows"], **kw)
        return o

    host_out = {}          # pinned landing buffers for the result, by shape (a fresh pageable one per step
                           # would put its page faults inside the timed region)

    def layer_e2e(i):
        (gu, dn), s = layers[i % args.layers], steps[i]
        a = s["a"].to(dev, non_blocking=True)
        fn(a, gu[0], gu[1], s["sizes"], s["eids"])
        h = s["h"].to(dev, non_blocking=True)
        o = fn(h, dn[0], dn[1], s["sizes"], s["eids"])
        buf = host_out.get(tuple(o.shape))
        if buf is None:
            buf = host_out[tuple(o.shape)] = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
        buf.copy_(o, non_blocking=False)      # device -> host read of the step's result, synchronous
        return buf

    # one bound host-buffer call per resident stack (the stack is checked once, not per step)
    host_runs = [tuple(nf4_grouped.HostGroupedGemm(w, sc, fmt=shape.fmt) for (w, sc) in (gu, dn)) for (gu, dn) in layers]
    for s in steps:                          # host group tables in the form the C entry point takes
        s["sizes_t"] = torch.tensor(s["sizes"], dtype=torch.int32)
        s["eids_t"] = torch.tensor(s["eids"], dtype=torch.int32)

    def pinned_out(rows, cols):
        buf = host_out.get((rows, cols))
        if buf is None:
            buf = host_out[(rows, cols)] = torch.empty(rows, cols, dtype=torch.bfloat16, pin_memory=True)
        return buf

    def layer_e2e_host(i):
        """Both GEMMs through the host-buffer C entry point: host activations and group tables in, host
        result out, each call blocking (the calling convention of the reference's native CPU kernels)."""
        (run_gu, run_dn), s = host_runs[i % args.layers], steps[i]
        run_gu(s["a"], s["sizes_t"], s["eids_t"], pinned_out(s["rows"], shape.gate_up[0]))
        return run_dn(s["h"], s["sizes_t"], s["eids_t"], pinned_out(s["rows"], shape.down[0]))

    host_ffns = ([nf4_grouped.HostGroupedFfn(gu[0], gu[1], dn[0], dn[1], fmt=shape.fmt) for (gu, dn) in layers]
                 if shape.gate_up[0] == 2 * shape.down[1] else None)

    def layer_e2e_ffn(i):
        """The layer as ONE blocking host call: gate_up GEMM, SiLU-GLU, down GEMM (the down input is the
        layer's own intermediate, not the synthetic `h`); one upload, one download, one synchronise."""
        s = steps[i]
        return host_ffns[i % args.layers](s["a"], s["sizes_t"], s["eids_t"], pinned_out(s["rows"], shape.down[0]))

    def time_e2e(step_fn):
        for i in range(W):
            step_fn(i)
        out = []
        for _ in range(max(1, args.repeats // 2)):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(W, W + K):
                step_fn(i)
            e1.record()
            barrier()
            out.append(e0.elapsed_time(e1))
        return out

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    import mxfp4_grouped

    def layer_ffn(i):
        """The layer as the fused expert FFN on device-resident inputs: gate_up, activation and down in one call
        (ONE kernel launch while every group has one row); the down input is the layer's own intermediate."""
        (gu, dn), d = layers[i % args.layers], dsteps[i]
        if shape.fmt == "nf4":
            return nf4_grouped.ffn_4bit_grouped(d["a"], gu[0], gu[1], dn[0], dn[1], None, d["eids"], group_offsets=d["off"],
                                                max_rows=d["max_rows"], tables_ready=True)
        return mxfp4_grouped.ffn_mxfp4_grouped(d["a"], gu[0], gu[1], dn[0], dn[1], None, d["eids"], group_offsets=d["off"],
                                               max_rows=d["max_rows"], tables_ready=True,
                                               act="gpt_oss" if shape.name.startswith("gpt_oss") else "silu")

    ffn_ok = shape.gate_up[0] == 2 * shape.down[1]

    def capture(what):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        step = layer_ffn if what == "ffn" else (lambda i: layer_resident(i, what))
        with torch.cuda.stream(side):
            step(W)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(W, W + K):
                step(i)
        return g

    def timed_replay(g, repeats, min_seconds=0.0):
        """`repeats` timed replays; then more of the same (timed too, at most 500) until `min_seconds` of
        load have passed, so that the 100 ms clock sampler sees the GPU under this load several times."""
        out = []
        t_begin = time.perf_counter()
        while len(out) < repeats or (time.perf_counter() - t_begin < min_seconds and len(out) < 500):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            barrier()
            out.append(e0.elapsed_time(e1))
        return out

    for i in range(W):                       # W untimed warm-up steps
        layer_resident(i)
    g_layer = capture("both")
    g_gu = capture("gate_up")
    g_ffn = capture("ffn") if ffn_ok else None
    g_layer.replay()
    g_gu.replay()
    if g_ffn is not None:
        g_ffn.replay()
    torch.cuda.synchronize()

    with ClockSampler(dev.index) as clk:
        t_layer = timed_replay(g_layer, args.repeats, min_seconds=0.5)
        t_gu = timed_replay(g_gu, args.repeats)
        t_ffn = timed_replay(g_ffn, args.repeats) if g_ffn is not None else None
        # end to end with host inputs and a host result: through the host-buffer C entry point (the
        # headline e2e), and through the tensor entry points with torch doing the copies
        e2e_t = time_e2e(layer_e2e_host)
        e2e_dev_t = time_e2e(layer_e2e)
        e2e_ffn_t = time_e2e(layer_e2e_ffn) if host_ffns else None
        # the same layer the way the reference's own harness times its kernels (and the reference_triton key below):
        # device-resident activations, host routing lists, eager calls, CUDA events around each layer pass
        eager_us = []
        for i in range(W, W + min(K, 60)):
            (gu, dn), s, d = layers[i % args.layers], steps[i], dsteps[i]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(d["a"], gu[0], gu[1], s["sizes"], s["eids"])
            fn(d["h"], dn[0], dn[1], s["sizes"], s["eids"])
            e1.record()
            torch.cuda.synchronize()
            eager_us.append(e0.elapsed_time(e1) * 1e3)
    status = nf4_grouped.last_status(dev)

    ms_layer = statistics.median(t_layer)
    ms_gu = statistics.median(t_gu)
    ms_e2e = statistics.median(e2e_t)
    ms_e2e_dev = statistics.median(e2e_dev_t)
    ms_e2e_ffn = statistics.median(e2e_ffn_t) if e2e_ffn_t else None
    if world > 1:
        t = torch.tensor([ms_layer, ms_gu, ms_e2e, ms_e2e_dev], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_layer, ms_gu, ms_e2e, ms_e2e_dev = t.tolist()

    rows = [s["rows"] for s in steps[W:]]
    act = [s["active"] for s in steps[W:]]
    by, fl = zip(*(algorithmic(shape, "gate_up", r, a) for r, a in zip(rows, act)))
    by_l = [algorithmic(shape, "gate_up", r, a)[0] + algorithmic(shape, "down", r, a)[0] for r, a in zip(rows, act)]
    fl_l = [algorithmic(shape, "gate_up", r, a)[1] + algorithmic(shape, "down", r, a)[1] for r, a in zip(rows, act)]
    peaks = measured_peaks()
    us_gu = ms_gu * 1e3 / K
    rows_per_group = statistics.mean(r / max(a, 1) for r, a in zip(rows, act))
    hbm_bound = rows_per_group <= 16
    if hbm_bound:
        ach = statistics.mean(by) / (us_gu * 1e-6) / 1e9
        roof = dict(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
    else:
        ach = statistics.mean(fl) / (us_gu * 1e-6) / 1e12
        # the gate_up graph is timed back to back under the power cap for at least half a second: the
        # sustained cuBLAS figure is its denominator when the timed passes are long (>= 20 ms each), the
        # burst figure (a short kernel timed alone) otherwise; `peak_kind` says which, both are reported
        sustained = ms_gu >= 20.0 and peaks.get("tflops_sustained")
        peak = peaks["tflops_sustained"] if sustained else peaks["tflops"]
        roof = dict(bound="tensor", achieved=ach, peak=peak, unit="TFLOP/s", frac=ach / peak,
                    peak_kind="sustained" if sustained else "burst", frac_of_burst_peak=ach / peaks["tflops"])
    roof.update(traffic=NCU_TRAFFIC_BYTES.get((shape.name, args.tokens)), kernel="gate_up grouped GEMM", us_per_launch=us_gu, peak_source=peaks["source"],
                algorithmic_bytes=statistics.mean(by), algorithmic_flops=statistics.mean(fl))
    us_layer = ms_layer * 1e3 / K
    us_e2e = ms_e2e * 1e3 / K
    # host-buffer entry point: per GEMM the activations and (2G+2) table ints go up, the whole result comes back
    h2d = statistics.mean((s["a"].numel() + s["h"].numel()) * 2 + 2 * (2 * len(s["sizes"]) + 2) * 4 for s in steps[W:])
    d2h = statistics.mean(s["rows"] * (shape.gate_up[0] + shape.down[0]) * 2 for s in steps[W:])
    # tensor entry points: the same uploads, only the layer's final result is read back
    h2d_dev = statistics.mean((s["a"].numel() + s["h"].numel()) * 2 + (2 * len(s["sizes"]) + 1) * 8 for s in steps[W:])
    d2h_dev = statistics.mean(s["rows"] * shape.down[0] * 2 for s in steps[W:])
    base = BASELINE_US.get((shape.name, args.tokens))
    line = {
        "metric": "grouped 4-bit MoE GEMM us/layer", "value": us_layer, "unit": "us/layer",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_layer / K, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": (us_layer / base) if base else None,
        "dtype": "bf16 activations x 4-bit weights, fp32 accumulate", "data": "synthetic",
        "config": workload_config(shape, args.tokens, args.layers),
        "e2e": {"value": us_e2e, "unit": "us/layer", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "gnf4b_gemm_grouped_host (nf4_grouped.HostGroupedGemm): host x, sizes, expert ids and "
                       "result per GEMM, two blocking calls per layer"},
        "e2e_tensor_api": {"value": ms_e2e_dev * 1e3 / K, "unit": "us/layer", "h2d_bytes_per_step": h2d_dev,
                           "d2h_bytes_per_step": d2h_dev,
                           "api": f"{fn.__name__} on CUDA tensors, torch copies from pinned memory, final result "
                                  "read back"},
        "eager_api": {"value": statistics.median(eager_us), "unit": "us/layer",
                      "api": f"{fn.__name__} on device-resident activations with host routing lists, eager calls, CUDA events "
                             "per layer pass (the method of the reference_triton key)"},
        "gpu_launches": 2 * K,
        "roofline": roof,
        "layer": {"decode_gbs": statistics.mean(by_l) / (us_layer * 1e-6) / 1e9,
                  "tflops": statistics.mean(fl_l) / (us_layer * 1e-6) / 1e12,
                  "rows_per_active_expert": rows_per_group, "active_experts": statistics.mean(act)},
        "clocks": clk.summary(), "device_status": status, "repeats_ms": t_layer[:16],
    }
    if t_ffn is not None:
        one_launch = all(d["max_rows"] == 1 for d in dsteps[W:])
        line["ffn"] = {"value": statistics.median(t_ffn) * 1e3 / K, "unit": "us/layer",
                       "launches_per_layer": 1 if one_launch else 3,
                       "api": "ffn_4bit_grouped / ffn_mxfp4_grouped on device-resident inputs (gnf4b_ffn_grouped): gate_up, "
                              "activation and down GEMM in one call -- more work than `value`, which leaves the activation out"}
    if ms_e2e_ffn is not None:
        if world > 1:
            t = torch.tensor([ms_e2e_ffn], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_e2e_ffn = t.item()
        line["e2e_ffn"] = {
            "value": ms_e2e_ffn * 1e3 / K, "unit": "us/layer",
            "h2d_bytes_per_step": statistics.mean(s["a"].numel() * 2 + (2 * len(s["sizes"]) + 2) * 4 for s in steps[W:]),
            "d2h_bytes_per_step": d2h_dev,
            "api": "gnf4b_ffn_grouped_host (nf4_grouped.HostGroupedFfn): gate_up GEMM, SiLU-GLU, down GEMM in one "
                   "blocking host call per layer (one fused kernel launch at one row per group); the intermediate stays "
                   "on the device"}
    if world == 1 and not args.no_cells:
        del dsteps, host_runs, host_ffns
        t0 = time.perf_counter()
        line["cells"] = measure_cells(args, dev, peaks, layers)
        line["cells_seconds"] = time.perf_counter() - t0
    if world == 1:
        try:
            ep_us = time_ep_layer_single_gpu(args, shape, layers, dev)
        except Exception as exc:      # an extra, never at the cost of the main number
            ep_us = None
            line["ep_layer_note"] = f"not timed: {type(exc).__name__}: {str(exc)[:120]}"
        if ep_us is not None:
            # the whole MoE layer (routing plan, GEMMs over device offsets, GLU, combine) on one GPU: what the
            # `--gpus N > 1` values (which add the exchanges) compare with
            line["ep_layer_single_gpu_us"] = ep_us
    return line


# --------------------------------------------------------------------------- more cells of the same run
def _roofline(shape, proj, rows, active, us, peaks, dgrad=False):
    """Roofline of ONE grouped call: HBM-bound while groups are decode-sized, tensor-bound beyond."""
    by, fl = algorithmic(shape, proj, rows, active)
    if not dgrad and rows / max(active, 1) <= 16:
        ach = by / (us * 1e-6) / 1e9
        return dict(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"],
                    us_per_launch=us, algorithmic_bytes=by, algorithmic_flops=fl)
    ach = fl / (us * 1e-6) / 1e12
    return dict(bound="tensor", achieved=ach, peak=peaks["tflops"], unit="TFLOP/s", frac=ach / peaks["tflops"],
                peak_kind="burst", us_per_launch=us, algorithmic_bytes=by, algorithmic_flops=fl)


def _graph_us(fn_step, n_steps, replays=5):
    """Median microseconds per step of `n_steps` calls of fn_step(i) captured in one CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn_step(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_steps):
            fn_step(i)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / n_steps)
    return statistics.median(ts)


def _sampled_error(shape, proj, op, x, out, W, S, sizes, eids):
    """max |out - ref| / max |ref| against the fp64 oracle on the first rows (at most 4) of the first and the
    last group."""
    import numpy as np
    from oracle import oracle as O
    offs = [0]
    for v in sizes:
        offs.append(offs[-1] + v)
    worst = 0.0
    for gi in sorted({0, len(sizes) - 1}):
        n = min(4, sizes[gi])
        if n == 0:
            continue
        r0, e = offs[gi], eids[gi]
        xs = x[r0:r0 + n].float().cpu().numpy()
        Wn = W[e:e + 1].cpu().numpy()
        Sn = S[e:e + 1].cpu()
        Sn = Sn.view(torch.int16).numpy().view(np.uint16) if Sn.dtype == torch.bfloat16 else Sn.numpy()
        f = O.dgrad_grouped_f64 if op == "dgrad" else O.gemm_grouped_f64
        ref = f(shape.fmt, xs, Wn, Sn, [n], [0])
        got = out[r0:r0 + n].double().cpu().numpy()
        worst = max(worst, float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)))
    return worst


def measure_cells(args, dev, peaks, default_layers):
    """The other cells of the benchmark matrix, each a few seconds: same method as the headline (K steps in one
    CUDA graph over resident layer stacks walked round-robin, CUDA events, median of 5 replays), each with the
    roofline of its gate_up call (of the one call, for dgrad) and an error sample against the fp64 oracle."""
    import nf4_grouped
    cells = []
    stacks = {"qwen3_30b_a3b": default_layers if args.config == "qwen3_30b_a3b" else None}

    def layers_of(name):
        if stacks.get(name) is None:
            shape = synth.CONFIGS[name]
            per_layer = sum(shape.experts * n * (k // 2 + k // 16) for n, k in (shape.gate_up, shape.down))
            n_layers = max(2, min(16, int(3.0e9 // per_layer)))
            stacks[name] = build_layers(shape, n_layers, dev, seed=4321, random_bytes=True)
        return stacks[name]

    def fwd_cell(name, tokens, one_row_groups=0):
        shape = synth.CONFIGS[name]
        layers = layers_of(name)
        fn = grouped(shape)
        n_steps = 4 if tokens >= 512 else 16
        gen = torch.Generator().manual_seed(1000 + tokens + one_row_groups)
        st = []
        for _ in range(n_steps):
            if one_row_groups:
                eids = torch.randperm(shape.experts, generator=gen)[:one_row_groups].sort().values.tolist()
                sizes = [1] * one_row_groups
                a = torch.randn(one_row_groups, shape.hidden, generator=gen).to(torch.bfloat16)
            else:
                x, idx, _ = synth.routed_batch(shape, tokens, gen)
                tok, sizes, eids, _ = synth.dispatch(idx, shape.experts)
                a = x[tok].contiguous()
            off = [0]
            for v in sizes:
                off.append(off[-1] + v)
            st.append(dict(a=a.to(dev), h=torch.randn(a.shape[0], shape.inter, generator=gen).to(torch.bfloat16).to(dev),
                           off=torch.tensor(off, dtype=torch.int32, device=dev),
                           eids=torch.tensor(eids, dtype=torch.int32, device=dev), sizes=sizes, eid_list=eids,
                           max_rows=max(sizes)))

        def step(i, what):
            (gu, dn), d = layers[i % len(layers)], st[i]
            o = None
            if what != "down":
                o = fn(d["a"], gu[0], gu[1], None, d["eids"], group_offsets=d["off"], max_rows=d["max_rows"], tables_ready=True)
            if what != "gate_up":
                o = fn(d["h"], dn[0], dn[1], None, d["eids"], group_offsets=d["off"], max_rows=d["max_rows"], tables_ready=True)
            return o

        us_layer = _graph_us(lambda i: step(i, "both"), n_steps)
        us_gu = _graph_us(lambda i: step(i, "gate_up"), n_steps)
        rows = statistics.mean(len(d["a"]) for d in st)
        active = statistics.mean(len(d["sizes"]) for d in st)
        d0 = st[0]
        err = _sampled_error(shape, "gate_up", "fwd", d0["a"], step(0, "gate_up"), layers[0][0][0], layers[0][0][1],
                             d0["sizes"], d0["eid_list"])
        what = f"{one_row_groups} one-row groups" if one_row_groups else f"{tokens} tokens"
        cells.append({"workload": f"{shape.name} {shape.fmt} MoE layer, {what}, gate_up {shape.gate_up} + down {shape.down}",
                      "tokens": tokens, "value": us_layer, "unit": "us/layer", "rows": rows, "active_experts": active,
                      "roofline": _roofline(shape, "gate_up", rows, active, us_gu, peaks), "max_rel_err": err})

    def dgrad_cell(name, tokens):
        shape = synth.CONFIGS[name]
        layers = layers_of(name)
        gen = torch.Generator().manual_seed(2000 + tokens)
        _, idx, _ = synth.routed_batch(shape, tokens, gen)
        tok, sizes, eids, _ = synth.dispatch(idx, shape.experts)
        off = [0]
        for v in sizes:
            off.append(off[-1] + v)
        off_t = torch.tensor(off, dtype=torch.int32, device=dev)
        eid_t = torch.tensor(eids, dtype=torch.int32, device=dev)
        for proj, pi in (("gate_up", 0), ("down", 1)):
            N, K = getattr(shape, proj)
            go = (torch.randn(len(tok), N, generator=gen) * 1e-3).to(torch.bfloat16).to(dev)
            call = (nf4_grouped.dgrad_4bit_grouped if shape.fmt == "nf4"
                    else __import__("mxfp4_grouped").dgrad_mxfp4_grouped)

            def step(i):
                W, S = layers[i % len(layers)][pi]
                return call(go, W, S, None, eid_t, group_offsets=off_t, max_rows=max(sizes))

            us = _graph_us(step, 4)
            err = _sampled_error(shape, proj, "dgrad", go, step(0), layers[0][pi][0], layers[0][pi][1], sizes, eids)
            cells.append({"workload": f"{shape.name} {shape.fmt} QLoRA dgrad, {proj} stack [{shape.experts}, {N}, {K}], "
                                      f"{len(tok)} rows of dY ~ N(0, 1e-3)",
                          "tokens": tokens, "value": us, "unit": "us/call", "rows": len(tok), "active_experts": len(eids),
                          "roofline": _roofline(shape, proj, len(tok), len(eids), us, peaks, dgrad=True), "max_rel_err": err})

    def gather_cell(name, k):
        """Residency feeder: the packed rows of k experts' gate_up blocks gathered into device slots by
        device-resident ids -- from a device pool (HBM-bound: every byte read once and written once) and from pinned
        host memory (PCIe-bound; the figure is reported, the roofline object is the device pool's)."""
        import host_gather
        shape = synth.CONFIGS[name]
        N, K = shape.gate_up
        row = N * (K // 2)
        gen = torch.Generator().manual_seed(3000 + k)
        n_pool = max(2 * k, min(shape.experts, int(1.0e9 // row)))
        pool = torch.randint(0, 256, (n_pool, row), dtype=torch.uint8, device=dev)
        host = torch.randint(0, 256, (min(n_pool, 32), row), dtype=torch.uint8).pin_memory()
        slots = [torch.empty(k, row, dtype=torch.uint8, device=dev) for _ in range(4)]
        ids = [torch.randperm(n_pool, generator=gen)[:k].to(torch.int32).to(dev) for _ in range(16)]
        ids_h = [torch.randperm(host.shape[0], generator=gen)[:k].to(torch.int32).to(dev) for _ in range(16)]
        us_dev = _graph_us(lambda i: host_gather.gather_expert_rows(slots[i % 4], pool, ids[i]), 16)
        us_host = _graph_us(lambda i: host_gather.gather_expert_rows(slots[i % 4], host, ids_h[i]), 16)
        host_gather.gather_expert_rows(slots[0], pool, ids[0])
        exact = bool(torch.equal(slots[0], pool[ids[0].long()]))
        moved = 2.0 * k * row                       # read once + written once
        ach = moved / (us_dev * 1e-6) / 1e9
        cells.append({"workload": f"{shape.name} residency feeder: {k} experts' packed gate_up rows ({row} bytes each) gathered "
                                  f"into device slots by device-resident ids",
                      "tokens": 0, "value": us_dev, "unit": "us/gather", "rows": k, "active_experts": k,
                      "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": ach / peaks["hbm_gbs"], "traffic": None, "us_per_launch": us_dev,
                                   "algorithmic_bytes": moved, "peak_source": peaks["source"],
                                   "kernel": "gather_rows_kernel, source = device pool"},
                      "pinned_host_source": {"us": us_host, "gbs": k * row / (us_host * 1e-6) / 1e9,
                                             "note": "zero-copy reads over PCIe; bytes counted once"},
                      "max_rel_err": 0.0 if exact else 1.0, "bit_exact": exact})

    plan = [lambda: fwd_cell("qwen3_30b_a3b", 0, one_row_groups=64), lambda: fwd_cell("qwen3_30b_a3b", 8),
            lambda: fwd_cell("qwen3_30b_a3b", 64), lambda: fwd_cell("qwen3_30b_a3b", 4096),
            lambda: dgrad_cell("qwen3_30b_a3b", 4096),
            lambda: fwd_cell("gpt_oss_20b", 1), lambda: fwd_cell("gpt_oss_20b", 0, one_row_groups=32),
            lambda: fwd_cell("gpt_oss_20b", 4096), lambda: fwd_cell("deepseek_v3", 0, one_row_groups=32),
            lambda: gather_cell("qwen3_30b_a3b", 8),
            lambda: gather_cell("deepseek_v3", 8)]
    for job in plan:
        try:
            job()
        except Exception as exc:      # a cell must never cost the headline
            cells.append({"workload": "cell failed", "error": f"{type(exc).__name__}: {str(exc)[:200]}"})
    return cells


# --------------------------------------------------------------------------- the reference's own GPU kernels
def run_reference_triton(args, shape):
    """Child-process mode (`--impl reference-triton`): the reference project's Triton kernels, through its public
    entry points, on this GPU and this workload -- the "beat this" column.  Needs the reference installed under
    baseline/_ref (git-ignored; `pip install --no-deps --target baseline/_ref <reference checkout>`); this
    repository's package is NOT importable in this process.  Method of the reference's own harness
    (bench/phase1/harness.py:915-930): eager calls, CUDA events, warm-up, median."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "nf4_grouped.py").exists():
        print(json.dumps({"unavailable": "the reference is not installed under baseline/_ref on this box"}))
        return 0
    sys.path[:] = [str(ref)] + [p for p in sys.path if "grouped-nf4-gemm_b200" not in p and p != str(ROOT)]
    for name in ("nf4_grouped", "mxfp4_grouped", "synth", "_gnf4b"):
        sys.modules.pop(name, None)
    try:
        import mxfp4_grouped as RM
        import nf4_grouped as RN
        assert str(ref) in RN.__file__, RN.__file__
        dev = torch.device("cuda", 0)
        gen = torch.Generator().manual_seed(5)
        n_layers, n_steps = 4, 24
        (n1, k1), (n2, k2) = shape.gate_up, shape.down
        layers = []
        for _ in range(n_layers):
            pair = []
            for (n, k) in ((n1, k1), (n2, k2)):
                W = torch.randint(0, 256, (shape.experts, n, k // 2), dtype=torch.uint8, device=dev)
                if shape.fmt == "nf4":
                    S = torch.rand(shape.experts, n, k // 64, device=dev) * 0.05 + 0.01
                else:
                    S = torch.randint(119, 126, (shape.experts, n, k // 32), dtype=torch.uint8, device=dev)
                pair.append((W, S))
            layers.append(pair)
        steps = []
        for _ in range(n_steps):
            logits = torch.randn(args.tokens, shape.experts, generator=gen)
            idx = torch.argsort(-logits, dim=-1, stable=True)[:, :shape.top_k].reshape(-1)
            uniq, counts = torch.unique_consecutive(idx[torch.argsort(idx, stable=True)], return_counts=True)
            rows = int(counts.sum())
            steps.append((torch.randn(rows, k1, generator=gen).to(torch.bfloat16).to(dev),
                          torch.randn(rows, k2, generator=gen).to(torch.bfloat16).to(dev), counts.tolist(), uniq.tolist()))
        fn = RN.gemm_4bit_grouped if shape.fmt == "nf4" else RM.gemm_mxfp4_grouped

        def layer(i, what):
            a, h, sizes, eids = steps[i % n_steps]
            (Wg, Sg), (Wd, Sd) = layers[i % n_layers]
            if what != "down":
                fn(a, Wg, Sg, sizes, eids)
            if what != "gate_up":
                fn(h, Wd, Sd, sizes, eids)

        def timed(what, n):
            out = []
            for i in range(n):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                layer(i, what)
                e1.record()
                torch.cuda.synchronize()
                out.append(e0.elapsed_time(e1) * 1e3)
            return statistics.median(out)

        for i in range(10):
            layer(i, "both")
        torch.cuda.synchronize()
        res = {"value": timed("both", 60), "unit": "us/layer", "gate_up_us": timed("gate_up", 60), "down_us": timed("down", 60),
               "method": "reference Triton kernels through the reference's public entry points (baseline/_ref), eager calls with "
                         "host routing lists, CUDA events per layer pass, 10 warm-up passes, median of 60",
               "triton": __import__("triton").__version__}
        print(json.dumps(res))
    except Exception as exc:
        print(json.dumps({"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}))
    return 0


def reference_triton_key(args):
    """Run the mode above in a child process (its imports must not meet this package's modules of the same names)
    and return its JSON object."""
    try:
        r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference-triton", "--tokens", str(args.tokens),
                            "--config", args.config], capture_output=True, text=True, timeout=600)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if lines:
            return json.loads(lines[-1])
        return {"unavailable": f"child exited {r.returncode}: {r.stderr[-200:]}"}
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--no-triton", action="store_true", help="skip the reference_triton key (the reference's own GPU kernels)")
    ap.add_argument("--tokens", type=int, default=1, help="tokens per GPU per layer pass (1 = batch-1 decode)")
    ap.add_argument("--config", default="qwen3_30b_a3b", choices=sorted(synth.CONFIGS))
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--repeats", type=int, default=7)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-cells", action="store_true", help="skip the extra cells (other batch sizes, MXFP4, dgrad)")
    ap.add_argument("--path", type=lambda v: int(v, 0), default=0,
                    help="kernel choice / ablation flags of the device-resident timed region (0 = the planner)")
    ap.add_argument("--random-bytes", action="store_true",
                    help="NF4 stacks from uniform random bytes (few set-up kernels; for profiler captures)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    shape = synth.CONFIGS[args.config]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    cpu_cut = None if args.tokens * shape.top_k <= 2048 else 2

    if args.impl == "reference-triton":
        return run_reference_triton(args, shape)
    if args.impl == "reference":
        if rank != 0:
            return 0
        # the whole job of the other arm: tokens per GPU x GPUs (weak scaling), on the host cores
        n = max(1, args.gpus)
        job_tokens = args.tokens * n
        cpu_cut = None if job_tokens * shape.top_k <= 2048 else 2
        cb = time_cpu(shape, job_tokens, args.steps, args.warmup, seed=7, max_rows_per_group=cpu_cut, budget_s=120.0)
        print(json.dumps({
            "impl": "reference", "metric": "grouped 4-bit MoE GEMM us/layer", "value": cb["value"], "unit": "us/layer",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["value"] / 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32 activations x 4-bit weights, fp32 accumulate (CPU)", "data": "synthetic",
            "config": workload_config(shape, args.tokens, args.layers, n),
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return 0

    if world > 1:
        torch.distributed.init_process_group("nccl")
    line = run_gpu(args, shape, rank, world) if world == 1 else run_gpu_ep(args, shape, rank, world)
    if rank == 0:
        if world == 1 and not args.no_triton:
            torch.cuda.empty_cache()
            line["reference_triton"] = reference_triton_key(args)
        if world == 1 and not args.no_cpu:
            try:
                line["cpu_baseline"] = time_cpu(shape, args.tokens, 8, 3, seed=7, max_rows_per_group=cpu_cut)
            except Exception as e:  # the CPU leg must not cost the GPU number
                line["cpu_baseline"] = {"value": None, "unit": "us/layer", "cores": 0, "kind": "reference",
                                        "sample": f"unavailable: {e}"}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def time_ep_layer_single_gpu(args, shape, layers, dev):
    """The expert-parallel layer's code on ONE rank (routing plan, grouped GEMMs over device offsets, GLU,
    combine; no exchange), K steps in one CUDA graph: the N = 1 point that is comparable with the
    `--gpus N > 1` values.  None when the batch is beyond the host-sync-free path."""
    import ep_moe
    if args.tokens * shape.top_k * shape.hidden * 2 > ep_moe.FIXED_CAPACITY_MAX_BYTES:
        return None
    K = min(args.steps, 32)
    gen = torch.Generator().manual_seed(4242)
    mods = [ep_moe.EPGroupedMoE(shape.experts, gu, dn, fmt=shape.fmt) for gu, dn in layers]
    batch = [tuple(t.to(dev) for t in synth.routed_batch(shape, args.tokens, gen)) for _ in range(K)]
    for i in range(min(K, len(mods) + 2)):
        mods[i % len(mods)].forward(*batch[i])
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(K):
            mods[i % len(mods)].forward(*batch[i])
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(K):
            mods[i % len(mods)].forward(*batch[i])
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / K)
    return statistics.median(ts)


#: further cells of the multi-GPU run: (config, tokens per GPU).  The prefill-sized Qwen3 layer and DeepSeek-V3 with
#: Zipf(1.1) routing at a decode-sized and a mid-sized batch; each a few seconds (few steps, two resident layers).
EP_CELLS = (("qwen3_30b_a3b", 4096), ("deepseek_v3", 8), ("deepseek_v3", 512))


def run_gpu_ep(args, shape, rank, world):
    import copy
    import ep_moe
    me = sys.modules[__name__]
    line = ep_moe.bench_ep(args, shape, rank, world, me)
    if args.no_cells:
        return line
    cells = []
    t0 = time.perf_counter()
    for cfg, tok in EP_CELLS:
        cs = synth.CONFIGS[cfg]
        if (cs.name == shape.name and tok == args.tokens) or cs.experts % world:
            continue
        a2 = copy.copy(args)
        a2.tokens, a2.steps, a2.warmup, a2.layers, a2.repeats = tok, (4 if tok >= 512 else 8), 3, 2, 2
        try:
            l2 = ep_moe.bench_ep(a2, cs, rank, world, me)
            cells.append({"workload": l2["config"].get("workload"), "tokens_per_gpu": tok, "value": l2["value"],
                          "unit": l2["unit"], "steps": a2.steps, "timing": l2["method"]["timing"],
                          "exchange": l2["method"]["exchange"], "zipf": l2["method"]["zipf"],
                          "phase_us_median": l2["ep"]["phase_us_median"],
                          "imbalance_max_over_mean": l2["ep"]["imbalance_max_over_mean"],
                          "aggregate_tflops": l2["ep"]["aggregate_tflops"], "parity": l2["ep"]["parity"],
                          "roofline": l2["roofline"], "device_status": l2["device_status"]})
        except Exception as exc:      # a cell never costs the headline
            cells.append({"workload": f"{cfg} at {tok} tokens per GPU: cell failed", "error": f"{type(exc).__name__}: {str(exc)[:200]}"})
        torch.cuda.empty_cache()
    line["cells"] = cells
    line["cells_seconds"] = time.perf_counter() - t0
    return line


if __name__ == "__main__":
    sys.exit(main())
