#!/usr/bin/env python
"""Benchmark of the fused GEMM-chain path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5] [--impl reference]

One "step" is one pass of the fused chain over this rank's shard of the workload (slices for the
attention chain, 128-row blocks for the MLP chain; the shards are contiguous and there is no
collective on the data path).  Rank 0 prints one JSON line:

* value / ms_per_step -- kernel-only throughput, inputs resident in HBM, CUDA events on the
  launching stream, max over ranks.  Two methods are run at every GPU count and both are reported: `cold`
  (one event pair per launch, L2 flushed in front of each) and `back_to_back` (one event pair around the K
  launches).  `value` is the cold figure, for every workload and at every N of a scaling sweep.
* sustained -- at least two seconds of back-to-back launches with the SM clock sampled, against the
  sustained cuBLAS peak.
* e2e -- the same pass through the public operator (ditto_b200.ops) starting from pinned HOST
  buffers: host->device copies, kernel and device->host copy of the result inside the timed region.
* roofline -- algorithmic FLOPs per launch / mean launch time against the measured cuBLAS bf16 peak.
* cpu_baseline -- the CPU port of the reference's fused loop nest timed on the host cores over a
  bounded sample (rank 0, 1 GPU only).

With --impl reference only the CPU path is timed (the reference itself needs TVM, which cannot be
installed here); rank 0 prints the line, other ranks exit.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
# DRAM traffic per unit of the dominant kernel from Nsight Compute captures (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch, divided by the units that launch processed; traffic grows in
# proportion to the units).  None = not captured.
NCU_TRAFFIC_BYTES_PER_UNIT = {
    "cfg5": (201.488e6 + 47.643e6) / 128,   # capture of the first 128 slices
    "cfg3": (101.050e6 + 11.025e6) / 512,   # capture of a full launch
    "cfg4": (50.484e6 + 5.570e6) / 128,     # capture of a full launch, 128 row blocks
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--units", type=int, default=0,
                    help="run only the first N units (slices / 128-row blocks) of the workload: small cases for profiling")
    ap.add_argument("--also", default="cfg4,cfg3,cfg2",
                    help="at 1 GPU, also time these workloads kernel-only and list them under other_workloads ('' = none)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the baseline sample")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the sustained leg (back-to-back launches with the clocks sampled); 0 = skip")
    ap.add_argument("--copy-ceiling", action="store_true",
                    help="also time plain pinned host<->device copies of the e2e volume on all ranks at once")
    ap.add_argument("--shape-table", action="store_true",
                    help="instead of the benchmark: time both chains on the reference's own benchmark shapes (1 GPU, "
                         "fp16, inputs resident, L2 flushed between launches) and print one JSON line")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": float(p["bf16_tflops"]), "tflops_sustained": float(p.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ---------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        "hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
        "hw_power_brake": 0x80,
    }

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------- the GPU arm
class DeviceRun:
    """This rank's shard of a workload on its GPU: device inputs, pinned host copies, timed passes."""

    def __init__(self, w, rank, world, device):
        import torch
        from ditto_b200 import ops
        from ditto_b200 import workloads as W
        self.torch, self.ops, self.w, self.device = torch, ops, w, device
        self.lo, self.hi = w.shard(rank, world)
        self.n = self.hi - self.lo
        tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
        # one seed per slice / 128-row block / weight matrix: a unit's data is the same at every GPU count
        if w.kind == "softmax":
            self.inputs = list(W.device_attention_inputs(w, self.lo, self.hi, device))
            self.resident = []
            self.out = torch.empty(self.n, w.M, w.N, dtype=tdt, device=device)
            self.flops = 2.0 * self.n * w.M * w.L * (w.K + w.N)
        else:
            rows = self.n * 128
            self.inputs = [W.device_mlp_inputs(w, self.lo, self.hi, device)]
            self.resident = list(W.device_mlp_weights(w, device))
            self.out = torch.empty(rows, w.N, dtype=tdt, device=device)
            self.flops = 2.0 * rows * w.L * (w.K + w.N)
        self.in_bytes = sum(t.numel() * t.element_size() for t in self.inputs)
        self.out_bytes = self.out.numel() * self.out.element_size()
        self.flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)

    def launch(self, inputs=None, out=None):
        w, ops = self.w, self.ops
        ins = inputs if inputs is not None else self.inputs
        out = out if out is not None else self.out
        if self.n == 0:
            return
        if w.kind == "softmax":
            ops.bmm_softmax_bmm(ins[0], ins[1], ins[2], out=out, scale=w.scale, key_layout="LK")
        else:
            ops.gemm_relu_gemm(ins[0], self.resident[0], self.resident[1], out=out,
                               activation="relu" if w.kind == "relu" else "identity")

    def sanity(self):
        """Largest violation of the parity tolerance on the first and the last unit of this rank's shard,
        against the CPU oracle evaluated on the same (copied back) inputs.  <= 0 means within tolerance."""
        import numpy as np
        from oracle import chain_oracle as co      # checker only: never on the measured path
        torch, w = self.torch, self.w
        if self.n == 0:
            return 0.0
        self.launch()
        torch.cuda.synchronize(self.device)
        code = co.FP16 if w.dtype == "float16" else co.BF16
        rtol, atol = (2e-2, 1e-3) if w.dtype == "float16" else (3e-2, 4e-3)
        worst = -1.0
        for u in sorted({0, self.n - 1}):
            if w.kind == "softmax":
                q, k, v = (t[u:u + 1].float().cpu().numpy() for t in self.inputs)
                want = co.bmm_softmax_bmm(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, w.scale, code)
                got = self.out[u:u + 1].float().cpu().numpy()
            else:
                x = self.inputs[0][u * 128:(u + 1) * 128].float().cpu().numpy()[None]
                w1, w2 = (t.float().cpu().numpy()[None] for t in self.resident)
                want = co.gemm_act_gemm(x, w1, w2, 1 if w.kind == "relu" else 0, code)
                got = self.out[u * 128:(u + 1) * 128].float().cpu().numpy()[None]
            if not np.isfinite(got).all():
                return float("inf")
            worst = max(worst, float((np.abs(got - want) - (rtol * np.abs(want) + atol)).max()))
        return worst

    def time_cold(self, steps, warmup, barrier):
        """Device time of `steps` launches, ms, each with its own event pair and L2 flushed in front of it
        (a buffer of twice the L2 size is overwritten between launches; the flush itself is not timed)."""
        torch = self.torch
        for _ in range(warmup):
            self.launch()
            self.flush.zero_()
        torch.cuda.synchronize(self.device)
        barrier()
        launches0 = self.ops.launch_count
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            starts[i].record()
            self.launch()
            stops[i].record()
            self.flush.zero_()
        torch.cuda.synchronize(self.device)
        barrier()
        return sum(s.elapsed_time(e) for s, e in zip(starts, stops)), self.ops.launch_count - launches0

    def time_back_to_back(self, steps, warmup, barrier):
        """Device time of `steps` launches back to back inside one pair of events, ms (the way a serving loop
        issues them: nothing in between; consecutive launches overlap their set-up with the previous tail)."""
        torch = self.torch
        for _ in range(warmup):
            self.launch()
        torch.cuda.synchronize(self.device)
        barrier()
        launches0 = self.ops.launch_count
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            self.launch()
        stop.record()
        torch.cuda.synchronize(self.device)
        barrier()
        return start.elapsed_time(stop), self.ops.launch_count - launches0

    def time_sustained(self, seconds, ms_per_launch, barrier):
        """At least `seconds` of back-to-back launches: (ms per launch, launches).  Long enough for the clocks
        to settle under the power cap, which the few-launch measurements above never reach."""
        torch = self.torch
        n = max(10, int(seconds * 1e3 / max(ms_per_launch, 1e-3)) + 1)
        torch.cuda.synchronize(self.device)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            self.launch()
        stop.record()
        torch.cuda.synchronize(self.device)
        barrier()
        return start.elapsed_time(stop) / n, n

    def time_e2e(self, steps, warmup, barrier, chunks=8):
        """Host buffers -> device -> host, every step, chunked so copies overlap the kernel. ms total."""
        torch, w = self.torch, self.w
        if self.n == 0:
            torch.cuda.synchronize(self.device)
            barrier()
            barrier()
            return 0.0
        unit_rows = 1 if w.kind == "softmax" else 128
        units = self.n
        if w.kind != "softmax":
            # a chunk of the MLP chain should still fill the GPU: 33 four-CTA clusters at once
            chunks = min(chunks, max(1, units // 33))
        chunks = max(1, min(chunks, units))
        per = -(-units // chunks)
        spans = [(c * per * unit_rows, min((c + 1) * per, units) * unit_rows) for c in range(chunks)
                 if c * per < units]
        host_in = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in self.inputs]
        for h, d in zip(host_in, self.inputs):
            h.copy_(d)
        host_out = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        nbuf = 3
        max_rows = max(b - a for a, b in spans)
        dev_in = [[torch.empty((max_rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device) for t in self.inputs]
                  for _ in range(nbuf)]
        dev_out = [torch.empty((max_rows,) + tuple(self.out.shape[1:]), dtype=self.out.dtype, device=self.device)
                   for _ in range(nbuf)]
        s_in, s_k, s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        main = torch.cuda.current_stream(self.device)

        freed = [None] * nbuf         # event: buffer's outputs copied out (buffer reusable); kept across steps
        counter = [0]

        def one_step():
            # Steps are pipelined like a serving loop would run them: step n+1's host->device copies
            # may overlap step n's kernel and device->host copies; every step still moves all of its
            # inputs and outputs, and the timed region ends when the last step's result is on the host.
            for (a, b) in spans:
                bi = counter[0] % nbuf
                counter[0] += 1
                with torch.cuda.stream(s_in):
                    if freed[bi] is not None:
                        s_in.wait_event(freed[bi])
                    for h, d in zip(host_in, dev_in[bi]):
                        d[: b - a].copy_(h[a:b], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                with torch.cuda.stream(s_k):
                    s_k.wait_event(ev_in)
                    self.launch([d[: b - a] for d in dev_in[bi]], dev_out[bi][: b - a])
                    ev_k = torch.cuda.Event()
                    ev_k.record(s_k)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k)
                    host_out[a:b].copy_(dev_out[bi][: b - a], non_blocking=True)
                    ev_o = torch.cuda.Event()
                    ev_o.record(s_out)
                freed[bi] = ev_o

        for s in (s_in, s_k, s_out):
            s.wait_stream(main)
        for _ in range(min(warmup, 2)):
            one_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.device)
        barrier()
        e0.record(main)
        for s in (s_in, s_k, s_out):
            s.wait_stream(main)
        for _ in range(steps):
            one_step()
        for s in (s_in, s_k, s_out):
            main.wait_stream(s)
        e1.record(main)
        torch.cuda.synchronize(self.device)
        barrier()
        self.e2e_checksum = float(host_out[:1].float().sum().item())
        return e0.elapsed_time(e1)


# ---------------------------------------------------------------------------- the CPU arm
def cpu_sample(w, seconds):
    """Time the CPU port of the reference's fused loop nest (oracle/chain_oracle.c:
    baseline_chain_fp32) on a bounded sample of the workload.  Returns (TFLOP/s, cores, description)."""
    import numpy as np
    from oracle import chain_oracle as co          # the benchmark's CPU-baseline leg may use the oracle
    from ditto_b200 import workloads as W
    # all host cores this process may use; torchrun exports OMP_NUM_THREADS=1, which is not what a
    # CPU baseline "on the box's host cores" means, so the thread count is set explicitly
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    kind = {"softmax": 0, "relu": 1, "identity": 2}[w.kind]
    if w.kind == "softmax":
        unit_flops = 2.0 * w.M * w.L * (w.K + w.N)
        q, k, v = W.attention_inputs(w, 0, min(8, w.batch))
        kt = np.ascontiguousarray(k.transpose(0, 2, 1))
        run = lambda: co.baseline_chain_fp32(q, kt, v, kind, w.scale, threads=cores)
        units_per_call, what = q.shape[0], "slices"
    else:
        unit_flops = 2.0 * 128 * w.L * (w.K + w.N)
        blocks = max(1, min(w.units, max(cores // 4, 1)))
        if w.kind == "identity" or w.batch > 1:
            a, b, c = W.chain_inputs(w)
            unit_flops, units_per_call, what = w.flops, 1, "full passes"
        else:
            w1, w2 = W.mlp_weights(w)
            a, b, c = W.mlp_inputs(w, 0, blocks)[None], w1[None], w2[None]
            units_per_call, what = blocks, "128-row blocks"
        run = lambda: co.baseline_chain_fp32(a, b, c, kind, 1.0, threads=cores)
    run()                                           # warm-up, page in
    t0 = time.perf_counter()
    calls = 0
    while True:
        run()
        calls += 1
        el = time.perf_counter() - t0
        if el >= seconds or calls >= 2000:
            break
    tflops = calls * units_per_call * unit_flops / el / 1e12
    return tflops, cores, f"{calls} calls x {units_per_call} {what} of {w.name} ({el:.1f} s, fp32, AVX2 FMA port)"


def reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(args.steps, 1), max(args.warmup, 0)
    per_step = max(0.5, min(8.0, 60.0 / (steps + warm)))
    vals = []
    desc = ""
    cores = 0
    for i in range(steps + warm):
        v, cores, desc = cpu_sample(w, per_step)
        if i >= warm:
            vals.append(v)
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": "fused GEMM-chain TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": w.flops / (value * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(w, max(args.gpus, 1), w.shard(0, max(args.gpus, 1))[1]),
        "note": "CPU port of the reference's fused loop nest on the host cores (the reference's own TVM/LLVM build "
                "cannot be installed here); each step times a bounded sample of the workload for seconds_per_step",
        "seconds_per_step": per_step,
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc + " per step"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- main
# The shape table of the reference's GPU benchmarks, (batch, M, N, K, L)
# (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:294-308, bmm_bmm_cuda.py:304-321; 196 tokens are rounded up
# to 208 and 49 to 64 there as well).
REFERENCE_SHAPES = [
    ("Bert-Small", 8, 512, 64, 64, 512), ("Bert-Base", 12, 512, 64, 64, 512), ("Bert-Large", 16, 512, 64, 64, 512),
    ("ViT-Base/14", 12, 256, 64, 64, 256), ("ViT-Large/14", 16, 256, 64, 64, 256), ("ViT-Huge/14", 16, 256, 80, 80, 256),
    ("ViT-Base/16", 12, 208, 64, 64, 208), ("ViT-Large/16", 16, 208, 64, 64, 208), ("ViT-Huge/16", 16, 208, 80, 80, 208),
    ("Mixer-Small/32-S", 1, 512, 64, 64, 256), ("Mixer-Base/32-S", 1, 768, 64, 64, 384), ("Mixer-Large/32-S", 1, 1024, 64, 64, 512),
]


def shape_table(steps):
    """Both chains on the reference's benchmark shapes: device time per launch, L2 flushed between launches."""
    import torch
    from ditto_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(11)
    rows = []
    for name, b, M, N, K, L in REFERENCE_SHAPES:
        a = (torch.rand(b, M, K, device=dev, generator=g) * 2 - 1).half()      # U(-1, 1) like the reference's inputs
        bm = (torch.rand(b, K, L, device=dev, generator=g) * 2 - 1).half()     # the reference's [batch, K, L] layout
        c = (torch.rand(b, L, N, device=dev, generator=g) * 2 - 1).half()
        out = torch.empty(b, M, N, dtype=torch.float16, device=dev)
        entry = {"shape": name, "batch_M_N_K_L": [b, M, N, K, L]}
        for chain, call in (("bmm_softmax_bmm", lambda: ops.bmm_softmax_bmm(a, bm, c, out=out, scale=K ** -0.5, key_layout="KL")),
                            ("bmm_bmm", lambda: ops.gemm_relu_gemm(a, bm, c, out=out, activation="identity"))):
            for _ in range(3):
                call()
            total = 0.0
            for _ in range(steps):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                call()
                e1.record()
                e1.synchronize()
                total += e0.elapsed_time(e1)
            us = total / steps * 1e3
            # back to back, as the reference's time_evaluator measures (warm L2, launches pipelined)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10 * steps):
                call()
            e1.record()
            e1.synchronize()
            us_warm = e0.elapsed_time(e1) / (10 * steps) * 1e3
            flops = 2.0 * b * M * L * (K + N)
            entry[chain] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 2),
                            "us_back_to_back": round(us_warm, 2), "tflops_back_to_back": round(flops / us_warm / 1e6, 2)}
        entry["device_status"] = ops.device_status(dev)
        rows.append(entry)
    print(json.dumps({"table": "reference benchmark shapes, fp16, one B200", "steps": steps, "rows": rows}))


def headline_method(w):
    """The timing method `value` uses: cold launches, for every workload and every GPU count.  Each launch is
    timed alone with its own event pair after an L2 flush, which is also the regime the burst peak the roofline
    divides by was measured in; the back-to-back and sustained figures printed beside it show what a tight
    loop of launches gets once the power cap pulls the clocks down."""
    return "cold"


def timing_text(method):
    return ("back to back: one event pair around the K launches" if method == "back_to_back"
            else "cold: one event pair per launch, L2 flushed before each launch; the same at every GPU count")


def config_of(w, world, units_per_gpu):
    """The `config` object of a JSON line -- the same keys for the GPU arm and the reference arm."""
    return {"workload": w.name, "kind": w.kind, "units": w.units, "units_per_gpu": units_per_gpu,
            "shape_batch_M_N_K_L": [w.batch, w.M, w.N, w.K, w.L], "scale": w.scale,
            "sharding": f"contiguous units over {world} GPU(s), no collective",
            "inputs": "one seed per slice / 128-row block / weight matrix: identical at every GPU count",
            "timing": timing_text(headline_method(w))}


def copy_ceiling(run, e2e, w, barrier, D, device):
    """What the host link allows: every rank copies the bytes one e2e step moves (its shard's inputs host ->
    device, its outputs device -> host) from / to pinned memory, both directions at once on two streams, all
    ranks at the same time, with no kernel in between.  Plain cudaMemcpyAsync, one call per tensor."""
    torch = run.torch
    if run.n == 0:
        barrier(); barrier()
        return None
    host_in = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in run.inputs]
    host_out = torch.empty(run.out.shape, dtype=run.out.dtype).pin_memory()
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    def step():
        with torch.cuda.stream(s_in):
            for h, d in zip(host_in, run.inputs):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(run.out, non_blocking=True)
    step()
    torch.cuda.synchronize(device)
    barrier()
    reps = 3
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    torch.cuda.synchronize(device)
    ms = (time.perf_counter() - t0) * 1e3 / reps
    barrier()
    ms_all = D.max_over_ranks(ms, device)
    return {"ms_per_step": ms_all, "h2d_gbs_per_rank": run.in_bytes / (ms * 1e-3) / 1e9,
            "d2h_gbs_per_rank": run.out_bytes / (ms * 1e-3) / 1e9,
            "value_if_only_copies": w.flops / (ms_all * 1e-3) / 1e12, "unit": "TFLOP/s",
            "e2e_frac_of_ceiling": e2e["value"] / (w.flops / (ms_all * 1e-3) / 1e12),
            "what": "pinned H2D of the inputs and D2H of the outputs, both directions at once, all ranks together"}


def mlp_cluster_slots():
    """Thread-block clusters of the two MLP-chain kernels the device holds at once (cudaOccupancyMaxActiveClusters)."""
    from ditto_b200 import _lib
    lib = _lib.load()
    return {"clusters_of_4": lib.ditto_b200_mlp_cluster_slots(_lib.DTYPE_BF16, _lib.EPILOGUE_QUAD_MMA),
            "clusters_of_8": lib.ditto_b200_mlp_cluster_slots(_lib.DTYPE_BF16, _lib.EPILOGUE_PAIR_MMA)}


def unfused_context(run, w, barrier):
    """Context only, never on the product path: the same shape as two library GEMMs with the hidden layer
    written to and read back from HBM (torch.matmul -> relu -> torch.matmul), cold launches like the fused
    number beside it.  What the fused form pays or gains for keeping the hidden layer on chip."""
    torch = run.torch
    x, (w1, w2) = run.inputs[0], run.resident
    def step():
        h = torch.matmul(x, w1)
        if w.kind == "relu":
            torch.relu_(h)
        return torch.matmul(h, w2)
    for _ in range(3):
        step()
        run.flush.zero_()
    torch.cuda.synchronize(run.device)
    total = 0.0
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        run.flush.zero_()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    ms = total / 10
    return {"ms_per_step": ms, "value": w.flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "what": "torch.matmul -> relu -> torch.matmul (cuBLAS), hidden layer through HBM"}


def feed_forward_context(run, w):
    """Beside the plain chain: the reference's feed-forward block on the same shape -- [out, in] weights, biases,
    ReLU after both GEMMs (nn/model/transformer.py:21-34) -- and its GELU form, through ops.ffn, cold launches."""
    torch = run.torch
    from ditto_b200 import ops
    x, (w1, w2) = run.inputs[0], run.resident
    w1t, w2t = w1.t().contiguous(), w2.t().contiguous()
    g = torch.Generator(device=run.device)
    g.manual_seed(4)
    b1 = torch.randn(w1t.shape[0], device=run.device, generator=g).to(x.dtype)
    b2 = torch.randn(w2t.shape[0], device=run.device, generator=g).to(x.dtype)
    out = torch.empty((x.shape[0], w2t.shape[0]), dtype=x.dtype, device=run.device)
    result = {}
    for name, (a1, a2) in (("bias_relu_relu", ("relu", "relu")), ("bias_gelu_identity", ("gelu", "identity"))):
        def step():
            ops.ffn(x, w1t, b1, w2t, b2, out=out, act1=a1, act2=a2)
        for _ in range(3):
            step()
            run.flush.zero_()
        torch.cuda.synchronize(run.device)
        total = 0.0
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            run.flush.zero_()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / 10
        result[name] = {"ms_per_step": ms, "value": w.flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}
    return result


def main():
    args = parse_args()
    if args.shape_table:
        shape_table(max(args.steps, 1))
        return
    from ditto_b200 import workloads as W
    if args.workload not in W.WORKLOADS:
        raise SystemExit(f"unknown workload {args.workload}; choose from {sorted(W.WORKLOADS)}")
    w = W.WORKLOADS[args.workload]
    if args.units:
        import dataclasses
        if w.kind == "softmax":
            w = dataclasses.replace(w, batch=min(args.units, w.batch), name=f"{w.name} [first {args.units} slices]")
        else:
            w = dataclasses.replace(w, M=128 * min(args.units, w.units), name=f"{w.name} [first {args.units} row blocks]")
    if args.impl == "reference":
        reference_arm(args, w)
        return
    if w.dtype == "float32":
        raise SystemExit("cfg1 is the reference's CPU-only fp32 case; it is covered by the tests, not benchmarked on the GPU")

    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world_env == 1:
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))

    import torch
    from ditto_b200 import distributed as D
    from ditto_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the chain kernels have no CPU fallback")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    rank, world = D.init(device=device)
    barrier = D.barrier
    peaks = measured_peaks()

    run = DeviceRun(w, rank, world, device)
    err = run.sanity()
    warm = max(args.warmup, 3)
    # Both methods at every GPU count; `value` takes the cold one everywhere (see headline_method).
    headline = headline_method(w)
    with ClockSampler(local) as clk:
        ms_cold, launches_cold = run.time_cold(args.steps, warm, barrier)
        ms_b2b, launches_b2b = run.time_back_to_back(args.steps, warm, barrier)
    status = ops.device_status(device)
    ms_cold = D.max_over_ranks(ms_cold, device) / args.steps
    ms_b2b = D.max_over_ranks(ms_b2b, device) / args.steps
    ms_step = ms_b2b if headline == "back_to_back" else ms_cold
    launches = launches_b2b if headline == "back_to_back" else launches_cold
    value = w.flops / (ms_step * 1e-3) / 1e12
    sustained = None
    if args.sustained_seconds > 0:
        with ClockSampler(local) as sclk:
            ms_sus, n_sus = run.time_sustained(args.sustained_seconds, ms_b2b, barrier)
        ms_sus = D.max_over_ranks(ms_sus, device)
        tf_sus = w.flops / (ms_sus * 1e-3) / 1e12
        sustained = {"value": tf_sus, "unit": "TFLOP/s", "ms_per_step": ms_sus, "launches_per_gpu": n_sus,
                     "seconds": ms_sus * n_sus / 1e3, "per_gpu": tf_sus / world,
                     "frac_of_sustained_peak": (tf_sus / world / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
                     "peak_sustained": peaks["tflops_sustained"], "clocks": sclk.summary()}
    status = max(status, ops.device_status(device))

    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(args.steps, 10))
        ms_e2e = D.max_over_ranks(run.time_e2e(e2e_steps, args.warmup, barrier), device) / e2e_steps
        e2e = {"value": w.flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "steps": e2e_steps,
               "h2d_bytes_per_step": int(D.sum_over_ranks(run.in_bytes, device)),
               "d2h_bytes_per_step": int(D.sum_over_ranks(run.out_bytes, device))}
        if args.copy_ceiling:
            e2e["copy_ceiling"] = copy_ceiling(run, e2e, w, barrier, D, device)
    err = D.max_over_ranks(err, device)
    status = int(D.max_over_ranks(status, device))
    run_flops, run_n = run.flops, run.n

    others = []
    if args.also and not args.units:
        run = None
        torch.cuda.empty_cache()
        for name in [n for n in args.also.split(",") if n and n != args.workload and n in W.WORKLOADS]:
            ow = W.WORKLOADS[name]
            if ow.dtype == "float32" or (world > 1 and ow.units < 8 * world):
                continue                      # config 2's twelve slices are a one-GPU case
            orun = DeviceRun(ow, rank, world, device)
            oerr = D.max_over_ranks(orun.sanity(), device)
            with ClockSampler(local) as oclk:
                oms_cold, _ = orun.time_cold(10, 3, barrier)
                oms_b2b, _ = orun.time_back_to_back(10, 3, barrier)
            oms_cold = D.max_over_ranks(oms_cold, device) / 10
            oms_b2b = D.max_over_ranks(oms_b2b, device) / 10
            oms = oms_b2b if headline_method(ow) == "back_to_back" else oms_cold
            otf = ow.flops / (oms * 1e-3) / 1e12
            entry = {"workload": ow.name, "value": otf, "unit": "TFLOP/s", "n_gpus": world, "ms_per_step": oms,
                     "timing": timing_text(headline_method(ow)),
                     "cold": {"ms_per_step": oms_cold, "value": ow.flops / (oms_cold * 1e-3) / 1e12},
                     "back_to_back": {"ms_per_step": oms_b2b, "value": ow.flops / (oms_b2b * 1e-3) / 1e12},
                     "frac_of_tensor_peak": otf / world / peaks["tflops"],
                     "algorithmic_gbs": ow.bytes / (oms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": ow.bytes / world / (oms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "sanity_worst_tolerance_excess_vs_oracle": oerr, "clocks": oclk.summary(),
                     "device_status": int(D.max_over_ranks(ops.device_status(device), device))}
            if ow.kind != "softmax":
                entry["cluster_slots"] = mlp_cluster_slots()
                if world == 1:
                    entry["context_unfused_torch"] = unfused_context(orun, ow, barrier)
                    if ow.kind == "relu" and len(orun.resident[0].shape) == 2:
                        entry["feed_forward_block"] = feed_forward_context(orun, ow)
            others.append(entry)
            del orun
            torch.cuda.empty_cache()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cores, desc = cpu_sample(w, args.cpu_seconds)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}

    if rank == 0:
        per_gpu_flops = run_flops                      # rank 0's launch (shards are equal for 1/2/4/8 GPUs)
        achieved = per_gpu_flops / (ms_step * 1e-3) / 1e12
        unit_traffic = NCU_TRAFFIC_BYTES_PER_UNIT.get(args.workload)
        line = {
            "metric": "fused GEMM-chain TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": {"float16": "fp16", "bfloat16": "bf16"}[w.dtype] + " in, f32 accumulate",
            "data": "synthetic",
            "config": config_of(w, world, run_n),
            "cold": {"ms_per_step": ms_cold, "value": w.flops / (ms_cold * 1e-3) / 1e12},
            "back_to_back": {"ms_per_step": ms_b2b, "value": w.flops / (ms_b2b * 1e-3) / 1e12},
            "sustained": sustained,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"],
                         "traffic": (unit_traffic * run_n) if unit_traffic else None,
                         "peak_source": peaks["source"] + " cuBLAS bf16 burst",
                         "algorithmic_gbs": w.bytes / world / (ms_step * 1e-3) / 1e9, "hbm_peak_gbs": peaks["hbm_gbs"]},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "other_workloads": others,
            "gpu_launches": launches,
            "clocks": clk.summary(),
            "sanity_worst_tolerance_excess_vs_oracle": err,
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    barrier()
    if D.dist.is_initialized():
        D.dist.destroy_process_group()


if __name__ == "__main__":
    main()
