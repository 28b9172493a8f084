#!/usr/bin/env python
"""Benchmark of the decode-matmul hot path on the Llama-2-70B linear stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One step = one pass of a [B, 8192] residual stream through the linear layers of 80
transformer blocks (qkv 10240x8192, o 8192x8192, gate+up 57344x8192, down 8192x28672; 17.1 GB
of 2-bit codes), synthetic seeded codes and codebook.  With N > 1 (launched by torchrun, one
rank per GPU) the stack is tensor-parallel: qkv and gate/up split by output rows, o and down
split by reduction index with an NCCL all-reduce, so the total work is fixed (strong scaling).

The JSON line reports compressed-weight GB/s: code bytes of the whole stack divided by the
step time.  `value` is timed with the inputs resident in HBM (CUDA-graph replay of the step),
`e2e` through the public Python API with the activations coming from pinned host memory and
the result copied back every step.  The weights are far larger than L2 (17 GB vs 126 MB), so
no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes moved per algorithmic byte by the dominant kernel, from one ncu capture (see
# profiles/umma_f8_57344x8192_b1.md): dram__bytes_read.sum + dram__bytes_write.sum = 122.00 MB
# for 117.68 MB of codes, activations, output and codebook.
NCU_TRAFFIC_PER_ALG_BYTE = 122.00 / 117.68
METRIC = "compressed_weight_hbm_gbs"
UNIT = "GB/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-shapes", action="store_true", help="skip the per-shape table and the batch-32 line (N = 1 only)")
    ap.add_argument("--shape", default=None, metavar="FAMILY:B:N:K",
                    help="instead of the stack: one product, e.g. fp16:1:57344:8192 or int8:8:28672:8192; runs it "
                         "--calls times (the smallest driver for a profiler) or, with --time, times it")
    ap.add_argument("--calls", type=int, default=3)
    ap.add_argument("--path", type=int, default=0, help="with --shape (fp16 family): DMM_PATH_* value, 0 = auto")
    ap.add_argument("--time", action="store_true")
    return ap.parse_args()


def workload_config(args, world):
    return {
        "workload": "llama2-70b-linear-stack (BASELINE.json configs[4]; layer shapes of configs[3])",
        "shapes": {"qkv": [10240, 8192], "o": [8192, 8192], "gate_up": [57344, 8192], "down": [8192, 28672]},
        "layers": args.layers,
        "batch": args.batch,
        "parallelism": f"tp{world}" if world > 1 else "single",
        "l2": "inputs larger than L2 (17.1 GB of codes per step), no flush",
    }


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU baseline: the reference's own CPU path (its test script's table-gather decode, then an
# fp32 torch.matmul), timed on the host cores on a bounded sample: one transformer block.
# ------------------------------------------------------------------------------------------
def cpu_reference_sample(batch, reps=1):
    import numpy as np
    import torch

    from oracle import dmm_oracle as o

    # torchrun exports OMP_NUM_THREADS=1 to every rank: take all host cores explicitly
    try:
        torch.set_num_threads(os.cpu_count() or 1)
    except RuntimeError:
        pass
    cb16 = o.synthetic_codebook(42)
    table = (o.decode_table(o.cb16_to_cb64(cb16)).astype(np.float32) / 4)  # [65536, 8]
    table_t = torch.from_numpy(table)
    rng = np.random.default_rng(46)
    shapes = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]
    total_bytes, t_decode, t_matmul = 0, 0.0, 0.0
    for _ in range(reps):
        for n, k in shapes:
            codes = torch.from_numpy(rng.integers(0, 65536, size=(n, k // 8), dtype=np.int64))
            x = torch.from_numpy(rng.standard_normal((batch, k)).astype(np.float16))
            t0 = time.perf_counter()
            w = table_t[codes].reshape(n, k)  # decode: gather of 8 weights per code
            t1 = time.perf_counter()
            y = torch.matmul(x.float(), w.t())
            t2 = time.perf_counter()
            t_decode += t1 - t0
            t_matmul += t2 - t1
            total_bytes += n * k // 4
            del w, y, codes
    seconds = t_decode + t_matmul
    return {
        "value": total_bytes / seconds / 1e9,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "sample": f"{reps} transformer block(s) of the stack (4 matmuls, {total_bytes / 1e6:.0f} MB of codes) at batch "
                  f"{batch}: decode {t_decode:.2f} s + fp32 matmul {t_matmul:.2f} s",
        "seconds": seconds,
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    info = None
    for i in range(args.warmup + args.steps):
        info = cpu_reference_sample(args.batch, reps=1)
        if i >= args.warmup:
            times.append(info["seconds"])
        if sum(times) > 150:  # keep the whole run within a few minutes
            break
    sample_bytes = 213909504
    sec = statistics.mean(times)
    value = sample_bytes / sec / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": dict(workload_config(args, 1), step="one transformer block (bounded sample of the stack)"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": "port", "sample": info["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_gpu_kernel": {"unavailable": "decode_matmul_cuda.cu builds only as a torch extension through the "
                                 "reference's own setup.py and accepts M = 8, K % 2048 == 0 only: it cannot run the "
                                 "batch-1 fp16 workload of the metric; the CPU path above is the reference arm"},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# single-shape timing (BASELINE.json configs[1..3] and the batch-32 half of the metric)
# ------------------------------------------------------------------------------------------
def time_shape(dmm, torch, family, batch, n, k, total_mb=700):
    """Median microseconds per call over 5 replays of a CUDA graph of back-to-back calls (programmatic
    dependent launch, atomic accumulation for the fp16 family), each call on another copy of the
    weights so that together the copies exceed the L2 cache several times."""
    code_bytes = n * k // 4
    nbuf = max(2, min(64, int(total_mb * 1e6 // code_bytes) + 1))
    gen = torch.Generator(device="cuda").manual_seed(1)
    bufs = [torch.randint(-32768, 32768, (n, k // 8), dtype=torch.int16, device="cuda", generator=gen)
            for _ in range(nbuf)]
    if family == "fp16":
        cb = dmm.synthetic_codebook(42, "cuda")
        x = torch.randn(batch, k, device="cuda", dtype=torch.float16)
        out = torch.zeros(batch, n, device="cuda", dtype=torch.float32)

        def call(w):
            dmm.decode_matmul_fp16(x, w, cb, 2.0 ** -10, out, accumulate=True, atomic=True, pdl=True)
    else:
        cb = dmm.build_codebook_abs("cuda")
        x = torch.randint(-128, 128, (batch, k), dtype=torch.int8, device="cuda")
        out = torch.zeros(batch, n, device="cuda", dtype=torch.int32)

        def call(w):
            dmm.decode_matmul_i8(x, w, cb, out, accumulate=True, pdl=True)
    reps = max(nbuf * 2, 40)
    call(bufs[0])
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        call(bufs[0])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(reps):
                call(bufs[i % nbuf])
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / reps)
    us = statistics.median(times)
    del graph, bufs
    return {"family": family, "batch": batch, "n": n, "k": k, "us": round(us, 2),
            "gbs": round(code_bytes / us / 1e3, 1), "tflops": round(2 * batch * n * k / us / 1e6, 1),
            "weight_copies": nbuf, "launches": reps}


def per_shape_table(dmm, torch, peaks):
    """BASELINE.json configs[1] (Llama-2-7B shapes, batch 1), configs[2] (batch sweep on the 7B gate/up
    and down shapes), configs[3] (Llama-2-70B shapes at batch 1 and 16) and the integer operator."""
    rows = []
    for n, k in [(4096, 4096), (11008, 4096), (4096, 11008)]:
        rows.append(dict(time_shape(dmm, torch, "fp16", 1, n, k), config="configs[1]"))
    for n, k in [(11008, 4096), (4096, 11008)]:
        for b in (2, 4, 8, 16, 32, 64):
            rows.append(dict(time_shape(dmm, torch, "fp16", b, n, k), config="configs[2]"))
    for n, k in [(10240, 8192), (8192, 8192), (28672, 8192), (8192, 28672)]:
        for b in (1, 16):
            rows.append(dict(time_shape(dmm, torch, "fp16", b, n, k), config="configs[3]"))
    for b in (8, 32):
        rows.append(dict(time_shape(dmm, torch, "int8", b, 28672, 8192), config="reference operator (int8)"))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    for r in rows:
        r["frac_of_hbm_measured"] = round(r["gbs"] / hbm, 3)
    return rows


def batch_tensor_line(dmm, torch, peaks, batch, sampler_index):
    """The batch-32 half of the metric: TFLOP/s of one 28672 x 8192 product at this batch, timed alone
    (burst peak is the denominator), with its own clock record."""
    sampler = ClockSampler(sampler_index)
    sampler.start()
    r = time_shape(dmm, torch, "fp16", batch, 28672, 8192, total_mb=1400)
    clocks = sampler.stop()
    burst = float(peaks.get("bf16_tflops", 1590.0))
    return {"shape": [28672, 8192], "batch": batch, "us": r["us"], "tflops": r["tflops"],
            "frac_of_bf16_burst": round(r["tflops"] / burst, 4), "peak_bf16_burst": burst,
            "frac_of_2250": round(r["tflops"] / 2250.0, 4), "gbs": r["gbs"],
            "kernel": ("umma_kernel<PolF8,16>" if batch <= 2 else "umma_kernel<PolF8,32>") if batch <= 8 else "umma_kernel<PolF8,64>" if batch <= 16 else "dmm_kernel<PolF8,128>",
            "launches": r["launches"], "clocks": clocks}

# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import decode_matmul_b200 as dmm
    from decode_matmul_b200.linear import LLAMA2_70B, LinearStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL serves set-up barriers and the parity check only (the timed step has no NCCL call), and this
        # process leaves without tearing the group down (see the end of this function): keep its buffers off
        # NVLink multicast objects, which must not be left bound when a rank exits
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    cfg = dict(LLAMA2_70B, layers=args.layers)
    stack = LinearStack(cfg, dmm.synthetic_codebook(42), dev, world=world, rank=rank, seed=46, scale=2.0 ** -12)
    B, H = args.batch, cfg["hidden"]
    gen = torch.Generator().manual_seed(1234)
    h_host = torch.randn(B, H, generator=gen, dtype=torch.float32).pin_memory()
    out_host = torch.empty(B, H, dtype=torch.float32).pin_memory()
    h_in = torch.empty(B, H, dtype=torch.float32, device=dev)
    h = torch.empty(B, H, dtype=torch.float32, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- capture one step (residual stream resident in HBM) ----
    stream = torch.cuda.Stream(dev)
    h_in.copy_(h_host)
    with torch.cuda.stream(stream):
        for _ in range(2):  # allocates the library workspace and NCCL buffers before capture
            h.copy_(h_in)
            stack.step(h)
        stream.synchronize()
        launches0 = dmm.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            h.copy_(h_in)
            stack.step(h)
        launches_per_step = dmm.launch_count() - launches0
        # the end-to-end step as ONE graph: host -> device copy of the step's activations from
        # pinned memory, the same kernels, device -> host copy of the result
        graph_e2e = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_e2e, stream=stream):
            h.copy_(h_host, non_blocking=True)
            stack.step(h)
            out_host.copy_(h, non_blocking=True)
    barrier()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps

    def step_resident():
        graph.replay()

    def step_e2e():
        graph_e2e.replay()
        stream.synchronize()  # the caller reads the result every step

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step_resident()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(step_resident, args.steps)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # ---- dominant kernel alone: every matmul of the stack back to back, no glue ----
    xs = {k: torch.randn(B, lin.in_features, device=dev, dtype=torch.float16) for k, lin in stack.layers[0].items()}
    outs = {k: torch.empty(B, lin.out_features, device=dev, dtype=torch.float32) for k, lin in stack.layers[0].items()}

    chained = world == 1 and B < 4 and getattr(stack, "chain_blocks", 0) > 0
    hk = torch.zeros(B, H, device=dev, dtype=torch.float32)

    def kernels_only():  # same launch mode as the step: PDL chain, atomic accumulation for small batch
        if chained:  # the step is nothing but the chained matmul launches (plus one fill): time those
            hk.zero_()
            stack.step(hk)
            return
        flat = [(k, lin) for blk in stack.layers for k, lin in blk.items()]
        for i, (k, lin) in enumerate(flat):
            if B <= 32:
                dmm.hint_next_weights(flat[i + 1][1].codes if i + 1 < len(flat) else None)  # as the step does
                dmm.decode_matmul_fp16(xs[k], lin.codes, lin.codebook, lin.scale, outs[k], accumulate=True,
                                       atomic=True, pdl=True)
            else:
                lin(xs[k], out=outs[k])

    with torch.cuda.stream(stream):
        kernels_only()
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph, stream=stream):
            kernels_only()
    ms_kernels = timed(kgraph.replay, max(3, args.steps // 4))
    status = dmm.status()

    # ---- parity of the fused step (what was timed) with the plain step, on a 2-block prefix ----
    saved_layers = stack.layers
    stack.layers = saved_layers[:2]
    with torch.cuda.stream(stream):
        h_a, h_b = h_in.clone(), h_in.clone()
        stack.step(h_a, fused=True)
        stack.step(h_b, fused=False)
        stream.synchronize()
    stack.layers = saved_layers
    parity = {"what": "fused step (timed) vs plain step (separate cast / activation / residual kernels), first 2 blocks",
              "max_abs_diff": float((h_a - h_b).abs().max()), "max_abs": float(h_b.abs().max())}
    if world > 1:
        t = torch.tensor([parity["max_abs_diff"]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity["max_abs_diff"] = float(t.item())

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    extra = {}
    if world == 1 and not args.no_shapes:
        del graph, graph_e2e, kgraph
        with torch.cuda.stream(stream):
            extra["batch32"] = batch_tensor_line(dmm, torch, peaks, 32, local)
            extra["batch16"] = batch_tensor_line(dmm, torch, peaks, 16, local)
            extra["per_shape"] = per_shape_table(dmm, torch, peaks)
        extra["per_shape_how"] = ("CUDA events around a CUDA graph of back-to-back calls cycling over weight copies that "
                                  "together exceed L2 several times; programmatic dependent launch; median of 5 replays")
        status |= dmm.status()

    if rank == 0:
        from oracle import dmm_oracle  # noqa: F401  (the checker; used below for the CPU baseline only)

        code_bytes = stack.code_bytes_total
        value = code_bytes / (ms * 1e-3) / 1e9
        e2e = code_bytes / (ms_e2e * 1e-3) / 1e9
        # algorithmic bytes of the matmul launches of this rank: codes + activations + outputs + codebook
        alg = 0
        for blk in stack.layers:
            for lin in blk.values():
                alg += lin.code_bytes + 2 * B * lin.in_features + 4 * B * lin.out_features + 4096
        n_launch = sum(len(blk) for blk in stack.layers)
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = alg / (ms_kernels * 1e-3) / 1e9
        cpu = cpu_reference_sample(B, reps=1)
        cpu.pop("seconds")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 x 2-bit codes (fp6/fp8 tensor-core operands, fp32 accumulate)", "data": "synthetic",
            "config": dict(workload_config(args, world), **({"tp_form": getattr(stack, "tp_form_used", "nccl")} if world > 1 else {})),
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": B * H * 4,
                    "d2h_bytes_per_step": B * H * 4},
            "gpu_launches": int(launches_per_step) * args.steps,
            "gpu_launches_per_step": int(launches_per_step),
            "tokens_per_s": B / (ms * 1e-3),
            "pct_of_8tbs": 100.0 * value / 8000.0 / world,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak,
                "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks else "6650 GB/s (of fallback)",
                "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_PER_ALG_BYTE * alg / n_launch if B <= 8 else None,
                "traffic_unit": "bytes per launch (mean over the stack's launches)",
                "traffic_source": "ncu capture of the 57344x8192 launch (profiles/umma_f8_57344x8192_b1.md): "
                                  "122.00 MB DRAM read+write for 117.68 MB algorithmic; scaled by algorithmic bytes",
                "algorithmic_bytes_per_launch": alg / n_launch,
                "kernel": ("umma_kernel<PolF8,32,chain> (8 products per launch)" if chained else ("umma_kernel<PolF8,16>" if B <= 2 else "umma_kernel<PolF8,32>")) if B <= 8 else ("umma_kernel<PolF8,64>" if B <= 16 else "dmm_kernel<PolF8,128>"),
                "how": "all matmul launches of the stack back to back in one CUDA graph, CUDA events; per-GPU figure"
                       + ("; achieved and traffic are per product (a chained launch runs 8 products)" if chained else ""),
                "ms": ms_kernels,
            },
            "cpu_baseline": cpu,
            "clocks": clocks,
            "status_word": status,
            "parity": parity,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave together.  The captured graphs hold kernels that spin on peer flags (and, in the NCCL form,
        # collectives): destroy them and every peer-mapped buffer first, drain the device, then skip the
        # process-group teardown -- destroy_process_group with graphs of its collectives alive blocked here for
        # the whole time limit, and a rank must not exit while a peer can still touch its memory.
        try:
            del graph, graph_e2e, kgraph
        except NameError:
            pass
        stack._peer = None
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_shape(args):
    """One product on cuda:0: a few plain calls (random codes, the synthetic {0.5..3.5} codebook for the fp16 family,
    the E8P table for the integer family; prints the device status word and a checksum), or one timing line."""
    import torch

    import decode_matmul_b200 as dmm

    family, b, n, k = args.shape.split(":")
    b, n, k = int(b), int(n), int(k)
    if args.time:
        print(json.dumps(dict(time_shape(dmm, torch, family, b, n, k), status=dmm.status())), flush=True)
        return
    w = torch.randint(-32768, 32768, (n, k // 8), dtype=torch.int16, device="cuda")
    if family == "fp16":
        cb = dmm.synthetic_codebook(42, "cuda")
        x = torch.randn(b, k, device="cuda", dtype=torch.float16)
        out = torch.zeros(b, n, device="cuda", dtype=torch.float32)
        for _ in range(args.calls):
            y = dmm.decode_matmul_fp16(x, w, cb, 1.0, out, path=args.path, accumulate=True, atomic=args.path in (0, 2, 3))
    else:
        cb = dmm.build_codebook_abs("cuda")
        x = torch.randint(-128, 128, (b, k), dtype=torch.int8, device="cuda")
        for _ in range(args.calls):
            y = dmm.decode_matmul_i8(x, w, cb)
    torch.cuda.synchronize()
    print("status", dmm.status(), "checksum", float(y.float().abs().sum()))


def main():
    args = parse()
    if args.shape:
        return run_shape(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
