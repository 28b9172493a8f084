"""Runs one decode-matmul shape a few times on cuda:0 -- the smallest driver for a profiler.

    python -m decode_matmul_b200.one_call fp16 1 28672 8192 [--calls 3] [--path 0..3] [--atomic]
    python -m decode_matmul_b200.one_call int8 8 8192 8192
    python -m decode_matmul_b200.one_call fp16 32 28672 8192 --time     (timing loop, one JSON line)

Random codes, the synthetic {0.5..3.5} codebook (fp16 family) or the E8P table (integer family),
prints the device status word and a checksum of the last result.
"""
import argparse

import torch

import decode_matmul_b200 as dmm


def time_shape(a, total_mb=700):
    """Median microseconds per call over 5 replays of a CUDA graph of back-to-back calls (programmatic
    dependent launch, atomic accumulation for the fp16 family), each call on another copy of the
    weights so that together they exceed the L2 cache."""
    import json
    import statistics

    code_bytes = a.n * a.k // 4
    nbuf = max(2, min(64, int(total_mb * 1e6 // code_bytes) + 1))
    gen = torch.Generator(device="cuda").manual_seed(1)
    bufs = [torch.randint(-32768, 32768, (a.n, a.k // 8), dtype=torch.int16, device="cuda", generator=gen)
            for _ in range(nbuf)]
    if a.family == "fp16":
        cb = dmm.synthetic_codebook(42, "cuda")
        x = torch.randn(a.batch, a.k, device="cuda", dtype=torch.float16)
        out = torch.zeros(a.batch, a.n, device="cuda", dtype=torch.float32)

        def call(w):
            dmm.decode_matmul_fp16(x, w, cb, 2.0 ** -10, out, path=a.path, accumulate=True, atomic=True, pdl=True)
    else:
        cb = dmm.build_codebook_abs("cuda")
        x = torch.randint(-128, 128, (a.batch, a.k), dtype=torch.int8, device="cuda")
        out = torch.zeros(a.batch, a.n, device="cuda", dtype=torch.int32)

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
    print(json.dumps({"family": a.family, "batch": a.batch, "n": a.n, "k": a.k, "us_per_call": round(us, 2),
                      "code_gb_per_s": round(code_bytes / us / 1e3, 1), "tflops": round(2 * a.batch * a.n * a.k / us / 1e6, 1),
                      "weight_copies": nbuf, "status": dmm.status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("family", choices=["fp16", "int8"])
    ap.add_argument("batch", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--calls", type=int, default=3)
    ap.add_argument("--path", type=int, default=dmm.PATH_AUTO)
    ap.add_argument("--atomic", action="store_true")
    ap.add_argument("--time", action="store_true",
                    help="time the shape: CUDA-graph replay of calls that cycle over weight buffers larger than L2")
    a = ap.parse_args()
    if a.time:
        return time_shape(a)
    w = torch.randint(-32768, 32768, (a.n, a.k // 8), dtype=torch.int16, device="cuda")
    if a.family == "fp16":
        cb = dmm.synthetic_codebook(42, "cuda")
        x = torch.randn(a.batch, a.k, device="cuda", dtype=torch.float16)
        out = torch.zeros(a.batch, a.n, device="cuda", dtype=torch.float32)
        for _ in range(a.calls):
            y = dmm.decode_matmul_fp16(x, w, cb, 1.0, out, path=a.path, accumulate=a.atomic, atomic=a.atomic)
    else:
        cb = dmm.build_codebook_abs("cuda")
        x = torch.randint(-128, 128, (a.batch, a.k), dtype=torch.int8, device="cuda")
        for _ in range(a.calls):
            y = dmm.decode_matmul_i8(x, w, cb)
    torch.cuda.synchronize()
    print("status", dmm.status(), "checksum", float(y.float().abs().sum()))


if __name__ == "__main__":
    main()
