"""Runs one decode-matmul shape a few times on cuda:0 -- the smallest driver for a profiler.

    python -m decode_matmul_b200.one_call fp16 1 28672 8192 [--calls 3] [--path 0..3] [--atomic]
    python -m decode_matmul_b200.one_call int8 8 8192 8192

Random codes, the synthetic {0.5..3.5} codebook (fp16 family) or the E8P table (integer family),
prints the device status word and a checksum of the last result.
"""
import argparse

import torch

import decode_matmul_b200 as dmm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("family", choices=["fp16", "int8"])
    ap.add_argument("batch", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--calls", type=int, default=3)
    ap.add_argument("--path", type=int, default=dmm.PATH_AUTO)
    ap.add_argument("--atomic", action="store_true")
    a = ap.parse_args()
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
