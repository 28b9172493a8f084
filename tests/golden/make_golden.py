"""Generate the golden fixtures in this folder from the reference's own Python code.

Run once in a container that has the reference checkout (read-only) mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference's test script imports its CUDA extension at module scope, so a
stub module named ``decode_matmul_cuda`` is installed first; only the pure
Python functions of the script (``decode``, ``decode_matmul_torch``,
``build_codebook_abs``, ``build_x_weights``, ``transpose_tile``) are executed,
on CPU tensors.  The outputs are what the oracle and the CUDA kernels are
checked against; nothing from the reference is copied, only its results.

Files written (all small, numpy ``.npz``):
  e8p_codebook.npz     codebook_abs int64[256] as the reference builds it
  decode_all_codes.npz table int8[65536,8]: reference decode() of every code word
  transpose_tile.npz   a logical code matrix and the reference's tiled form of it
  matmul_small.npz     x, codes and decode_matmul_torch(x, codes, cb) at 8x16x64 and 3x32x32
  matmul_ref_shape.npz the reference test's own shape 8x16x4096 (CPU generator, seed 42)
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch


def load_reference(ref_root):
    stub = types.ModuleType("decode_matmul_cuda")
    stub.decode_matmul = None
    sys.modules["decode_matmul_cuda"] = stub
    spec = importlib.util.spec_from_file_location("ref_test", os.path.join(ref_root, "test_decode_matmul.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of nalzok/decode-matmul>")
    ref_root = sys.argv[1]
    out = os.path.dirname(os.path.abspath(__file__))
    ref = load_reference(ref_root)
    torch.random.manual_seed(42)

    cb = ref.build_codebook_abs("cpu")
    np.savez_compressed(os.path.join(out, "e8p_codebook.npz"), codebook_abs=cb.numpy())

    table = np.zeros((65536, 8), dtype=np.int8)
    codes = torch.arange(65536, dtype=torch.int32).to(torch.int16)  # wraps to the int16 bit patterns
    for c in range(65536):
        table[c] = ref.decode(codes[c], cb).to(torch.int8).numpy()
    np.savez_compressed(os.path.join(out, "decode_all_codes.npz"), table=table)

    x, w = ref.build_x_weights(8, 64, 256, "cpu")
    np.savez_compressed(os.path.join(out, "transpose_tile.npz"), logical=w.numpy(),
                        tiled=ref.transpose_tile(w).numpy())

    small = {}
    for tag, (m, n, k) in {"a": (8, 16, 64), "b": (3, 32, 32)}.items():
        x, w = ref.build_x_weights(m, n, k, "cpu")
        y = ref.decode_matmul_torch(x, w, cb)
        small.update({f"x_{tag}": x.numpy(), f"codes_{tag}": w.numpy(), f"y_{tag}": y.numpy()})
    np.savez_compressed(os.path.join(out, "matmul_small.npz"), **small)

    torch.random.manual_seed(42)
    x, w = ref.build_x_weights(8, 16, 4096, "cpu")
    y = ref.decode_matmul_torch(x, w, cb)
    np.savez_compressed(os.path.join(out, "matmul_ref_shape.npz"), x=x.numpy(), codes=w.numpy(), y=y.numpy(),
                        tiled=ref.transpose_tile(w).numpy())


if __name__ == "__main__":
    main()
