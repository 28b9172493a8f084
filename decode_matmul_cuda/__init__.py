"""Drop-in for the reference's ``decode_matmul_cuda`` extension module.

``from decode_matmul_cuda import decode_matmul`` keeps working: same name, same positional
arguments, same tensor layouts and dtypes, same int32 result
(decode_matmul_cuda/decode_matmul_cuda.cu:178-181,237-239).  Differences, all relaxations:
any M >= 1 and any K % 32 == 0 are accepted, the call does not synchronise the device, and
a CUDA error raises instead of ending the process.
"""
from decode_matmul_b200.ops import decode_matmul_fp16 as _fp16
from decode_matmul_b200.ops import decode_matmul_i8 as _i8
from decode_matmul_b200.ops import decode_weights  # noqa: F401  (fp16-family addition)


def decode_matmul(x, weights_compressed, codebook_abs):
    """Fused Decode Matrix Multiplication: returns a new int32 [M, N] tensor."""
    return _i8(x, weights_compressed, codebook_abs)


def decode_matmul_fp16(x, weights_compressed, codebook_fp16, scale=1.0):
    """fp16-activation variant: returns a new fp32 [M, N] tensor."""
    return _fp16(x, weights_compressed, codebook_fp16, scale)
