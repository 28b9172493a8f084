"""Drop-in for the reference's ``fast_decode_matmul_cuda`` extension module.

``decode_matmul(x, weights_compressed, codebook_abs, output)`` accumulates into ``output``
and returns it (decode_matmul_cuda/fast_decode_matmul_cuda.cu:137-141,183,187-189), with
that file's sign convention (parity -> weight 0, fast_decode_matmul_cuda.cu:52-53).
"""
from decode_matmul_b200 import _lib
from decode_matmul_b200.ops import decode_matmul_i8 as _i8


def decode_matmul(x, weights_compressed, codebook_abs, output):
    """Fused Decode Matrix Multiplication, in place: output += x . decode(codes)^T."""
    return _i8(x, weights_compressed, codebook_abs, output, sign_convention=_lib.SIGN_FAST,
               layout=_lib.LAYOUT_FAST, accumulate=True)
