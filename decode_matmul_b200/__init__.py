"""decode_matmul_b200: B200 (sm_100a) codebook decode-and-matmul.

The product is the CUDA library ``libdmm.so`` behind the C ABI of ``include/dmm.h``; this
package is its PyTorch-facing host side.  Drop-in modules named like the reference's
extensions live at the repository root (``decode_matmul_cuda``, ``fast_decode_matmul_cuda``).
"""
from ._lib import (FLAG_ACCUMULATE, FLAG_ATOMIC, FLAG_PDL, LAYOUT_FAST, LAYOUT_TILE, PATH_AUTO, PATH_GEMV, PATH_TCGEN05, PATH_TCGEN05_F8,
                   SIGN_FAST, SIGN_SLOW, X_F16, X_F32, X_F32_SILU_MUL)
from .codebook import (build_codebook_abs, build_x_weights, codebook_from_fp16, codebook_to_fp16, pack_codebook,
                       synthetic_codebook)
from .layout import convert_sign_convention, fast_pack, fast_unpack, shard_cols, shard_fused_rows, shard_rows, transpose_tile, untranspose_tile
from .ops import decode_matmul_chain, decode_matmul_fused, decode_matmul_fp16, decode_matmul_fp16_noalloc, decode_matmul_i8, decode_weights, hint_next_weights, launch_count, set_wait_limit_ms, status, workspace_bytes, xrank_allreduce_add, xrank_barrier

__all__ = [
    "decode_matmul_i8", "decode_matmul_fp16", "decode_matmul_fp16_noalloc", "decode_matmul_fused", "decode_matmul_chain", "X_F16", "X_F32", "X_F32_SILU_MUL", "decode_weights", "status", "launch_count", "hint_next_weights", "set_wait_limit_ms", "workspace_bytes", "xrank_barrier", "xrank_allreduce_add",
    "transpose_tile", "untranspose_tile", "fast_pack", "fast_unpack", "shard_rows", "shard_cols", "shard_fused_rows",
    "build_codebook_abs", "build_x_weights", "convert_sign_convention", "pack_codebook", "codebook_to_fp16", "codebook_from_fp16", "synthetic_codebook",
    "SIGN_SLOW", "SIGN_FAST", "LAYOUT_TILE", "LAYOUT_FAST", "PATH_AUTO", "PATH_GEMV", "PATH_TCGEN05", "PATH_TCGEN05_F8",
    "FLAG_ACCUMULATE", "FLAG_PDL", "FLAG_ATOMIC",
]
