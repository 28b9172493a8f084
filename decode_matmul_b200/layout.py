"""Code-matrix layouts: logical [N, K/8] <-> what the kernels stream.

Works on tensors of any device; these are offline packing steps, not part of a forward pass.
"""
from __future__ import annotations

import torch


def transpose_tile(codes: torch.Tensor) -> torch.Tensor:
    """Logical int16 [N, K/8] -> tile layout of ``decode_matmul_cuda`` (same contract as the
    reference's ``transpose_tile``, test_decode_matmul.py:101-109): flat order
    [N/16][K/32][g:8][t:4][h:2] with row n = 16*nt + 8*h + g and code column j = 4*kt + t.
    The returned tensor keeps the shape [N, K/8]."""
    n, k8 = codes.shape
    if n % 16 or k8 % 4:
        raise RuntimeError("transpose_tile: need N % 16 == 0 and K % 32 == 0")
    t = codes.reshape(n // 16, 2, 8, k8 // 4, 4).permute(0, 3, 2, 4, 1)
    return t.contiguous().reshape(n, k8)


def untranspose_tile(tiled: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`transpose_tile`."""
    n, k8 = tiled.shape
    t = tiled.reshape(n // 16, k8 // 4, 8, 4, 2).permute(0, 4, 2, 1, 3)
    return t.contiguous().reshape(n, k8)


def fast_pack(codes: torch.Tensor) -> torch.Tensor:
    """Logical int16 [N, K/8] -> the layout of ``fast_decode_matmul_cuda``: flat uint32 order
    [N/32][K/16][lane:32], word = code(n = 32*nb + lane, j = 2*kp) | code(j = 2*kp + 1) << 16.
    The reference's fast kernel reads one such word per lane, a warp covering 32 consecutive
    output columns (fast_decode_matmul_cuda.cu:106,110-113,130); its k addressing is not
    self-consistent, so this build defines the completion.  Shape stays [N, K/8]."""
    n, k8 = codes.shape
    if n % 32 or k8 % 4:
        raise RuntimeError("fast_pack: need N % 32 == 0 and K % 32 == 0")
    t = codes.reshape(n // 32, 32, k8 // 2, 2).permute(0, 2, 1, 3)
    return t.contiguous().reshape(n, k8)


def fast_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`fast_pack`."""
    n, k8 = packed.shape
    t = packed.reshape(n // 32, k8 // 2, 32, 2).permute(0, 2, 1, 3)
    return t.contiguous().reshape(n, k8)


def shard_rows(codes: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Column-parallel shard (split N) of a LOGICAL code matrix."""
    n = codes.shape[0]
    if n % (16 * world):
        raise RuntimeError("shard_rows: N must be a multiple of 16 * world")
    step = n // world
    return codes[rank * step:(rank + 1) * step]


def shard_cols(codes: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Row-parallel shard (split K) of a LOGICAL code matrix; tile-pack each shard afterwards."""
    k8 = codes.shape[1]
    if k8 % (4 * world):
        raise RuntimeError("shard_cols: K must be a multiple of 32 * world")
    step = k8 // world
    return codes[:, rank * step:(rank + 1) * step]
