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


def shard_fused_rows(codes: torch.Tensor, parts, world: int, rank: int) -> torch.Tensor:
    """Column-parallel shard of a LOGICAL code matrix whose rows are several projections fused
    along N (``parts`` = their row counts, e.g. q, k, v or gate, up): rank r gets the r-th slice of
    EVERY part, concatenated in the same order, so that its output is [q_r | k_r | v_r] and the
    row-parallel layer that follows can take its K-shard r of the next weight matrix."""
    if sum(parts) != codes.shape[0]:
        raise RuntimeError("shard_fused_rows: parts do not add up to N")
    out, row = [], 0
    for n in parts:
        if n % (16 * world):
            raise RuntimeError("shard_fused_rows: every part must be a multiple of 16 * world rows")
        step = n // world
        out.append(codes[row + rank * step:row + (rank + 1) * step])
        row += n
    return torch.cat(out, 0)


def shard_cols(codes: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Row-parallel shard (split K) of a LOGICAL code matrix; tile-pack each shard afterwards."""
    k8 = codes.shape[1]
    if k8 % (4 * world):
        raise RuntimeError("shard_cols: K must be a multiple of 32 * world")
    step = k8 // world
    return codes[:, rank * step:(rank + 1) * step]


def convert_sign_convention(codes: torch.Tensor, src: int, dst: int) -> torch.Tensor:
    """Re-encodes int16 codes (any layout: the map is per code word) so that decoding the result
    under sign convention ``dst`` gives what ``codes`` decode to under ``src``.

    Slow convention (decode_matmul_cuda.cu:50-53): stored bit i (code bit 8 + i) is the sign of
    weight i for i < 7 and the parity of the seven stored bits is the sign of weight 7.  Fast
    convention (fast_decode_matmul_cuda.cu:52-53): the parity is the sign of weight 0 and stored
    bit i is the sign of weight i + 1.  Either way the eight signs have even parity, and every
    even-parity sign vector has exactly one encoding in each convention, so the conversion is
    lossless for ALL 65 536 code words (a bijection; index byte and shift bit are untouched):
        slow -> fast: stored' = (stored >> 1) | (parity << 6)   (drop the sign of weight 0, which the
                                                                  new parity reproduces)
        fast -> slow: stored' = ((stored << 1) & 0x7F) | parity."""
    if src not in (0, 1) or dst not in (0, 1):
        raise RuntimeError("convert_sign_convention: conventions are 0 (slow) and 1 (fast)")
    if codes.dtype != torch.int16:
        raise RuntimeError("convert_sign_convention: codes must be int16")
    if src == dst:
        return codes.clone()
    c = codes.to(torch.int32) & 0xFFFF
    s7 = (c >> 8) & 0x7F
    par = s7 ^ (s7 >> 4)
    par = par ^ (par >> 2)
    par = (par ^ (par >> 1)) & 1
    new = (s7 >> 1) | (par << 6) if src == 0 else ((s7 << 1) & 0x7F) | par
    out = (c & 0x80FF) | (new << 8)
    return torch.where(out >= 32768, out - 65536, out).to(torch.int16)
