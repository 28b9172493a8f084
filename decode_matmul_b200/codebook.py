"""Codebook and input helpers: the E8P table, synthetic tables, int64 <-> fp16 views, random operands."""
from __future__ import annotations

from itertools import product

import torch


def build_codebook_abs(device) -> torch.Tensor:
    """The 256-entry E8P table as int64[256]; byte i of an entry is int8(4 * value_i).
    Same construction and entry order as the reference's ``build_codebook_abs``
    (test_decode_matmul.py:74-86): {0.5,1.5,2.5}^8 with the last coordinate negated on odd
    sums, the norm filter, one extra row, sorted by squared norm."""
    rows = []
    for xs in product((0.5, 1.5, 2.5), repeat=8):
        if sum(xs) % 2 != 0:
            xs = xs[:-1] + (-xs[-1],)
        z = sum(y * y for y in xs)
        small = all(abs(y) <= 1.5 for y in xs)
        if z <= 10 or (z == 12 and small and sum(abs(y) == 0.5 for y in xs[:4]) % 2 == 0):
            rows.append(xs)
    rows.append((0.5, 0.5, 0.5, 1.5, 1.5, 1.5, 1.5, -1.5))
    cb = torch.tensor(rows)
    cb = cb[cb.square().sum(1).argsort(), :]
    return pack_codebook(cb).to(device)


def pack_codebook(values: torch.Tensor) -> torch.Tensor:
    """[256, 8] real values (multiples of 1/4) -> int64[256]."""
    q = (values.to(torch.float64) * 4).round().to(torch.int64)
    if not torch.equal(q.to(torch.float64), values.to(torch.float64) * 4):
        raise RuntimeError("codebook values must be multiples of 1/4")
    shifts = 8 * torch.arange(8, device=values.device)
    return ((q & 255) << shifts).sum(1)


def codebook_to_fp16(cb64: torch.Tensor) -> torch.Tensor:
    """int64[256] -> fp16 [256, 8]: value = int8 byte / 4 (exact)."""
    b = cb64.contiguous().view(torch.int8).reshape(-1, 8)
    return (b.to(torch.float32) / 4).to(torch.float16)


def codebook_from_fp16(cb16: torch.Tensor) -> torch.Tensor:
    return pack_codebook(cb16.to(torch.float64))


def synthetic_codebook(seed: int = 42, device="cpu") -> torch.Tensor:
    """Seeded fp16 [256, 8] table with entries drawn uniformly from {0.5, 1.5, 2.5, 3.5}."""
    gen = torch.Generator().manual_seed(seed)
    m = torch.randint(0, 4, (256, 8), generator=gen)
    return (m.to(torch.float32) + 0.5).to(torch.float16).to(device)


def build_x_weights(M: int, N: int, K: int, device):
    """Random operands for the integer operator, as the reference's ``build_x_weights``
    (test_decode_matmul.py:89-98): ``x`` int8 [M, K] uniform over the whole int8 range and LOGICAL
    codes int16 [N, K/8] uniform over the whole int16 range, both drawn on ``device`` from
    torch's global generator (seed it with ``torch.random.manual_seed``).  Tile-pack the codes
    with ``transpose_tile`` before passing them to ``decode_matmul``."""
    x = torch.randint(-128, 128, size=(M, K), dtype=torch.int8, device=device)
    weights_compressed = torch.randint(-32768, 32768, size=(N, K // 8), dtype=torch.int16, device=device)
    return x, weights_compressed
