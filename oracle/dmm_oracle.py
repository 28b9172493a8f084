"""CPU oracle for the codebook decode-and-matmul operator.  TEST INFRASTRUCTURE ONLY.

This module restates, in vectorised numpy, the algorithm that the reference
defines in ``test_decode_matmul.py``.  It is the checker used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.  Nothing on the product path may import it: the product
path is the CUDA library and fails loudly when that library is missing.

Parity status
-------------
* slow convention (``SIGN_SLOW``): PINNED.  ``tests/golden/make_golden.py`` runs the
  reference's own ``decode()``, ``build_codebook_abs()``, ``transpose_tile()`` and
  ``decode_matmul_torch()`` and stores their outputs; ``tests/test_oracle.py``
  checks every function here against those files.
* fast convention (``SIGN_FAST``): parity unpinned.  The reference has no CPU
  definition and no test of ``fast_decode_matmul_cuda.cu``; the sign map is
  restated from ``decode_matmul_cuda/fast_decode_matmul_cuda.cu:49-64``.
* fp16 family: parity unpinned by the reference (it has no fp16 path).  It is
  derived from the pinned integer decode: weight = decoded int8 / 4.

Code word (16 bit): bits 0..7 index the codebook, bits 8..14 are seven stored
sign bits, bit 15 is the shift bit (``test_decode_matmul.py:30-33``).
"""
from __future__ import annotations

import itertools

import numpy as np

SIGN_SLOW = 0  # decode_matmul_cuda.cu:50-53 / test_decode_matmul.py:31-32: parity -> weight 7
SIGN_FAST = 1  # fast_decode_matmul_cuda.cu:52-53: parity -> weight 0, stored bit j -> weight j+1


def build_codebook_abs() -> np.ndarray:
    """E8P table as int64[256]; byte i of an entry is int8(4 * value_i).

    Follows ``test_decode_matmul.py:74-86``: all tuples of {0.5,1.5,2.5}^8 in
    ``itertools.product`` order, last coordinate negated when the sum is odd,
    kept when the squared norm is <= 10 or in a norm-12 sub-family, one extra
    hand-added row, sorted by squared norm.  The reference sorts with torch's
    default (unstable) ``argsort``, so the order inside an equal-norm group is
    not defined by the algorithm: this restatement returns the same SET of 256
    entries in stable order, and the reference's actual order is pinned by
    ``tests/golden/e8p_codebook.npz`` (use ``golden_codebook_abs``).
    """
    rows = []
    for xs in itertools.product(*([[0.5, 1.5, 2.5]] * 8)):
        if sum(xs) % 2 != 0:
            xs = (*xs[:-1], -xs[-1])
        z = sum(y * y for y in xs)
        if z <= 10 or (
            z == 12
            and all(abs(y) <= 1.5 for y in xs)
            and (sum(abs(y) == 0.5 for y in xs[0:4]) % 2 == 0)
        ):
            rows.append(xs)
    rows.append((0.5, 0.5, 0.5, 1.5, 1.5, 1.5, 1.5, -1.5))
    cb = np.asarray(rows, dtype=np.float64)
    order = np.argsort((cb * cb).sum(1), kind="stable")
    cb = cb[order]
    return pack_codebook(cb)


def golden_codebook_abs() -> np.ndarray:
    """The E8P table exactly as the reference's ``build_codebook_abs`` returned it."""
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    return np.load(os.path.join(here, "..", "tests", "golden", "e8p_codebook.npz"))["codebook_abs"]


def pack_codebook(values: np.ndarray) -> np.ndarray:
    """[256,8] real values (multiples of 1/4) -> int64[256] (``test_decode_matmul.py:85``)."""
    q = np.rint(np.asarray(values, dtype=np.float64) * 4).astype(np.int64)
    assert np.all(q == np.asarray(values, dtype=np.float64) * 4), "codebook values must be multiples of 1/4"
    assert np.all((q >= -128) & (q <= 127))
    packed = np.zeros(q.shape[0], dtype=np.uint64)
    for i in range(8):
        packed |= (q[:, i] & 255).astype(np.uint64) << np.uint64(8 * i)
    return packed.view(np.int64)


def unpack_codebook(cb64: np.ndarray) -> np.ndarray:
    """int64[256] -> int8[256,8] (byte i of entry e), little-endian byte order."""
    cb64 = np.ascontiguousarray(np.asarray(cb64, dtype=np.int64))
    return cb64.view(np.uint8).reshape(-1, 8).view(np.int8).copy()


def cb64_to_cb16(cb64: np.ndarray) -> np.ndarray:
    """fp16 view of the table: value = int8 byte / 4 (exact in fp16)."""
    return (unpack_codebook(cb64).astype(np.float32) / 4).astype(np.float16)


def cb16_to_cb64(cb16: np.ndarray) -> np.ndarray:
    return pack_codebook(np.asarray(cb16, dtype=np.float64))


def synthetic_codebook(seed: int = 42) -> np.ndarray:
    """Seeded [256,8] fp16 table with entries drawn uniformly from {0.5,1.5,2.5,3.5}."""
    rng = np.random.default_rng(seed)
    return (rng.integers(0, 4, size=(256, 8)).astype(np.float32) + 0.5).astype(np.float16)


def sign_bits(codes: np.ndarray, convention: int) -> np.ndarray:
    """[...,] uint16 codes -> [...,8] bool, True where weight i is negated."""
    c = np.asarray(codes).astype(np.uint16).astype(np.uint32)
    s7 = (c >> 8) & 0x7F
    parity = np.zeros_like(s7)
    for b in range(7):
        parity ^= (s7 >> b) & 1
    if convention == SIGN_SLOW:
        s8 = s7 | (parity << 7)  # test_decode_matmul.py:31-32
    elif convention == SIGN_FAST:
        s8 = (s7 << 1) | parity  # fast_decode_matmul_cuda.cu:52-53
    else:
        raise ValueError("unknown sign convention")
    return ((s8[..., None] >> np.arange(8, dtype=np.uint32)) & 1).astype(bool)


def decode_table(cb64: np.ndarray, convention: int = SIGN_SLOW) -> np.ndarray:
    """All 65 536 code words -> int8[65536, 8] (= 4 x weight).

    Follows ``decode()`` (``test_decode_matmul.py:29-55``) step by step with
    int8 wrap-around: take byte i of the table entry as int8, negate it when
    the sign bit is set, then subtract one when the shift bit is set, else add one.
    """
    codes = np.arange(65536, dtype=np.uint32)
    table = unpack_codebook(cb64)  # int8 [256, 8]
    v = table[codes & 0xFF].astype(np.int16)  # test_decode_matmul.py:35,38
    neg = sign_bits(codes, convention)
    v = np.where(neg, -v, v).astype(np.int8).astype(np.int16)  # :41-42, int8 wrap of -(-128)
    shift = ((codes >> 15) & 1).astype(bool)[:, None]
    v = np.where(shift, v - 1, v + 1).astype(np.int8)  # :44-47
    return v


def decode_weights(codes: np.ndarray, cb64: np.ndarray, convention: int = SIGN_SLOW) -> np.ndarray:
    """logical codes int16 [N, K/8] -> int8 [N, K] (= 4 x weight)."""
    codes = np.asarray(codes)
    assert codes.dtype == np.int16 and codes.ndim == 2
    table = decode_table(cb64, convention)
    n, k8 = codes.shape
    return table[codes.view(np.uint16).astype(np.int64)].reshape(n, k8 * 8)


def decode_weights_f16(codes: np.ndarray, cb16: np.ndarray, convention: int = SIGN_SLOW) -> np.ndarray:
    """logical codes -> fp16 [N, K]; every value is an exact multiple of 1/4."""
    w4 = decode_weights(codes, cb16_to_cb64(cb16), convention)
    return (w4.astype(np.float32) / 4).astype(np.float16)


def decode_matmul_int(x: np.ndarray, codes: np.ndarray, cb64: np.ndarray, convention: int = SIGN_SLOW) -> np.ndarray:
    """int8 x [M,K] times decoded weights -> int32 [M,N] (``test_decode_matmul.py:58-71``)."""
    assert x.dtype == np.int8
    w = decode_weights(codes, cb64, convention).astype(np.int64)
    y = x.astype(np.int64) @ w.T
    return y.astype(np.int32)  # int32 accumulation wraps; never reached at supported sizes


def decode_matmul_f16(x: np.ndarray, codes: np.ndarray, cb16: np.ndarray, scale: float = 1.0,
                      convention: int = SIGN_SLOW) -> np.ndarray:
    """fp16 x [M,K] -> fp32 [M,N] = scale * (x @ W^T), accumulated in float64 then rounded once."""
    assert x.dtype == np.float16
    w = decode_weights_f16(codes, cb16, convention).astype(np.float64)
    return (float(scale) * (x.astype(np.float64) @ w.T)).astype(np.float32)


def tile_pack(codes: np.ndarray) -> np.ndarray:
    """logical [N, K/8] -> the tile layout of ``decode_matmul_cuda`` (``test_decode_matmul.py:101-109``).

    Flat order is [N/16][K/32][g:8][t:4][h:2] with row n = 16*nt + 8*h + g and
    code column j = 4*kt + t.  The result keeps the (misleading) shape [N, K/8].
    """
    n, k8 = codes.shape
    assert n % 16 == 0 and k8 % 4 == 0
    a = codes.reshape(n // 16, 2, 8, k8 // 4, 4)  # nt, h, g, kt, t
    a = a.transpose(0, 3, 2, 4, 1)  # nt, kt, g, t, h
    return np.ascontiguousarray(a).reshape(n, k8)


def tile_unpack(tiled: np.ndarray) -> np.ndarray:
    n, k8 = tiled.shape
    a = tiled.reshape(n // 16, k8 // 4, 8, 4, 2)  # nt, kt, g, t, h
    a = a.transpose(0, 4, 2, 1, 3)  # nt, h, g, kt, t
    return np.ascontiguousarray(a).reshape(n, k8)


def fast_pack(codes: np.ndarray) -> np.ndarray:
    """logical [N, K/8] -> the layout this build defines for ``fast_decode_matmul_cuda``.

    The reference's fast kernel reads one uint32 (two codes = 16 consecutive k of one
    output column) per lane, a warp covering 32 consecutive columns
    (``fast_decode_matmul_cuda.cu:106,110-113,130``); its k-addressing is not
    self-consistent, so the completion is defined here: flat uint32 order
    [N/32][K/16][lane:32], word = codes (n = 32*nb + lane, j = 2*kp) | (j = 2*kp+1) << 16.
    """
    n, k8 = codes.shape
    assert n % 32 == 0 and k8 % 2 == 0
    a = codes.reshape(n // 32, 32, k8 // 2, 2)  # nb, lane, kp, half
    a = a.transpose(0, 2, 1, 3)  # nb, kp, lane, half
    return np.ascontiguousarray(a).reshape(n, k8)


def fast_unpack(packed: np.ndarray) -> np.ndarray:
    n, k8 = packed.shape
    a = packed.reshape(n // 32, k8 // 2, 32, 2)
    a = a.transpose(0, 2, 1, 3)
    return np.ascontiguousarray(a).reshape(n, k8)


def convert_sign_convention(codes: np.ndarray, src: int, dst: int) -> np.ndarray:
    """codes such that decode(result, dst) == decode(codes, src), for every code word.

    Both conventions encode an even-parity vector of eight signs in seven stored bits
    (``decode_matmul_cuda.cu:50-53``: the parity is the sign of weight 7;
    ``fast_decode_matmul_cuda.cu:52-53``: of weight 0), so the map is a bijection."""
    c = np.asarray(codes).view(np.uint16).astype(np.uint32)
    if src == dst:
        return np.asarray(codes).copy()
    s7 = (c >> 8) & 0x7F
    par = np.zeros_like(s7)
    for b in range(7):
        par ^= (s7 >> b) & 1
    new = (s7 >> 1) | (par << 6) if src == SIGN_SLOW else ((s7 << 1) & 0x7F) | par
    return ((c & 0x80FF) | (new << 8)).astype(np.uint16).view(np.int16)
