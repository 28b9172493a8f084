"""Parity on the shapes the benchmark measures: the Llama-2-70B layer shapes of the stack step
(incl. the fused 57344 x 8192 gate+up launch and K = 28672, where fp32 accumulation is tightest)
and the batch sweep on the Llama-2-7B gate/up and down shapes.  Every output element is compared
with the C restatement of the reference's decode-then-matmul (test_decode_matmul.py:58-71; double
accumulation, OpenMP).  Needs a B200."""
import ctypes

import numpy as np
import pytest
import torch

import decode_matmul_b200 as dmm
from oracle import dmm_oracle as o

pytestmark = pytest.mark.gpu

MAX_ABS_ERR = 1e-2  # fp16 family: |y| is a few hundred at these K, so this is about 3e-5 relative
REL_L2 = 1e-3


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(-32768, 32768, size=(N, K // 8), dtype=np.int16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    return codes, x


def _oracle_f16(oracle_c, x, codes, cb16, scale):
    M, K = x.shape
    N = codes.shape[0]
    out = np.empty((M, N), np.float32)
    xf = np.ascontiguousarray(x.astype(np.float32))
    cb64 = np.ascontiguousarray(o.cb16_to_cb64(cb16))
    oracle_c.oracle_matmul_f64acc(_p(xf), _p(codes), _p(cb64), 0, ctypes.c_double(scale), ctypes.c_int64(M),
                                  ctypes.c_int64(N), ctypes.c_int64(K), _p(out))
    return out


def _check(y, want, what):
    err = float(np.abs(y - want).max())
    rel = float(np.linalg.norm(y - want) / max(np.linalg.norm(want), 1e-30))
    assert err <= MAX_ABS_ERR and rel <= REL_L2, f"{what}: max abs err {err:.3e}, rel L2 {rel:.3e}"
    return err, rel


LLAMA70B = [(1, 28672, 8192), (16, 28672, 8192), (32, 28672, 8192), (1, 8192, 28672), (16, 8192, 28672),
            (1, 57344, 8192), (1, 10240, 8192), (16, 10240, 8192), (16, 8192, 8192)]
SWEEP_7B = [(B, N, K) for (N, K) in [(11008, 4096), (4096, 11008)] for B in (16, 32, 64)]


@pytest.mark.parametrize("M,N,K", LLAMA70B + SWEEP_7B)
def test_fp16_family_on_benchmark_shapes(M, N, K, oracle_c):
    codes, x = _inputs(M, N, K, 1000 + M + N // 16 + K)
    cb16 = o.synthetic_codebook(42)
    want = _oracle_f16(oracle_c, x, codes, cb16, 1.0)
    tiled, cb = _dev(o.tile_pack(codes)), _dev(cb16)
    y = dmm.decode_matmul_fp16(_dev(x), tiled, cb, 1.0).cpu().numpy()
    _check(y, want, f"auto path {M}x{N}x{K}")
    if M <= 32:  # the mode the stack step runs: atomic accumulation onto what the buffer holds
        base = np.random.default_rng(5).standard_normal((M, N)).astype(np.float32)
        out = _dev(base)
        dmm.decode_matmul_fp16(_dev(x), tiled, cb, 1.0, out, accumulate=True, atomic=True, pdl=True)
        _check(out.cpu().numpy(), base + want, f"atomic {M}x{N}x{K}")
    assert dmm.status() == 0


def test_fused_gate_up_launch_of_the_stack(oracle_c):
    """The widest launch of the benchmark (55 % of its bytes): 57344 x 8192, fp32 activations rounded to
    fp16 by the loaders, atomic accumulation, the output cleared on the way by the call before."""
    M, N, K = 1, 57344, 8192
    codes, x = _inputs(M, N, K, 77)
    cb16 = o.synthetic_codebook(42)
    x32 = x.astype(np.float32) + np.float32(2.0 ** -14)  # not representable in fp16: the loaders must round
    xr = x32.astype(np.float16)
    want = _oracle_f16(oracle_c, xr, codes, cb16, 2.0 ** -7)
    tiled, cb = _dev(o.tile_pack(codes)), _dev(cb16)
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    dmm.decode_matmul_fused(_dev(x32), tiled, cb, 2.0 ** -7, out, x_kind=dmm.X_F32, accumulate=True, atomic=True, pdl=True)
    _check(out.cpu().numpy(), want, "fused gate+up")
    assert dmm.status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 28672, 8192), (8, 8192, 28672), (32, 10240, 8192)])
def test_int_family_on_benchmark_shapes(M, N, K, oracle_c):
    rng = np.random.default_rng(M + N + K)
    codes = rng.integers(-32768, 32768, size=(N, K // 8), dtype=np.int16)
    x = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    cb64 = np.ascontiguousarray(o.golden_codebook_abs())
    want = np.empty((M, N), np.int32)
    oracle_c.oracle_matmul_i8(_p(x), _p(codes), _p(cb64), 0, ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), _p(want))
    y = dmm.decode_matmul_i8(_dev(x), _dev(o.tile_pack(codes)), _dev(cb64))
    assert np.array_equal(y.cpu().numpy(), want)
    assert dmm.status() == 0


def test_accumulation_error_at_the_longest_reduction(oracle_c):
    """K = 28672 is where fp32 accumulation on the tensor core has the least room: print the error
    at scale 1 (|y| up to about 1500) and hold it to the absolute tolerance and to 1e-5 of max |y|."""
    M, N, K = 4, 8192, 28672
    codes, x = _inputs(M, N, K, 4242)
    cb16 = o.synthetic_codebook(42)
    want = _oracle_f16(oracle_c, x, codes, cb16, 1.0)
    y = dmm.decode_matmul_fp16(_dev(x), _dev(o.tile_pack(codes)), _dev(cb16), 1.0).cpu().numpy()
    err, rel = _check(y, want, "K = 28672")
    print(f"K=28672: max |y| {np.abs(want).max():.1f}, max abs err {err:.3e}, rel L2 {rel:.3e}")
    assert err <= 1e-5 * np.abs(want).max()


def test_fast_layout_streams_natively_on_a_benchmark_shape(oracle_c):
    """fast_decode_matmul_cuda.decode_matmul (fast layout, that file's sign convention, in-place accumulate)
    at 8 x 28672 x 8192: the tcgen05 kernel reads the fast layout as it lies in memory (no re-tiling pass);
    exact against the oracle, and the same codes converted to the other convention and the tile layout
    give the same integers through decode_matmul_cuda."""
    import decode_matmul_cuda as slow
    import fast_decode_matmul_cuda as fast

    M, N, K = 8, 28672, 8192
    rng = np.random.default_rng(99)
    codes = rng.integers(-32768, 32768, size=(N, K // 8), dtype=np.int16)
    x = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    cb64 = np.ascontiguousarray(o.golden_codebook_abs())
    want = np.empty((M, N), np.int32)
    oracle_c.oracle_matmul_i8(_p(x), _p(codes), _p(cb64), 1, ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), _p(want))
    launches = dmm.launch_count()
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    got = fast.decode_matmul(_dev(x), _dev(o.fast_pack(codes)), _dev(cb64), out)
    assert dmm.launch_count() == launches + 1, "one kernel: no re-tiling pass"
    assert np.array_equal(got.cpu().numpy(), want)
    # the converter: the same weights in the other convention and layout
    slow_codes = dmm.convert_sign_convention(torch.from_numpy(codes), dmm.SIGN_FAST, dmm.SIGN_SLOW)
    y = slow.decode_matmul(_dev(x), dmm.transpose_tile(slow_codes).cuda(), _dev(cb64))
    assert np.array_equal(y.cpu().numpy(), want)
    # fp16 family on the fast layout, batch 1 and 20 (the wide variant)
    cb16 = o.synthetic_codebook(42)
    for B in (1, 20):
        xh = rng.standard_normal((B, K)).astype(np.float16)
        yh = dmm.decode_matmul_fp16(_dev(xh), _dev(o.fast_pack(codes)), _dev(cb16), 1.0, layout=dmm.LAYOUT_FAST).cpu().numpy()
        _check(yh, _oracle_f16(oracle_c, xh, codes, cb16, 1.0), f"fp16 fast layout batch {B}")
    assert dmm.status() == 0
