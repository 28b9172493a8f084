"""The oracle against the reference's own outputs (tests/golden, made by make_golden.py)."""
import ctypes

import numpy as np

from oracle import dmm_oracle as o


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_codebook_same_entries_as_reference(golden):
    ref = golden["e8p_codebook"]["codebook_abs"]
    mine = o.build_codebook_abs()
    assert ref.shape == (256,) and ref.dtype == np.int64
    assert sorted(ref.tolist()) == sorted(mine.tolist())
    assert np.array_equal(o.golden_codebook_abs(), ref)
    b = o.unpack_codebook(ref)
    assert set(np.unique(b).tolist()) == {-10, -6, -2, 2, 6, 10}
    assert (b[:, :7] > 0).all()  # negatives only in the last column
    assert np.array_equal(o.pack_codebook(b / 4.0), ref)
    assert np.array_equal(o.cb16_to_cb64(o.cb64_to_cb16(ref)), ref)


def test_decode_table_all_codes(golden):
    cb = golden["e8p_codebook"]["codebook_abs"]
    assert np.array_equal(o.decode_table(cb, o.SIGN_SLOW), golden["decode_all_codes"]["table"])


def test_known_answers(golden):
    table = o.decode_table(golden["e8p_codebook"]["codebook_abs"])
    known = {
        0x0000: [3, 3, 3, 3, 3, 3, 3, 3],
        0x8000: [1, 1, 1, 1, 1, 1, 1, 1],
        0x0100: [-1, 3, 3, 3, 3, 3, 3, -1],
        0xFFFF: [-7, -3, -3, -7, -3, -7, -7, 5],
        0x3039: [3, 7, 7, 3, -1, -1, 7, -1],
    }
    for code, want in known.items():
        assert table[code].tolist() == want
    assert set(np.unique(table).tolist()) == set(range(-11, 12, 2))


def test_c_oracle_matches(golden, oracle_c):
    cb = np.ascontiguousarray(golden["e8p_codebook"]["codebook_abs"])
    t = np.zeros((65536, 8), np.int8)
    oracle_c.oracle_decode_table(_p(cb), 0, _p(t))
    assert np.array_equal(t, golden["decode_all_codes"]["table"])
    oracle_c.oracle_decode_table(_p(cb), 1, _p(t))
    assert np.array_equal(t, o.decode_table(cb, o.SIGN_FAST))


def test_fast_convention_is_a_sign_permutation(golden):
    cb = golden["e8p_codebook"]["codebook_abs"]
    slow, fast = o.decode_table(cb, o.SIGN_SLOW), o.decode_table(cb, o.SIGN_FAST)
    codes = np.arange(65536)
    s_slow, s_fast = o.sign_bits(codes, o.SIGN_SLOW), o.sign_bits(codes, o.SIGN_FAST)
    assert np.array_equal(s_fast[:, 1:], s_slow[:, :7]) and np.array_equal(s_fast[:, 0], s_slow[:, 7])
    assert (s_slow.sum(1) % 2 == 0).all() and (s_fast.sum(1) % 2 == 0).all()
    assert not np.array_equal(slow, fast)


def test_tile_layout(golden):
    g = golden["transpose_tile"]
    assert np.array_equal(o.tile_pack(g["logical"]), g["tiled"])
    assert np.array_equal(o.tile_unpack(g["tiled"]), g["logical"])
    n, k8 = g["logical"].shape
    flat = g["tiled"].reshape(-1)
    for (nn, j) in [(0, 0), (5, 7), (9, 3), (17, 12), (63, 31)]:
        nt, h, gg, kt, t = nn // 16, (nn % 16) // 8, nn % 8, j // 4, j % 4
        assert flat[((nt * (k8 // 4) + kt) * 8 + gg) * 8 + 2 * t + h] == g["logical"][nn, j]


def test_c_tile_pack(golden, oracle_c):
    g = golden["transpose_tile"]
    logical = np.ascontiguousarray(g["logical"])
    out = np.zeros_like(logical)
    oracle_c.oracle_tile_pack(_p(logical), ctypes.c_int64(logical.shape[0]), ctypes.c_int64(logical.shape[1] * 8), _p(out))
    assert np.array_equal(out, g["tiled"])


def test_fast_layout_roundtrip():
    rng = np.random.default_rng(1)
    c = rng.integers(-32768, 32768, size=(64, 24)).astype(np.int16)
    assert np.array_equal(o.fast_unpack(o.fast_pack(c)), c)


def test_matmul_against_reference_loops(golden, oracle_c):
    cb = np.ascontiguousarray(golden["e8p_codebook"]["codebook_abs"])
    cases = [(golden["matmul_small"][f"x_{t}"], golden["matmul_small"][f"codes_{t}"], golden["matmul_small"][f"y_{t}"])
             for t in "ab"]
    r = golden["matmul_ref_shape"]
    cases.append((r["x"], r["codes"], r["y"]))
    for x, codes, y in cases:
        assert np.array_equal(o.decode_matmul_int(x, codes, cb), y)
        x, codes = np.ascontiguousarray(x), np.ascontiguousarray(codes)
        out = np.zeros(y.shape, np.int32)
        m, k = x.shape
        oracle_c.oracle_matmul_i8(_p(x), _p(codes), _p(cb), 0, ctypes.c_int64(m), ctypes.c_int64(codes.shape[0]),
                                  ctypes.c_int64(k), _p(out))
        assert np.array_equal(out, y)


def test_fp16_family_is_the_integer_decode_in_quarter_units(golden):
    cb = golden["e8p_codebook"]["codebook_abs"]
    rng = np.random.default_rng(3)
    codes = rng.integers(-32768, 32768, size=(32, 16)).astype(np.int16)
    w4 = o.decode_weights(codes, cb)
    w16 = o.decode_weights_f16(codes, o.cb64_to_cb16(cb))
    assert np.array_equal(w16.astype(np.float32) * 4, w4.astype(np.float32))
    x = rng.standard_normal((2, 128)).astype(np.float16)
    y = o.decode_matmul_f16(x, codes, o.cb64_to_cb16(cb), 0.5)
    want = 0.5 * (x.astype(np.float64) @ (w4.astype(np.float64) / 4).T)
    assert np.allclose(y, want, rtol=1e-6, atol=1e-6)
    syn = o.synthetic_codebook(42)
    assert syn.shape == (256, 8) and set(np.unique(syn).tolist()) == {0.5, 1.5, 2.5, 3.5}


def test_worst_case_sum_fits_int32(golden):
    table = golden["decode_all_codes"]["table"].astype(np.int64)
    assert np.abs(table).max() * 128 * 28672 < 2 ** 31
