"""Host-side logic that needs no GPU: packers, codebooks, the C ABI's exports and its
argument validation (every check returns before any CUDA call)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import decode_matmul_b200 as dmm
from decode_matmul_b200 import _lib
from oracle import dmm_oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "dmm.h")).read()
    declared = set(re.findall(r"\b(dmm_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    L = _lib.lib()
    for name in declared:
        assert getattr(L, name) is not None
    assert L.dmm_version().decode().count(".") == 1


def test_constants_match_header():
    header = open(os.path.join(ROOT, "include", "dmm.h")).read()
    vals = {k: int(v.rstrip("u"), 0) for k, v in re.findall(r"#define (DMM_[A-Z0-9_]+) \(?(-?[0-9a-fx]+u?)\)?", header)}
    assert vals["DMM_SIGN_SLOW"] == _lib.SIGN_SLOW and vals["DMM_SIGN_FAST"] == _lib.SIGN_FAST
    assert vals["DMM_LAYOUT_TILE"] == _lib.LAYOUT_TILE and vals["DMM_LAYOUT_FAST"] == _lib.LAYOUT_FAST
    assert (vals["DMM_PATH_AUTO"], vals["DMM_PATH_GEMV"], vals["DMM_PATH_TCGEN05"]) == (0, 1, 2)
    assert vals["DMM_FLAG_ACCUMULATE"] == _lib.FLAG_ACCUMULATE and vals["DMM_FLAG_PDL"] == _lib.FLAG_PDL


def test_argument_errors_are_status_codes_not_crashes():
    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    a = ctypes.addressof(buf)
    a = (a + 255) & ~255
    p = ctypes.c_void_p(a)
    assert L.dmm_i8(None, p, p, p, 8, 16, 32, 0, 0, 0, None, 0, None) == -1
    assert L.dmm_i8(p, p, p, p, 0, 16, 32, 0, 0, 0, None, 0, None) == -2
    assert L.dmm_i8(p, p, p, p, 8, 24, 32, 0, 0, 0, None, 0, None) == -2
    assert L.dmm_i8(p, p, p, p, 8, 16, 48, 0, 0, 0, None, 0, None) == -2
    assert L.dmm_i8(ctypes.c_void_p(a + 4), p, p, p, 8, 16, 32, 0, 0, 0, None, 0, None) == -3
    assert L.dmm_i8(p, p, p, p, 8, 16, 32, 7, 0, 0, None, 0, None) == -4
    assert L.dmm_f16(p, p, p, 1.0, p, 8, 16, 32, 0, 0, 9, 0, None, 0, None) == -4
    assert L.dmm_decode(p, None, 0, p, 16, 32, 0, 0, None) == -1
    assert L.dmm_status(None) == -1
    for code in (0, -1, -2, -3, -4, -5, -6):
        assert len(L.dmm_error_string(code)) > 0


def test_python_wrappers_reject_bad_tensors():
    x = torch.zeros((8, 64), dtype=torch.int8)
    w = torch.zeros((16, 8), dtype=torch.int16)
    cb = torch.zeros(256, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        dmm.decode_matmul_i8(x, w, cb)
    import decode_matmul_cuda
    import fast_decode_matmul_cuda
    with pytest.raises(RuntimeError):
        decode_matmul_cuda.decode_matmul(x, w, cb)
    with pytest.raises(RuntimeError):
        fast_decode_matmul_cuda.decode_matmul(x, w, cb, torch.zeros((8, 16), dtype=torch.int32))


def test_transpose_tile_matches_reference(golden):
    g = golden["transpose_tile"]
    t = dmm.transpose_tile(torch.from_numpy(g["logical"]))
    assert np.array_equal(t.numpy(), g["tiled"])
    assert np.array_equal(dmm.untranspose_tile(t).numpy(), g["logical"])
    with pytest.raises(RuntimeError):
        dmm.transpose_tile(torch.zeros((8, 4), dtype=torch.int16))


def test_codebooks(golden):
    cb = dmm.build_codebook_abs("cpu")
    assert np.array_equal(cb.numpy(), golden["e8p_codebook"]["codebook_abs"])
    cb16 = dmm.codebook_to_fp16(cb)
    assert np.array_equal(cb16.numpy(), o.cb64_to_cb16(cb.numpy()))
    assert torch.equal(dmm.codebook_from_fp16(cb16), cb)
    syn = dmm.synthetic_codebook(42)
    assert syn.shape == (256, 8) and syn.dtype == torch.float16
    assert set(syn.unique().tolist()) == {0.5, 1.5, 2.5, 3.5}
    with pytest.raises(RuntimeError):
        dmm.pack_codebook(torch.full((256, 8), 0.3))


def test_shards_tile_independently():
    rng = np.random.default_rng(5)
    codes = torch.from_numpy(rng.integers(-32768, 32768, size=(64, 32)).astype(np.int16))
    rows = [dmm.shard_rows(codes, 2, r) for r in range(2)]
    # a column-parallel shard of the tiled matrix is a contiguous byte range of it
    whole = dmm.transpose_tile(codes).reshape(-1)
    for r in range(2):
        assert torch.equal(dmm.transpose_tile(rows[r]).reshape(-1), whole[r * whole.numel() // 2:(r + 1) * whole.numel() // 2])
    cols = [dmm.shard_cols(codes, 2, r) for r in range(2)]
    assert torch.equal(torch.cat(cols, 1), codes)


def test_fast_layout_packers_match_oracle():
    import numpy as np
    import torch

    from decode_matmul_b200 import layout
    from oracle import dmm_oracle as o

    rng = np.random.default_rng(4)
    codes = rng.integers(-32768, 32768, size=(96, 40)).astype(np.int16)
    t = torch.from_numpy(codes)
    packed = layout.fast_pack(t)
    assert np.array_equal(packed.numpy(), o.fast_pack(codes))
    assert torch.equal(layout.fast_unpack(packed), t)
    with pytest.raises(RuntimeError):
        layout.fast_pack(t[:48])  # N % 32


def test_sign_convention_converter_is_lossless_on_every_code_word(golden):
    """decode(convert(c, src, dst), dst) == decode(c, src) for all 65 536 code words, both ways:
    the slow map (decode_matmul_cuda.cu:50-53) and the fast map (fast_decode_matmul_cuda.cu:52-53)
    both encode an even-parity sign vector, so the conversion is a bijection."""
    codes = np.arange(65536, dtype=np.uint16).view(np.int16)
    cb = np.ascontiguousarray(golden["e8p_codebook"]["codebook_abs"])
    slow, fast = o.decode_table(cb, o.SIGN_SLOW), o.decode_table(cb, o.SIGN_FAST)
    assert np.array_equal(slow, golden["decode_all_codes"]["table"])  # the pinned side
    t = torch.from_numpy(codes)
    to_fast = dmm.convert_sign_convention(t, dmm.SIGN_SLOW, dmm.SIGN_FAST).numpy()
    to_slow = dmm.convert_sign_convention(t, dmm.SIGN_FAST, dmm.SIGN_SLOW).numpy()
    assert np.array_equal(fast[to_fast.view(np.uint16)], slow)
    assert np.array_equal(slow[to_slow.view(np.uint16)], fast)
    assert np.array_equal(to_fast, o.convert_sign_convention(codes, o.SIGN_SLOW, o.SIGN_FAST))
    assert np.array_equal(to_slow, o.convert_sign_convention(codes, o.SIGN_FAST, o.SIGN_SLOW))
    back = dmm.convert_sign_convention(torch.from_numpy(to_fast), dmm.SIGN_FAST, dmm.SIGN_SLOW)
    assert torch.equal(back, t)
    assert len(np.unique(to_fast.view(np.uint16))) == 65536
    # index byte and shift bit are untouched
    assert np.array_equal(to_fast.view(np.uint16) & 0x80FF, codes.view(np.uint16) & 0x80FF)
    with pytest.raises(RuntimeError):
        dmm.convert_sign_convention(t.to(torch.int32), 0, 1)


def test_build_x_weights_shapes_and_ranges():
    """Same contract as the reference's input builder (test_decode_matmul.py:89-98)."""
    torch.random.manual_seed(42)
    x, w = dmm.build_x_weights(8, 64, 4096, "cpu")
    assert x.dtype == torch.int8 and tuple(x.shape) == (8, 4096)
    assert w.dtype == torch.int16 and tuple(w.shape) == (64, 512)
    assert int(x.min()) == -128 and int(x.max()) == 127
    assert int(w.min()) < -32000 and int(w.max()) > 32000
    torch.random.manual_seed(42)
    x2, w2 = dmm.build_x_weights(8, 64, 4096, "cpu")
    assert torch.equal(x, x2) and torch.equal(w, w2)


def test_workspace_bytes_without_a_gpu():
    """dmm_workspace_bytes is host arithmetic (tickets + stream-K partial sums + activation planes): callable
    without a device, positive for valid shapes, growing with the batch, and what LinearStack sizes its own
    scratch by."""
    import decode_matmul_b200 as dmm

    small = dmm.workspace_bytes(1, 8192, 8192)
    big = dmm.workspace_bytes(32, 57344, 8192)
    assert small > 0 and big >= small
    assert dmm.workspace_bytes(1, 8, 64) == 0  # fewer than 16 rows: no such product
