"""The no-allocation entry point, dmm_f16_noalloc, against dmm_f16.

Collected last on purpose (file name): a run that stops at the first failure has then
already run every other test.  The entry point serves callers that cannot let the library
call cudaMalloc (a process whose own allocator holds all device memory, a loop that cannot
afford the allocator lock); its scratch is a fixed array inside the library.  Two calls in a row must both
match the allocating entry point: the array keeps the first call's contents, and the second
call has to cope with that.
"""
import numpy as np
import pytest
import torch

import decode_matmul_b200 as dmm
from oracle import dmm_oracle as o

pytestmark = pytest.mark.gpu

MAX_ABS_ERR = 1e-2
REL_L2 = 1e-3


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 1040, 2080), (3, 8192, 8192)])
def test_noalloc_matches_allocating_entry_point(M, N, K):
    rng = np.random.default_rng(N + K + M)
    cb16 = o.synthetic_codebook(42)
    codes = rng.integers(-32768, 32768, size=(N, K // 8)).astype(np.int16)
    tiled, cb = _dev(o.tile_pack(codes)), _dev(cb16)
    for call in range(2):  # two calls in a row share the scratch array
        x = rng.standard_normal((M, K)).astype(np.float16)
        want = dmm.decode_matmul_fp16(_dev(x), tiled, cb, 0.5, path=dmm.PATH_TCGEN05_F8).cpu().numpy()
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        got = dmm.decode_matmul_fp16_noalloc(_dev(x), tiled, cb, 0.5, out)
        assert got.data_ptr() == out.data_ptr()
        got = got.cpu().numpy()
        err = np.abs(got - want).max()
        rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
        assert err <= MAX_ABS_ERR and rel <= REL_L2, f"call {call}: max abs err {err}, rel L2 {rel}"
        oracle = o.decode_matmul_f16(x, codes, cb16, 0.5)
        assert np.abs(got - oracle).max() <= MAX_ABS_ERR
    assert dmm.status() == 0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    x = torch.zeros((9, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((16, 8), dtype=torch.int16, device="cuda")
    cb = _dev(o.synthetic_codebook(42))
    out = torch.zeros((9, 16), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="fixed scratch"):
        dmm.decode_matmul_fp16_noalloc(x, w, cb, 1.0, out)


_FRESH_PROCESS = r"""
import sys
sys.path.insert(0, sys.argv[1])
import torch
import decode_matmul_b200 as dmm
# dmm_f16_noalloc is the ONLY entry point of the library this process calls
M, N, K = 2, 4096, 4096
x = torch.randn(M, K, device="cuda", dtype=torch.float16)
w = torch.randint(-32768, 32768, (N, K // 8), dtype=torch.int16, device="cuda")
cb = dmm.synthetic_codebook(42, "cuda")
out = torch.empty(M, N, device="cuda", dtype=torch.float32)
dmm.decode_matmul_fp16_noalloc(x, w, cb, 1.0, out)   # first call: kernels and the scratch array are placed now
torch.cuda.synchronize()
first = out.clone()
free0, _ = torch.cuda.mem_get_info()
for _ in range(3):
    dmm.decode_matmul_fp16_noalloc(x, w, cb, 1.0, out)
torch.cuda.synchronize()
free1, _ = torch.cuda.mem_get_info()
W = None
ok = free0 == free1 and torch.equal(first, out) and bool(torch.isfinite(out).all())
print("FREE", free0, free1, "OK" if ok else "FAIL", flush=True)
sys.exit(0 if ok else 1)
"""


def test_noalloc_holds_no_new_device_memory_in_a_fresh_process(tmp_path):
    """The property itself: in a process whose only library call is dmm_f16_noalloc, the device's free
    memory is the same before and after further calls (the first call places the kernels and the fixed
    scratch array; nothing is allocated afterwards), and the calls agree with one another."""
    import os
    import subprocess
    import sys

    script = tmp_path / "fresh.py"
    script.write_text(_FRESH_PROCESS)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, str(script), root], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-1000:] + res.stderr[-2000:]
    assert "OK" in res.stdout


def test_noalloc_rejects_the_atomic_flag():
    """The fixed scratch serves the ticketed reduction only: DMM_FLAG_ATOMIC is an argument error here."""
    import ctypes

    from decode_matmul_b200 import _lib

    x = torch.zeros((1, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((16, 8), dtype=torch.int16, device="cuda")
    cb = _dev(o.synthetic_codebook(42))
    out = torch.zeros((1, 16), dtype=torch.float32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = _lib.lib().dmm_f16_noalloc(p(x), p(w), p(cb), 1.0, p(out), 1, 16, 64, 0, _lib.FLAG_ATOMIC, None)
    assert rc == -4
