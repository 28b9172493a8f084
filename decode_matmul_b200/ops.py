"""PyTorch-facing operators over the C ABI of libdmm.

PyTorch is used for device memory and streams only: every function checks its tensors,
takes raw pointers and the current CUDA stream, and calls one entry point of
include/dmm.h.  Nothing here computes on the CPU and nothing synchronises the device.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_input(t: torch.Tensor, name: str, dtype: torch.dtype) -> None:
    # same checks as CHECK_INPUT / TORCH_CHECK(scalar_type) in decode_matmul_cuda.cu:16-18,186-188
    _req(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _req(t.is_cuda, f"{name} must be a CUDA tensor")
    _req(t.is_contiguous(), f"{name} must be contiguous")
    _req(t.dtype == dtype, f"{name} must have dtype {dtype}")


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def decode_matmul_i8(x, weights_compressed, codebook_abs, output=None, *, sign_convention=_lib.SIGN_SLOW,
                     layout=_lib.LAYOUT_TILE, accumulate=False, pdl=False):
    """int32 [M, N] = x (int8 [M, K]) . decode(codes)^T, exact.

    ``weights_compressed`` is int16 [N, K/8] in the given layout, ``codebook_abs`` int64[256].
    With ``output`` given the result is written (or, with ``accumulate``, added) in place and
    the same tensor is returned; otherwise a new tensor is returned
    (decode_matmul_cuda.cu:178-234, fast_decode_matmul_cuda.cu:137-184)."""
    _check_input(x, "x", torch.int8)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_abs, "codebook_abs", torch.int64)
    _req(x.dim() == 2 and weights_compressed.dim() == 2, "x and weights_compressed must be 2-D")
    _req(codebook_abs.numel() == 256, "codebook_abs must have 256 entries")
    _req(x.size(-1) == weights_compressed.size(-1) << 3, "x.size(-1) must equal 8 * weights_compressed.size(-1)")
    M, K = x.shape
    N = weights_compressed.size(0)
    with torch.cuda.device(x.device):
        if output is None:
            _req(not accumulate, "accumulate needs an output tensor")
            output = torch.empty((M, N), dtype=torch.int32, device=x.device)
        else:
            _check_input(output, "output", torch.int32)
            _req(tuple(output.shape) == (M, N), "output must have shape [M, N]")
        flags = (_lib.FLAG_ACCUMULATE if accumulate else 0) | (_lib.FLAG_PDL if pdl else 0)
        rc = _lib.lib().dmm_i8(_ptr(x), _ptr(weights_compressed), _ptr(codebook_abs), _ptr(output), M, N, K,
                               sign_convention, layout, flags, None, 0, _stream_ptr(x.device))
    _lib.check(rc, "decode_matmul")
    return output


def decode_matmul_fp16(x, weights_compressed, codebook_fp16, scale=1.0, output=None, *,
                       sign_convention=_lib.SIGN_SLOW, layout=_lib.LAYOUT_TILE, path=_lib.PATH_AUTO,
                       accumulate=False, pdl=False, atomic=False):
    """fp32 [M, N] = scale * x (fp16 [M, K]) . W^T with W = decode(codes) / 4, fp32 accumulation.
    ``codebook_fp16`` is fp16 [256, 8] whose entries are odd multiples of 1/2."""
    _check_input(x, "x", torch.float16)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    _req(x.dim() == 2 and weights_compressed.dim() == 2, "x and weights_compressed must be 2-D")
    _req(tuple(codebook_fp16.shape) == (256, 8), "codebook_fp16 must have shape [256, 8]")
    _req(x.size(-1) == weights_compressed.size(-1) << 3, "x.size(-1) must equal 8 * weights_compressed.size(-1)")
    M, K = x.shape
    N = weights_compressed.size(0)
    with torch.cuda.device(x.device):
        if output is None:
            _req(not accumulate, "accumulate needs an output tensor")
            output = torch.empty((M, N), dtype=torch.float32, device=x.device)
        else:
            _check_input(output, "output", torch.float32)
            _req(tuple(output.shape) == (M, N), "output must have shape [M, N]")
        _req(not atomic or accumulate, "atomic reduction adds into output: pass accumulate=True (and zero it first)")
        flags = ((_lib.FLAG_ACCUMULATE if accumulate else 0) | (_lib.FLAG_PDL if pdl else 0)
                 | (_lib.FLAG_ATOMIC if atomic else 0))
        rc = _lib.lib().dmm_f16(_ptr(x), _ptr(weights_compressed), _ptr(codebook_fp16), float(scale), _ptr(output),
                                M, N, K, sign_convention, layout, path, flags, None, 0, _stream_ptr(x.device))
    _lib.check(rc, "decode_matmul_fp16")
    return output


def decode_matmul_fused(x, weights_compressed, codebook_fp16, scale, output, *, x_kind=_lib.X_F32, k=None, x_gap=0,
                        sign_convention=_lib.SIGN_SLOW, accumulate=False, pdl=False, atomic=False, zero=None,
                        workspace=None):
    """``decode_matmul_fp16`` reading the previous layer's fp32 output directly.

    ``x`` is fp32 [M, ld] (or fp16 with ``x_kind=X_F16``); the kernel's loaders round it to fp16
    themselves (``X_F32``) or first form ``silu(x[:, :k]) * x[:, x_gap:x_gap + k]``
    (``X_F32_SILU_MUL``), so no separate cast / activation kernel runs between two layers.
    ``k`` is the reduction length (default: the whole row); the result is written or added to
    ``output`` (fp32 [M, N]).  ``zero``: an fp32 tensor that this kernel clears on its way (the
    output of a later ``atomic`` call); it must not be an operand of this call or the one before.
    ``workspace``: a zero-initialised uint8 tensor of at least ``workspace_bytes(M, N, K)`` bytes that this
    call uses as scratch instead of the library's buffer (calls that may overlap on the GPU, e.g. two stacks
    on two streams, need distinct ones)."""
    _check_input(x, "x", torch.float16 if x_kind == _lib.X_F16 else torch.float32)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    _check_input(output, "output", torch.float32)
    _req(x.dim() == 2 and weights_compressed.dim() == 2, "x and weights_compressed must be 2-D")
    M, ld = x.shape
    N, K = weights_compressed.size(0), weights_compressed.size(1) * 8
    _req(k is None or k == K, "k must equal 8 * weights_compressed.size(-1)")
    _req(ld >= K, "x rows are shorter than the reduction length")
    _req(tuple(output.shape) == (M, N), "output must have shape [M, N]")
    _req(not atomic or accumulate, "atomic reduction adds into output: pass accumulate=True")
    if zero is not None:
        _check_input(zero, "zero", torch.float32)
    flags = ((_lib.FLAG_ACCUMULATE if accumulate else 0) | (_lib.FLAG_PDL if pdl else 0)
             | (_lib.FLAG_ATOMIC if atomic else 0))
    with torch.cuda.device(x.device):
        rc = _lib.lib().dmm_f16_fused(_ptr(x), x_kind, ld, x_gap, _ptr(weights_compressed), _ptr(codebook_fp16),
                                      float(scale), _ptr(output), M, N, K, sign_convention, _lib.LAYOUT_TILE,
                                      _lib.PATH_AUTO, flags, None if zero is None else _ptr(zero),
                                      0 if zero is None else zero.numel(), None if workspace is None else _ptr(workspace),
                                      0 if workspace is None else workspace.numel() * workspace.element_size(),
                                      _stream_ptr(x.device))
    _lib.check(rc, "decode_matmul_fused")
    return output


def workspace_bytes(M: int, N: int, K: int) -> int:
    """Bytes of scratch a call of shape (M, N, K) needs (``dmm_workspace_bytes``)."""
    return int(_lib.lib().dmm_workspace_bytes(M, N, K))


def decode_matmul_fused_tp(x, weights_compressed, codebook_fp16, scale, peer_out_ptrs, out_shape, *, x_kind=_lib.X_F32,
                           x_gap=0, sign_convention=_lib.SIGN_SLOW, pdl=False, zero=None, move_src=None, move_dst=None):
    """Row-parallel product whose epilogue adds the partial result into the same [M, N] fp32 buffer
    on every rank (``dmm_f16_fused_tp``).  ``peer_out_ptrs``: device addresses of that buffer on each
    rank (this rank's own included), e.g. from symmetric memory; ``out_shape`` = (M, N).
    ``move_src`` / ``move_dst``: local fp32 tensors, ``move_dst += move_src; move_src = 0`` first."""
    _check_input(x, "x", torch.float16 if x_kind == _lib.X_F16 else torch.float32)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    M, ld = x.shape
    N, K = weights_compressed.size(0), weights_compressed.size(1) * 8
    _req(tuple(out_shape) == (M, N), "out_shape must be (M, N)")
    _req(1 <= len(peer_out_ptrs) <= 8, "1 to 8 ranks")
    if zero is not None:
        _check_input(zero, "zero", torch.float32)
    n_move = 0
    if move_src is not None:
        _check_input(move_src, "move_src", torch.float32)
        _check_input(move_dst, "move_dst", torch.float32)
        _req(move_src.numel() == move_dst.numel(), "move_src and move_dst differ in size")
        n_move = move_src.numel()
    ptrs = (ctypes.c_void_p * len(peer_out_ptrs))(*[int(v) for v in peer_out_ptrs])
    with torch.cuda.device(x.device):
        rc = _lib.lib().dmm_f16_fused_tp(_ptr(x), x_kind, ld, x_gap, _ptr(weights_compressed), _ptr(codebook_fp16),
                                         float(scale), ptrs, len(peer_out_ptrs), M, N, K, sign_convention,
                                         _lib.FLAG_PDL if pdl else 0, None if zero is None else _ptr(zero),
                                         0 if zero is None else zero.numel(), None if n_move == 0 else _ptr(move_src),
                                         None if n_move == 0 else _ptr(move_dst), n_move, _stream_ptr(x.device))
    _lib.check(rc, "decode_matmul_fused_tp")


def tp_produce(x, weights_compressed, codebook_fp16, scale, peer_slot_ptrs, peer_flag_ptrs, rank, out_features, *,
               x_kind=_lib.X_F32, x_gap=0, sign_convention=_lib.SIGN_SLOW, pdl=False):
    """Row-parallel product of a tensor-parallel step in the slots form (``dmm_f16_tp_produce``): the partial
    product goes into this rank's slot on every rank (``peer_slot_ptrs`` / ``peer_flag_ptrs``: device addresses
    of every rank's slot array and flag words, this rank's own at index ``rank``)."""
    _check_input(x, "x", torch.float16 if x_kind == _lib.X_F16 else torch.float32)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    M, ld = x.shape
    N, K = weights_compressed.size(0), weights_compressed.size(1) * 8
    _req(N == out_features, "weights_compressed has the wrong number of rows")
    world = len(peer_slot_ptrs)
    slots = (ctypes.c_void_p * world)(*[int(v) for v in peer_slot_ptrs])
    flg = (ctypes.c_void_p * world)(*[int(v) for v in peer_flag_ptrs])
    with torch.cuda.device(x.device):
        rc = _lib.lib().dmm_f16_tp_produce(_ptr(x), x_kind, ld, x_gap, _ptr(weights_compressed), _ptr(codebook_fp16),
                                           float(scale), slots, flg, rank, world, M, N, K, sign_convention,
                                           _lib.FLAG_PDL if pdl else 0, _stream_ptr(x.device))
    _lib.check(rc, "tp_produce")


def tp_consume(h_in, h_out, slots, flags, world, weights_compressed, codebook_fp16, scale, output, *,
               sign_convention=_lib.SIGN_SLOW, pdl=False, zero=None):
    """Column-parallel product whose loaders read ``h_in`` + the partial products that all ranks pushed into this
    rank's ``slots`` (``dmm_f16_tp_consume``); the summed residual stream is written to ``h_out``."""
    _check_input(h_in, "h_in", torch.float32)
    _check_input(h_out, "h_out", torch.float32)
    _check_input(slots, "slots", torch.float32)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    _check_input(output, "output", torch.float32)
    _req(h_in.shape == h_out.shape and h_in.data_ptr() != h_out.data_ptr(), "h_out must be another buffer of h_in's shape")
    M, ld = h_in.shape
    N, K = weights_compressed.size(0), weights_compressed.size(1) * 8
    _req(tuple(output.shape) == (M, N), "output must have shape [M, N]")
    _req(slots.numel() == 2 * world * M * K, "slots must hold [2][world][M * K] floats")
    if zero is not None:
        _check_input(zero, "zero", torch.float32)
    with torch.cuda.device(h_in.device):
        rc = _lib.lib().dmm_f16_tp_consume(_ptr(h_in), _ptr(h_out), ld, _ptr(slots), _ptr(flags), world, M * K,
                                           _ptr(weights_compressed), _ptr(codebook_fp16), float(scale), _ptr(output), M, N, K,
                                           sign_convention, _lib.FLAG_PDL if pdl else 0, None if zero is None else _ptr(zero),
                                           0 if zero is None else zero.numel(), _stream_ptr(h_in.device))
    _lib.check(rc, "tp_consume")


def tp_finalize(h_in, h_out, slots, flags, world):
    """``h_out = h_in + the slots of the last epoch`` (``dmm_tp_finalize``)."""
    _check_input(h_in, "h_in", torch.float32)
    _check_input(h_out, "h_out", torch.float32)
    with torch.cuda.device(h_in.device):
        rc = _lib.lib().dmm_tp_finalize(_ptr(h_in), _ptr(h_out), _ptr(slots), _ptr(flags), world, h_in.numel(),
                                        _stream_ptr(h_in.device))
    _lib.check(rc, "tp_finalize")


def xrank_barrier(peer_flag_ptrs, rank, device):
    """Barrier kernel between the ranks of a tensor-parallel group (``dmm_xrank_barrier``)."""
    ptrs = (ctypes.c_void_p * len(peer_flag_ptrs))(*[int(v) for v in peer_flag_ptrs])
    with torch.cuda.device(device):
        rc = _lib.lib().dmm_xrank_barrier(ptrs, rank, len(peer_flag_ptrs), _stream_ptr(device))
    _lib.check(rc, "xrank_barrier")


def xrank_allreduce_add(dst, peer_src_ptrs, peer_flag_ptrs, rank, *, zero=None):
    """``dst += sum over ranks of the buffers at peer_src_ptrs`` as one kernel that first waits for all
    ranks (``dmm_xrank_allreduce_add``); ``zero``: local fp32 tensor cleared as well."""
    _check_input(dst, "dst", torch.float32)
    if zero is not None:
        _check_input(zero, "zero", torch.float32)
        _req(zero.numel() == dst.numel(), "zero and dst differ in size")
    world = len(peer_src_ptrs)
    src = (ctypes.c_void_p * world)(*[int(v) for v in peer_src_ptrs])
    flg = (ctypes.c_void_p * world)(*[int(v) for v in peer_flag_ptrs])
    with torch.cuda.device(dst.device):
        rc = _lib.lib().dmm_xrank_allreduce_add(_ptr(dst), src, None if zero is None else _ptr(zero), dst.numel(), flg,
                                                rank, world, _stream_ptr(dst.device))
    _lib.check(rc, "xrank_allreduce_add")


def decode_matmul_chain(ops, codebook_fp16, *, sign_convention=_lib.SIGN_SLOW, pdl=False):
    """Up to ``CHAIN_MAX_OPS`` dependent products in one launch (``dmm_f16_chain``).

    ``ops`` is a list of dicts with the keyword arguments of :func:`decode_matmul_fused` for one
    product each: ``x``, ``weights_compressed``, ``scale``, ``output`` and optionally ``x_kind``,
    ``x_gap``, ``zero``.  Every product is ADDED to its ``output`` with atomic adds, and op k + 1
    may read what op k wrote.  Batch at most 8; needs the whole GPU (cooperative launch)."""
    _req(2 <= len(ops) <= _lib.CHAIN_MAX_OPS, f"a chain has 2 to {_lib.CHAIN_MAX_OPS} ops")
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    arr = (_lib.ChainOp * len(ops))()
    M = ops[0]["x"].shape[0]
    for i, op in enumerate(ops):
        x, w, out = op["x"], op["weights_compressed"], op["output"]
        x_kind = op.get("x_kind", _lib.X_F32)
        _check_input(x, "x", torch.float16 if x_kind == _lib.X_F16 else torch.float32)
        _check_input(w, "weights_compressed", torch.int16)
        _check_input(out, "output", torch.float32)
        N, K = w.size(0), w.size(1) * 8
        _req(x.dim() == 2 and x.shape[0] == M and x.shape[1] >= K, "x must be [M, >= K]")
        _req(tuple(out.shape) == (M, N), "output must have shape [M, N]")
        zero = op.get("zero")
        if zero is not None:
            _check_input(zero, "zero", torch.float32)
        arr[i] = _lib.ChainOp(x.data_ptr(), x_kind, x.shape[1], op.get("x_gap", 0), w.data_ptr(), float(op["scale"]),
                              out.data_ptr(), N, K, None if zero is None else zero.data_ptr(),
                              0 if zero is None else zero.numel())
    dev = ops[0]["x"].device
    with torch.cuda.device(dev):
        rc = _lib.lib().dmm_f16_chain(ctypes.byref(arr), len(ops), _ptr(codebook_fp16), M, sign_convention,
                                      _lib.FLAG_PDL if pdl else 0, _stream_ptr(dev))
    _lib.check(rc, "decode_matmul_chain")


def decode_matmul_fp16_noalloc(x, weights_compressed, codebook_fp16, scale, output, *,
                               sign_convention=_lib.SIGN_SLOW, accumulate=False, pdl=False):
    """``decode_matmul_fp16`` for programs that cannot let the library allocate device memory
    (a server whose pool allocator already owns all of HBM, a latency-critical loop that must
    not take the allocator lock or the device synchronisation that cudaMalloc implies).  The caller supplies ``output``; the kernel's
    scratch is a fixed array inside the library, so nothing is allocated here or below.
    Batch at most 8, N at most 262144.  Calls on one device share that array: do not let two
    of them overlap on the GPU.  The first call on a device looks up the array's address and should come before any
    stream capture."""
    _check_input(x, "x", torch.float16)
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _check_input(codebook_fp16, "codebook_fp16", torch.float16)
    _check_input(output, "output", torch.float32)
    _req(x.dim() == 2 and weights_compressed.dim() == 2, "x and weights_compressed must be 2-D")
    _req(tuple(codebook_fp16.shape) == (256, 8), "codebook_fp16 must have shape [256, 8]")
    _req(x.size(-1) == weights_compressed.size(-1) << 3, "x.size(-1) must equal 8 * weights_compressed.size(-1)")
    M, K = x.shape
    N = weights_compressed.size(0)
    _req(tuple(output.shape) == (M, N), "output must have shape [M, N]")
    flags = (_lib.FLAG_ACCUMULATE if accumulate else 0) | (_lib.FLAG_PDL if pdl else 0)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dmm_f16_noalloc(_ptr(x), _ptr(weights_compressed), _ptr(codebook_fp16), float(scale),
                                        _ptr(output), M, N, K, sign_convention, flags, _stream_ptr(x.device))
    _lib.check(rc, "decode_matmul_fp16_noalloc")
    return output


def decode_weights(weights_compressed, codebook, *, sign_convention=_lib.SIGN_SLOW, layout=_lib.LAYOUT_TILE):
    """Decoded weights in logical order: int8 [N, K] (= 4 * weight) for an int64 codebook,
    fp16 [N, K] for an fp16 codebook."""
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    _req(weights_compressed.dim() == 2, "weights_compressed must be 2-D")
    is_f16 = codebook.dtype == torch.float16
    _check_input(codebook, "codebook", torch.float16 if is_f16 else torch.int64)
    _req(codebook.numel() == (2048 if is_f16 else 256), "codebook must have 256 entries")
    N, K8 = weights_compressed.shape
    with torch.cuda.device(weights_compressed.device):
        out = torch.empty((N, K8 * 8), dtype=torch.float16 if is_f16 else torch.int8,
                          device=weights_compressed.device)
        rc = _lib.lib().dmm_decode(_ptr(weights_compressed), _ptr(codebook), int(is_f16), _ptr(out), N, K8 * 8,
                                   sign_convention, layout, _stream_ptr(out.device))
    _lib.check(rc, "decode_weights")
    return out


def status(device=None) -> int:
    """Reads and clears the device status word (synchronises): 0 when every kernel since the
    last call finished its bounded waits and accepted its codebook."""
    v = ctypes.c_uint(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(_lib.lib().dmm_status(ctypes.byref(v)), "dmm_status")
    return v.value


def hint_next_weights(weights_compressed) -> None:
    """Tells the library which weight matrix the product AFTER the next one will stream (``dmm_hint_next_weights``):
    the next product's kernel then prefetches that matrix's first codes into L2.  ``None`` clears the hint."""
    if weights_compressed is None:
        _lib.check(_lib.lib().dmm_hint_next_weights(None, 0, 0), "dmm_hint_next_weights")
        return
    _check_input(weights_compressed, "weights_compressed", torch.int16)
    n, k8 = weights_compressed.shape
    _lib.check(_lib.lib().dmm_hint_next_weights(_ptr(weights_compressed), n, k8 * 8), "dmm_hint_next_weights")


def set_wait_limit_ms(ms: int) -> None:
    """Limit of the cross-rank waits (``dmm_set_wait_limit_ms``); 0 restores the default."""
    _lib.check(_lib.lib().dmm_set_wait_limit_ms(int(ms)), "dmm_set_wait_limit_ms")


def launch_count() -> int:
    return int(_lib.lib().dmm_launch_count())
