"""The bounded cross-rank waits, made to run out on ONE GPU without faulting anything: a world of two
whose second rank does not exist (its flag words are ordinary local memory that nobody writes).
The kernel must give up after the configured limit, raise DMM_STATUS_WAIT_TIMEOUT, finish normally,
and leave the context usable for the next call.  Needs a B200."""
import time

import pytest
import torch

import decode_matmul_b200 as dmm
from decode_matmul_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture()
def short_limit():
    dmm.set_wait_limit_ms(5)
    yield
    dmm.set_wait_limit_ms(0)


def test_rank_barrier_gives_up_when_a_rank_never_arrives(short_limit):
    dev = torch.device("cuda")
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    ghost = torch.zeros(64, dtype=torch.int32, device=dev)  # the flag words of a rank that never runs
    assert dmm.status() == 0
    t0 = time.perf_counter()
    dmm.xrank_barrier([mine.data_ptr(), ghost.data_ptr()], 0, dev)
    st = dmm.status()  # synchronises
    assert time.perf_counter() - t0 < 1.0, "the wait did not end within its limit"
    assert st & _lib.STATUS_WAIT_TIMEOUT
    assert int(ghost[0]) != 0, "this rank did signal the other one before waiting"
    # the context is intact: a barrier of a world of one completes, and so does a product
    dmm.xrank_barrier([mine.data_ptr()], 0, dev)
    assert dmm.status() == 0
    x = torch.randn(1, 256, device=dev, dtype=torch.float16)
    w = torch.randint(-32768, 32768, (64, 32), dtype=torch.int16, device=dev)
    y = dmm.decode_matmul_fp16(x, w, dmm.synthetic_codebook(42, dev), 1.0)
    assert torch.isfinite(y).all() and dmm.status() == 0


def test_allreduce_kernel_gives_up_and_leaves_the_destination_alone(short_limit):
    dev = torch.device("cuda")
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    ghost = torch.zeros(64, dtype=torch.int32, device=dev)
    src0 = torch.full((1, 8192), 2.0, device=dev)
    src1 = torch.full((1, 8192), 3.0, device=dev)
    dst = torch.full((1, 8192), 1.0, device=dev)
    t0 = time.perf_counter()
    dmm.xrank_allreduce_add(dst, [src0.data_ptr(), src1.data_ptr()], [mine.data_ptr(), ghost.data_ptr()], 0)
    st = dmm.status()
    assert time.perf_counter() - t0 < 1.0
    assert st & _lib.STATUS_WAIT_TIMEOUT
    assert torch.equal(dst, torch.full_like(dst, 1.0)), "nothing may be summed when a rank is missing"
    # a world of one afterwards: dst += src0, and the partial buffer named by `zero` is cleared
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)
    dmm.xrank_allreduce_add(dst, [src0.data_ptr()], [flags1.data_ptr()], 0, zero=src1)
    assert dmm.status() == 0
    assert torch.equal(dst, torch.full_like(dst, 3.0)) and float(src1.abs().sum()) == 0.0


def test_slots_consumer_gives_up_when_a_rank_never_pushes(short_limit):
    """The consumer of the slots form (the default tensor-parallel step) waits in its activation loaders for
    every rank's flag.  A world of two whose second rank never raises its flag: the wait runs out, the status
    says so, the kernel still completes (with what the slots hold), and a world of one works afterwards."""
    dev = torch.device("cuda")
    M, K, N = 1, 1024, 512
    cb = dmm.synthetic_codebook(42, dev)
    w = torch.randint(-32768, 32768, (N, K // 8), dtype=torch.int16, device=dev)
    h_in = torch.randn(M, K, device=dev)
    want = dmm.decode_matmul_fused(h_in, w, cb, 1.0, torch.zeros(M, N, device=dev), x_kind=dmm.X_F32, accumulate=True, atomic=True)
    assert dmm.status() == 0

    def consume(world, ghost_flag):
        slots = torch.zeros(2 * world * M * K, device=dev)
        flags = torch.zeros(64, dtype=torch.int32, device=dev)
        flags[18] = 1      # epoch 1 is "in production" ...
        flags[0] = 1       # ... and this rank has pushed it
        if world > 1:
            flags[1] = ghost_flag
        h_out = torch.empty_like(h_in)
        out = torch.zeros(M, N, device=dev)
        from decode_matmul_b200 import ops
        ops.tp_consume(h_in, h_out, slots, flags, world, w, cb, 1.0, out)
        return h_out, out

    t0 = time.perf_counter()
    h_out, out = consume(2, 0)
    st = dmm.status()  # synchronises
    assert time.perf_counter() - t0 < 1.0, "the wait did not end within its limit"
    assert st & _lib.STATUS_WAIT_TIMEOUT
    assert torch.isfinite(out).all()
    # the context is intact: the same call with every flag up is the plain product of h_in (the slots are zero)
    for world in (2, 1):
        h_out, out = consume(world, 1)
        assert dmm.status() == 0
        assert torch.equal(h_out, h_in)
        assert float((out - want).abs().max()) <= 1e-3
