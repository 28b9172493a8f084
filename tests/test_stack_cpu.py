"""Tensor-parallel sharding of the operator on CPU: two gloo ranks, the oracle as the compute.

Column-parallel (split N) shards are concatenated, row-parallel (split K) shards are summed
with an all-reduce; both must reproduce the unsharded product, and a shard must tile-pack
independently of the rest (what every rank of the GPU stack relies on)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    from decode_matmul_b200.layout import shard_cols, shard_rows, transpose_tile, untranspose_tile
    from oracle import dmm_oracle as o

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)  # same data on every rank
    M, N, K = 3, 64, 256
    cb16 = o.synthetic_codebook(42)
    x = rng.standard_normal((M, K)).astype(np.float16)
    codes = rng.integers(-32768, 32768, size=(N, K // 8)).astype(np.int16)
    full = o.decode_matmul_f16(x, codes, cb16, 1.0)

    # column-parallel: my rows, tile-packed on their own, then unpacked again as a kernel would see them
    mine = shard_rows(torch.from_numpy(codes), world, rank)
    mine = untranspose_tile(transpose_tile(mine)).numpy()
    part = torch.from_numpy(o.decode_matmul_f16(x, mine, cb16, 1.0))
    gathered = [torch.zeros_like(part) for _ in range(world)]
    dist.all_gather(gathered, part)
    col_ok = np.allclose(torch.cat(gathered, 1).numpy(), full, rtol=1e-6, atol=1e-5)

    # row-parallel: my slice of K, all-reduce of the partial products
    mine = shard_cols(torch.from_numpy(codes), world, rank)
    mine = untranspose_tile(transpose_tile(mine)).numpy()
    kl = K // world
    part = torch.from_numpy(o.decode_matmul_f16(np.ascontiguousarray(x[:, rank * kl:(rank + 1) * kl]), mine, cb16, 1.0))
    dist.all_reduce(part)
    row_ok = np.allclose(part.numpy(), full, rtol=1e-5, atol=1e-4)
    results[rank] = (col_ok, row_ok)
    dist.destroy_process_group()


def test_column_and_row_parallel_shards_reproduce_the_product():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results[r] == (True, True) for r in range(world)), dict(results)


def _numpy_step(stack, h, world, rank, allreduce):
    """The data flow of LinearStack.step with the oracle as the compute: column-parallel qkv / gate-up
    on this rank's shard, row-parallel o / down summed over the ranks by `allreduce`."""
    import decode_matmul_b200 as dmm
    from oracle import dmm_oracle as o

    cb16 = stack.layers[0]["qkv"].codebook.numpy()
    hid_loc, ffn_loc = stack.hidden // world, stack.ffn // world

    def lin(layer, x16):
        codes = dmm.untranspose_tile(layer.codes).numpy()
        return o.decode_matmul_f16(np.ascontiguousarray(x16), codes, cb16, layer.scale).astype(np.float64)

    for blk in stack.layers:
        a = lin(blk["qkv"], h.astype(np.float16))
        h = h + allreduce(lin(blk["o"], a[:, :hid_loc].astype(np.float16)))
        g = lin(blk["gate_up"], h.astype(np.float16))
        act = (g[:, :ffn_loc] / (1 + np.exp(-g[:, :ffn_loc])) * g[:, ffn_loc:]).astype(np.float16)
        h = h + allreduce(lin(blk["down"], act))
    return h


def _stack_worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    import decode_matmul_b200 as dmm
    from decode_matmul_b200.linear import LinearStack

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = dict(hidden=256, kv_heads=2, head_dim=32, ffn=512, layers=2)
    cb = dmm.synthetic_codebook(42)
    h0 = np.random.default_rng(3).standard_normal((2, 256))

    def allreduce(part):
        t = torch.from_numpy(part)
        dist.all_reduce(t)
        return t.numpy()

    sharded = LinearStack(cfg, cb, "cpu", world=world, rank=rank, logical_seed=11, scale=2.0 ** -8)
    whole = LinearStack(cfg, cb, "cpu", world=1, rank=0, logical_seed=11, scale=2.0 ** -8)
    got = _numpy_step(sharded, h0.copy(), world, rank, allreduce)
    want = _numpy_step(whole, h0.copy(), 1, 0, lambda p: p)
    results[rank] = float(np.abs(got - want).max())
    dist.destroy_process_group()


def test_logical_seed_stack_gives_the_same_step_on_one_and_two_ranks():
    """LinearStack(logical_seed=...) shards ONE set of logical matrices (q, k, v and gate, up part by
    part; o and down by reduction index): the step over two gloo ranks, with the oracle as the
    compute and an all-reduce after the row-parallel layers, equals the unsharded step."""
    world = 2
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_stack_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results[r] <= 1e-3 for r in range(world)), dict(results)
