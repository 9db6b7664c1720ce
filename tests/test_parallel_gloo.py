"""world_size-2 CPU (gloo) ranks: row sharding by row0, the activation all-gather with its backward, and
the flat dC all-reduce.  The rank-local product is the oracle here (no GPU), so what is tested is the
partitioning and collective plumbing of randumb_b200.parallel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from randumb_b200 import parallel


class _OracleLinear(torch.autograd.Function):
    """y = x @ (S[row0:row0+n] @ C).T with explicit S on the CPU (float64)."""

    @staticmethod
    def forward(ctx, x, coef, seed, n_local, row0):
        S = torch.from_numpy(O.noise_f32(n_local, coef.shape[0], seed, row0=row0)).to(x.dtype)
        ctx.save_for_backward(x, coef, S)
        return x @ (S @ coef).t()

    @staticmethod
    def backward(ctx, dy):
        x, coef, S = ctx.saved_tensors
        g = dy @ S
        return g @ coef, g.t() @ x, None, None, None


def _local_linear(x, coef, seed, n_local, row0):
    return _OracleLinear.apply(x, coef, seed, n_local, row0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_features, gather):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        T, K, R, seed = 6, 16, 4, 7
        x_full = torch.randn(T, K, dtype=torch.float64)
        dy_full = torch.randn(T, out_features, dtype=torch.float64)
        layer = parallel.RowShardedRandumbLinear(K, out_features, R, seed, gather_output=gather, dtype=torch.float64,
                                                 local_linear=_local_linear)
        # replicas start identical
        gathered = [torch.empty_like(layer.weight_coef.data) for _ in range(world)]
        dist.all_gather(gathered, layer.weight_coef.data)
        assert all(torch.equal(g, gathered[0]) for g in gathered)

        x = x_full.clone().requires_grad_(True)
        y = layer(x)
        lo, hi = layer.row_lo, layer.row_hi
        y_ref, dx_ref, dc_ref = O.linear_reference(x_full, layer.weight_coef.data, seed, out_features, dy=dy_full)
        if gather:
            assert y.shape == (T, out_features)
            torch.testing.assert_close(y, y_ref, rtol=1e-10, atol=1e-12)
            y.backward(dy_full)
        else:
            assert y.shape == (T, hi - lo)
            torch.testing.assert_close(y, y_ref[:, lo:hi], rtol=1e-10, atol=1e-12)
            y.backward(dy_full[:, lo:hi].contiguous())
        # each rank holds the contribution of its own rows; the sums over ranks are the full gradients
        nbytes = parallel.allreduce_coef_grads([layer.weight_coef], average=False)
        assert nbytes == layer.weight_coef.numel() * 8
        torch.testing.assert_close(layer.weight_coef.grad, dc_ref, rtol=1e-9, atol=1e-11)
        dx = x.grad.clone()
        dist.all_reduce(dx)
        torch.testing.assert_close(dx, dx_ref, rtol=1e-9, atol=1e-11)

        # data-parallel pattern: different tokens per rank, averaged dC
        p = torch.nn.Parameter(torch.zeros(3, 5, dtype=torch.float64))
        q = torch.nn.Parameter(torch.zeros(7, dtype=torch.float64))
        p.grad = torch.full((3, 5), float(rank + 1), dtype=torch.float64)
        q.grad = torch.full((7,), float(10 * (rank + 1)), dtype=torch.float64)
        parallel.allreduce_coef_grads([p, q], average=True)
        mean = sum(range(1, world + 1)) / world
        assert torch.allclose(p.grad, torch.full((3, 5), mean, dtype=torch.float64))
        assert torch.allclose(q.grad, torch.full((7,), 10 * mean, dtype=torch.float64))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("out_features,gather", [(40, False), (40, True), (44, True)])
def test_row_sharding_two_ranks(out_features, gather):
    mp.spawn(_worker, args=(2, _free_port(), out_features, gather), nprocs=2, join=True)


def test_all_gather_rows_backward_sums_over_ranks():
    mp.spawn(_rows_worker, args=(2, _free_port()), nprocs=2, join=True)


def _rows_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = [3, 2]
        x = torch.full((sizes[rank], 4), float(rank + 1), requires_grad=True)
        # the plan of the peer-memory layer: contiguous row and token ranges that cover everything once
        plan = parallel.ShardedLayerPlan(96, 44, world, rank)
        assert plan.row_ranges == parallel.all_shard_ranges(44, world) and plan.tok_sizes == [48, 48]
        assert (plan.row_lo, plan.row_hi) == plan.row_ranges[rank] and (plan.tok_lo, plan.tok_hi) == (48 * rank, 48 * rank + 48)
        # the peer-memory exchange exists only between GPUs on NCCL ranks: on a gloo group it declines (the caller
        # then uses the collective path) without touching CUDA
        assert parallel.PeerExchange.create(plan, 16, torch.device("cpu")) is None
        z = parallel.all_gather_rows(x, sizes)
        assert z.shape == (5, 4) and float(z[0, 0]) == 1.0 and float(z[4, 0]) == 2.0
        (z * (rank + 1)).sum().backward()          # d/dz = rank+1 on every rank -> summed = 3
        assert torch.allclose(x.grad, torch.full_like(x, 3.0))
    finally:
        dist.destroy_process_group()
