"""Row-sharded layer on the GPU kernels with two ranks.  Both ranks share cuda:0 and talk through gloo
(host-mediated collectives; no kernel of one rank waits on a kernel of the other), which exercises the
real sharding code -- row0 regeneration, token-sliced dense products, all four exchanges -- on one GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import randumb_b200 as rb
        from randumb_b200 import kernels as K
        from oracle import oracle as O
        torch.cuda.set_device(0)
        T, Kin, N, R, seed = 1000, 264, 528, 72, 7
        g = torch.Generator().manual_seed(5)
        x = torch.randn(T, Kin, generator=g).bfloat16().cuda()
        C = (torch.randn(R, Kin, generator=g) * 0.05).bfloat16().cuda()
        dy = torch.randn(T, N, generator=g).bfloat16().cuda()
        plan = rb.parallel.ShardedLayerPlan(T, N, world, rank)
        y_r = rb.parallel.sharded_forward(x, C, seed, plan)
        dx, dc = rb.parallel.sharded_backward(dy[:, plan.row_lo:plan.row_hi].contiguous(), x, C, seed, plan)
        # nothing replicated: token slice of dX, input-feature slice of dC
        lean_dx, lean_dc = rb.parallel.sharded_backward(dy[:, plan.row_lo:plan.row_hi].contiguous(), x, C, seed, plan,
                                                        replicate=False)
        # data parallel: this rank's half of the tokens, dC all-reduced after the backward ...
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        dp_dx, dp_dc = rb.parallel.data_parallel_backward(dy[lo:hi].contiguous(), x[lo:hi].contiguous(), C, seed)
        # ... or behind the dX product: the same products, launched one by one
        os.environ["RANDUMB_B200_DP_BACKWARD"] = "hidden"
        try:
            hid_dx, hid_dc = rb.parallel.data_parallel_backward(dy[lo:hi].contiguous(), x[lo:hi].contiguous(), C, seed)
        finally:
            del os.environ["RANDUMB_B200_DP_BACKWARD"]
        torch.cuda.synchronize()
        K.check_status()
        assert O.close(hid_dx, dp_dx, 1e-2) and O.close(hid_dc, dp_dc, 1e-2)
        torch.save({"y": y_r.cpu(), "dx": dx.cpu(), "dc": dc.cpu(), "rows": (plan.row_lo, plan.row_hi),
                    "dp_dx": dp_dx.cpu(), "dp_dc": dp_dc.cpu(), "tok": (lo, hi),
                    "lean_dx": lean_dx.cpu(), "lean_dc": lean_dc.cpu()}, os.path.join(tmp, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_single_gpu(tmp_path):
    from oracle import oracle as O
    from randumb_b200 import kernels as K
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    T, Kin, N, R, seed = 1000, 264, 528, 72, 7
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, Kin, generator=g).bfloat16()
    C = (torch.randn(R, Kin, generator=g) * 0.05).bfloat16()
    dy = torch.randn(T, N, generator=g).bfloat16()
    y_ref, dx_ref, dc_ref = O.linear_reference(x, C, seed, N, 0, dy, dtype=torch.float32)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(2)]
    assert parts[0]["rows"][0] == 0 and parts[0]["rows"][1] == parts[1]["rows"][0] and parts[1]["rows"][1] == N
    y = torch.cat([p["y"] for p in parts], dim=1)
    assert O.close(y, y_ref, 2e-2)
    for p in parts:                       # dX and dC are complete (and identical) on every rank
        assert O.close(p["dx"], dx_ref, 2e-2) and O.close(p["dc"], dc_ref, 2e-2)
    assert torch.equal(parts[0]["dx"], parts[1]["dx"]) and torch.equal(parts[0]["dc"], parts[1]["dc"])
    # unreplicated gradients: the ranks' pieces tile dX by tokens and dC by input features
    assert O.close(torch.cat([p["lean_dx"] for p in parts], dim=0), dx_ref, 2e-2)
    assert O.close(torch.cat([p["lean_dc"] for p in parts], dim=1), dc_ref, 2e-2)
    # data parallel: token halves of dX, the same summed dC on both ranks
    for p in parts:
        lo, hi = p["tok"]
        assert O.close(p["dp_dx"], dx_ref[lo:hi], 2e-2) and O.close(p["dp_dc"], dc_ref, 2e-2)
    assert torch.equal(parts[0]["dp_dc"], parts[1]["dp_dc"])
    # the sharded forward is bit-identical to the unsharded kernels on this GPU
    y_one = K.linear_fwd(x.cuda(), C.cuda(), seed, N).cpu()
    assert torch.equal(y, y_one)
