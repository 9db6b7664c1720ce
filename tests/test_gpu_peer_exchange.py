"""Row-sharded layer with the exchanges done by the library's own kernels over peer memory: one process per GPU (NCCL only
for set-up and for the comparison path), at least two GPUs -- skipped on a single-GPU machine.  Checked against the
unsharded kernels on one GPU and against the float32 oracle, with the scatter fused into the product kernel and with the
separate scatter kernel, two steps in a row (the exchange buffers and barrier epochs are reused)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

T, KIN, N, R, SEED = 1024, 264, 528, 256, 7


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, KIN, generator=g).bfloat16()
    C = (torch.randn(R, KIN, generator=g) * 0.05).bfloat16()
    dy = torch.randn(T, N, generator=g).bfloat16()
    return x, C, dy


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"           # plain peer loads/stores everywhere in this test
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import randumb_b200 as rb
        from randumb_b200 import kernels as K
        x, C, dy = _inputs()
        x, C, dy = x.to(dev), C.to(dev), dy.to(dev)
        plan = rb.parallel.ShardedLayerPlan(T, N, world, rank)
        ex = rb.parallel.PeerExchange.create(plan, R, dev)
        out = {"have_exchange": ex is not None, "rows": (plan.row_lo, plan.row_hi), "tok": (plan.tok_lo, plan.tok_hi),
               "cols": rb.parallel.shard_range(KIN, world, rank)}
        if ex is not None:
            out["how"] = ex.how
            dy_r = dy[:, plan.row_lo:plan.row_hi].contiguous()
            for step in range(2):
                timer = rb.parallel.PhaseTimer()
                y = rb.parallel.sharded_forward_peer(x, C, SEED, plan, ex, timer)
                dx, dc = rb.parallel.sharded_backward_peer(dy_r, x, C, SEED, plan, ex, timer, fused_scatter=(step == 0))
                torch.cuda.synchronize()
                K.check_status()
                out[f"y{step}"], out[f"dx{step}"], out[f"dc{step}"] = y.cpu(), dx.cpu(), dc.cpu()
                out[f"phases{step}"] = timer.durations()
            # two forwards in a row (inference): the second one's stores wait for every rank's first y product
            ya = rb.parallel.sharded_forward_peer(x, C, SEED, plan, ex)
            yb = rb.parallel.sharded_forward_peer(x, C, SEED, plan, ex)
            torch.cuda.synchronize()
            K.check_status()
            out["y_twice"] = bool(torch.equal(ya, y) and torch.equal(yb, y))
            # a backward that reads the noise rows the forward left in the exchange object: same bits as one that hashes them again
            dxk, dck = rb.parallel.sharded_backward_peer(dy_r, x, C, SEED, plan, ex, keep_noise=True)
            torch.cuda.synchronize()
            K.check_status()
            out["keep_noise"] = bool(torch.equal(dxk, dx) and torch.equal(dck, dc))
            # the NCCL path on the same inputs
            y_n = rb.parallel.sharded_forward(x, C, SEED, plan)
            dx_n, dc_n = rb.parallel.sharded_backward(dy_r, x, C, SEED, plan, replicate=False)
            torch.cuda.synchronize()
            out["y_nccl"], out["dx_nccl"], out["dc_nccl"] = y_n.cpu(), dx_n.cpu(), dc_n.cpu()
        # the all-reduce over peer memory: sum in rank order with float32 accumulation, the same bits on every rank, for a size
        # that divides into whole 16-byte chunks per rank and for one that needs padding; twice in a row
        for numel in (72 * KIN, 1001):
            par = rb.parallel.PeerAllReduce.create(numel, dev)
            out[f"allreduce_{numel}"] = par is not None
            if par is not None:
                for rep in range(2):
                    gen = torch.Generator().manual_seed(100 * rep + rank)
                    mine = torch.randn(numel, generator=gen).bfloat16().to(dev)
                    parts = [torch.empty_like(mine) for _ in range(world)]
                    dist.all_gather(parts, mine)
                    want = torch.stack(parts).float().sum(0)          # rank order is the stacking order
                    acc = torch.zeros(numel, dtype=torch.float32, device=dev)
                    for p_ in parts:
                        acc += p_.float()
                    got = par.all_reduce(mine.clone())
                    torch.cuda.synchronize()
                    K.check_status()
                    out[f"allreduce_{numel}"] = out[f"allreduce_{numel}"] and bool(torch.equal(got, acc.bfloat16())) and \
                        bool(torch.allclose(got.float(), want, rtol=2e-2, atol=1e-2))
        torch.save(out, os.path.join(tmp, f"r{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs one GPU per rank (at least two)")
def test_peer_exchange_matches_single_gpu_and_oracle(tmp_path):
    from oracle import oracle as O
    world = 2 if torch.cuda.device_count() < 4 else 4
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert all(p["have_exchange"] for p in parts), "ranks on separate GPUs of one node could not map each other's memory"
    x, C, dy = _inputs()
    y_ref, dx_ref, dc_ref = O.linear_reference(x, C, SEED, N, 0, dy, dtype=torch.float32)
    for step in range(2):
        y = torch.cat([p[f"y{step}"] for p in parts], dim=1)
        dx = torch.cat([p[f"dx{step}"] for p in parts], dim=0)
        dc = torch.cat([p[f"dc{step}"] for p in parts], dim=1)
        assert O.close(y, y_ref, 2e-2), f"step {step}: y rel {O.rel_fro(y, y_ref):.3e}"
        assert O.close(dx, dx_ref, 2e-2), f"step {step}: dx rel {O.rel_fro(dx, dx_ref):.3e}"
        assert O.close(dc, dc_ref, 2e-2), f"step {step}: dc rel {O.rel_fro(dc, dc_ref):.3e}"
    # the fused scatter and the separate scatter kernel move the same bf16 partial products: identical sums
    for p in parts:
        assert torch.equal(p["dx0"], p["dx1"]) and torch.equal(p["dc0"], p["dc1"]) and torch.equal(p["y0"], p["y1"])
        assert {"z product", "z exchange + noise fill", "y product", "g product", "g exchange", "dX product", "dC product"} <= set(p["phases0"])
    # same forward bits as the NCCL path (z is bit-identical whichever way it travels); gradients agree within tolerance
    # (NCCL sums the partial g in its own order, this path in rank order)
    for p in parts:
        assert p["y_twice"] and p["keep_noise"] and p[f"allreduce_{72 * KIN}"] and p["allreduce_1001"]
        assert torch.equal(p["y0"], p["y_nccl"])
        assert O.close(p["dx0"], p["dx_nccl"], 2e-2) and O.close(p["dc0"], p["dc_nccl"], 2e-2)
