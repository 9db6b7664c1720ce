"""Multi-GPU use of the layer: one process per GPU, torch.distributed (NCCL over NVLink) for the two
exchanges the path has.

* Row sharding of one large virtual layer: rank r owns output rows ``[r*N/G, (r+1)*N/G)`` and
  regenerates exactly those noise rows from ``(seed, row0)`` -- no weight bytes ever move.  The only
  traffic is activations: ``sharded_forward`` / ``sharded_backward`` split the row-independent products by
  tokens and exchange the small ``z`` (all-gather) and ``g`` (all-reduce), then ``dX`` (all-gather) and
  ``dC`` (all-reduce); ``RowShardedRandumbLinear`` is the simple module form (optionally all-gathers ``y``).
* Data parallel training: every rank holds all of ``C``; the coefficient gradients are summed with one
  flat all-reduce per step (``allreduce_coef_grads``), or per layer right after its backward, or behind its dX
  product (``data_parallel_backward``).  (The reference's only parallelism is DDP in its GPT app:
  modded-nanogpt/train_gpt2.py:261, 346, 441.)

The collectives are plain NCCL calls on separate buffers; none of the compute kernels reads a peer's
memory.  ``local_*`` callables are injectable so the partitioning and collective plumbing can be
exercised with CPU (gloo) ranks.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib

def _overlap_sms() -> int:
    """SMs left without a CTA of the persistent product kernels while a collective runs beside them; given to that one
    launch as a per-call option.  ``RANDUMB_B200_OVERLAP_SMS`` overrides the default and must lie in the library's range."""
    v = int(os.environ.get("RANDUMB_B200_OVERLAP_SMS", "32"))
    if not 0 <= v <= _lib.MAX_RESERVE_SMS:
        raise ValueError(f"RANDUMB_B200_OVERLAP_SMS={v} is outside 0..{_lib.MAX_RESERVE_SMS}")
    return v


OVERLAP_SMS = _overlap_sms()


# ------------------------------------------------------------------------------------------------
# partition arithmetic
# ------------------------------------------------------------------------------------------------
def shard_range(total: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """[lo, hi) of the ``rank``-th of ``world`` contiguous shards of ``total`` items.

    Shard sizes are multiples of ``multiple`` (the tensor-core kernels want rows in groups of 8) except
    possibly the last, and differ by at most one group.
    """
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    groups = (total + multiple - 1) // multiple
    base, extra = divmod(groups, world)
    lo_g = rank * base + min(rank, extra)
    hi_g = lo_g + base + (1 if rank < extra else 0)
    return min(lo_g * multiple, total), min(hi_g * multiple, total)


def all_shard_ranges(total: int, world: int, multiple: int = 8) -> List[Tuple[int, int]]:
    return [shard_range(total, world, r, multiple) for r in range(world)]


# ------------------------------------------------------------------------------------------------
# autograd-aware collectives
# ------------------------------------------------------------------------------------------------
def _gather_blocks(x: torch.Tensor, sizes: Sequence[int], dim: int, group) -> List[torch.Tensor]:
    """all_gather of blocks whose extent along ``dim`` differs per rank (padded to the largest)."""
    big = max(sizes)
    if x.shape[dim] != big:
        pad_shape = list(x.shape)
        pad_shape[dim] = big - x.shape[dim]
        x = torch.cat([x, x.new_zeros(pad_shape)], dim=dim)
    parts = [torch.empty_like(x) for _ in sizes]
    dist.all_gather(parts, x.contiguous(), group=group)
    return [p.narrow(dim, 0, n) for p, n in zip(parts, sizes)]


class _AllGatherCols(torch.autograd.Function):
    """Concatenate per-rank column blocks [T, n_r] into [T, sum n_r]; backward keeps this rank's block."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, sizes: Sequence[int], group):
        ctx.group, ctx.sizes = group, list(sizes)
        ctx.rank = dist.get_rank(group)
        return torch.cat(_gather_blocks(x, sizes, 1, group), dim=1)

    @staticmethod
    def backward(ctx, grad):
        lo = sum(ctx.sizes[:ctx.rank])
        return grad[:, lo:lo + ctx.sizes[ctx.rank]].contiguous(), None, None


class _AllGatherRows(torch.autograd.Function):
    """Concatenate per-rank row blocks [t_r, R] into [sum t_r, R]; backward sums the gradient over ranks
    (every rank consumed the full gathered tensor) and keeps this rank's rows."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, sizes: Sequence[int], group):
        ctx.group, ctx.sizes = group, list(sizes)
        ctx.rank = dist.get_rank(group)
        return torch.cat(_gather_blocks(x, sizes, 0, group), dim=0)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        lo = sum(ctx.sizes[:ctx.rank])
        return grad[lo:lo + ctx.sizes[ctx.rank]].contiguous(), None, None


def all_gather_cols(x: torch.Tensor, sizes: Sequence[int], group=None) -> torch.Tensor:
    return _AllGatherCols.apply(x, sizes, group)


def all_gather_rows(x: torch.Tensor, sizes: Sequence[int], group=None) -> torch.Tensor:
    return _AllGatherRows.apply(x, sizes, group)


# ------------------------------------------------------------------------------------------------
# row-sharded virtual layer
# ------------------------------------------------------------------------------------------------
def _default_local_linear(x, coef, seed, n_local, row0):
    from . import ops
    return ops.rlinear(x, coef, seed, n_local, row0)


class RowShardedRandumbLinear(torch.nn.Module):
    """Rank-local part of a virtual layer with ``out_features`` rows split over the process group.

    forward(x) with x replicated on every rank returns this rank's columns ``y[:, lo:hi]`` (the
    column-parallel convention) or, with ``gather_output=True``, the full ``y`` after an all-gather of
    the activations.  ``coef`` is replicated; its gradient is the sum over ranks of the local
    contributions (``allreduce_coef_grads``), as is the gradient of the replicated input.
    """

    def __init__(self, in_features: int, out_features: int, d_c: int, seed: int, group=None, gather_output: bool = False,
                 device=None, dtype=None, init_std: Optional[float] = None,
                 local_linear: Callable = _default_local_linear):
        super().__init__()
        from .layers import coef_std_for, kaiming_out_std
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features, self.out_features, self.d_c, self.seed = in_features, out_features, d_c, int(seed)
        self.ranges = all_shard_ranges(out_features, self.world)
        self.row_lo, self.row_hi = self.ranges[self.rank]
        self.gather_output = gather_output
        self.local_linear = local_linear
        self.weight_coef = torch.nn.Parameter(torch.empty((d_c, in_features), device=device, dtype=dtype))
        std = coef_std_for(init_std if init_std is not None else kaiming_out_std(in_features), d_c)
        gen = torch.Generator(device=self.weight_coef.device).manual_seed(self.seed & 0x7FFFFFFFFFFFFFFF)
        with torch.no_grad():
            self.weight_coef.normal_(0.0, std, generator=gen)  # same seed on every rank => identical replicas

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local_linear(x, self.weight_coef, self.seed, self.row_hi - self.row_lo, self.row_lo)
        if self.gather_output and self.world > 1:
            lead = y.shape[:-1]
            y2 = all_gather_cols(y.reshape(-1, y.shape[-1]), [hi - lo for lo, hi in self.ranges], self.group)
            y = y2.reshape(*lead, self.out_features)
        return y


# ------------------------------------------------------------------------------------------------
# row-sharded layer with the row-independent products split by tokens
# ------------------------------------------------------------------------------------------------
def _all_gather_rows_plain(x: torch.Tensor, sizes: Sequence[int], group) -> torch.Tensor:
    if len(sizes) == 1:
        return x
    if all(n == sizes[0] for n in sizes):
        out = x.new_empty((sum(sizes), x.shape[1]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out
    return torch.cat(_gather_blocks(x, sizes, 0, group), dim=0)


class ShardedLayerPlan:
    """Who computes what when output rows are split over ``world`` ranks.

    Rank r owns noise rows ``[row_lo, row_hi)`` (regenerated locally from ``row0 = row_lo``) and, for the
    products that do not depend on the row split (``z = x C^T``, ``dX = g C``, ``dC = g^T x``), the token
    slice ``[tok_lo, tok_hi)``; computing those on every rank would cost more than the sharded part.
    """

    def __init__(self, tokens: int, out_features: int, world: int, rank: int):
        self.world, self.rank = world, rank
        self.row_ranges = all_shard_ranges(out_features, world)
        self.tok_ranges = all_shard_ranges(tokens, world)
        self.row_lo, self.row_hi = self.row_ranges[rank]
        self.tok_lo, self.tok_hi = self.tok_ranges[rank]
        self.tok_sizes = [hi - lo for lo, hi in self.tok_ranges]


def sharded_forward(x: torch.Tensor, coef: torch.Tensor, seed: int, plan: ShardedLayerPlan, group=None) -> torch.Tensor:
    """y[:, row_lo:row_hi] for replicated x[T, K], coef[R, K]: token-sliced z, all-gather z (T x R, small),
    then the generated-operand product for this rank's rows.  bf16, tensor-core kernels."""
    from . import kernels as K
    z_loc = K.gemm_dense(x[plan.tok_lo:plan.tok_hi].contiguous(), coef)                      # [t_r, R]
    z = _all_gather_rows_plain(z_loc, plan.tok_sizes, group) if plan.world > 1 else z_loc
    return K.noise_product(z, plan.row_hi - plan.row_lo, seed, False, plan.row_lo)               # [T, n_r]


def sharded_backward(dy_local: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, plan: ShardedLayerPlan,
                     group=None, replicate: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gradients from this rank's slice dY[:, row_lo:row_hi].

    ``replicate=True``: (dX[T, K], dC[R, K]) complete on every rank.  The partial g = dY_r S_r is summed over ranks
    (T x R, small) with every rank keeping only its token slice (reduce-scatter), then dX and dC are computed for this
    rank's tokens and exchanged; the dX all-gather runs while the tensor cores compute dC.

    ``replicate=False``: every gradient element is computed on exactly one rank and stays there -- returns
    (dX[tok_lo:tok_hi, :], dC[:, k_lo:k_hi]) with ``k_lo, k_hi = shard_range(K, world, rank)``.  g is all-reduced
    (the only exchange: T x R); dC is split by input features, which needs the full g but no reduction.
    """
    from . import kernels as K
    R = coef.shape[0]
    g = K.noise_product(dy_local.contiguous(), R, seed, True, plan.row_lo)                       # partial [T, R]
    if not replicate:
        if plan.world > 1:
            dist.all_reduce(g, group=group)
        k_lo, k_hi = shard_range(x.shape[1], plan.world, plan.rank)
        dx_loc = K.gemm_dense(g[plan.tok_lo:plan.tok_hi].contiguous(), coef, True, False)     # [t_r, K]
        dc_cols = K.gemm_dense(g, x[:, k_lo:k_hi].contiguous(), False, False)                 # [R, k_r]
        return dx_loc, dc_cols
    # the tensor forms of reduce-scatter / all-gather need equal shards and NCCL
    equal = (all(n == plan.tok_sizes[0] for n in plan.tok_sizes) and plan.world > 1 and dist.get_backend(group) == "nccl")
    if plan.world > 1 and equal:
        g_loc = g.new_empty((plan.tok_sizes[0], R))
        dist.reduce_scatter_tensor(g_loc, g, group=group)
    else:
        if plan.world > 1:
            dist.all_reduce(g, group=group)
        g_loc = g[plan.tok_lo:plan.tok_hi].contiguous()
    x_loc = x[plan.tok_lo:plan.tok_hi].contiguous()
    dx_loc = K.gemm_dense(g_loc, coef, True, False)                                           # [t_r, K]
    if plan.world == 1:
        return dx_loc, K.gemm_dense(g_loc, x_loc, False, False)
    if equal:
        dx = dx_loc.new_empty((sum(plan.tok_sizes), dx_loc.shape[1]))
        work_dx = dist.all_gather_into_tensor(dx, dx_loc, group=group, async_op=True)
        dc = K.gemm_dense(g_loc, x_loc, False, False, options=_lib.CallOptions(reserve_sms=OVERLAP_SMS))   # partial [R, K]
        dist.all_reduce(dc, group=group)
        work_dx.wait()
    else:
        dc = K.gemm_dense(g_loc, x_loc, False, False)
        dist.all_reduce(dc, group=group)
        dx = _all_gather_rows_plain(dx_loc, plan.tok_sizes, group)
    return dx, dc


# ------------------------------------------------------------------------------------------------
# the same layer with the exchanges done by the library's own kernels over peer memory
# ------------------------------------------------------------------------------------------------
class PhaseTimer:
    """Device time of the phases of one step as the launching stream sees them: ``mark(name)`` records an event on the
    current stream after a phase; ``durations()`` (after a synchronise) gives name -> milliseconds since the previous mark."""

    def __init__(self):
        self.events: List[Tuple[str, torch.cuda.Event]] = []
        self.mark("start")

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.events.append((name, ev))

    def durations(self) -> dict:
        out: dict = {}
        for (_, a), (name, b) in zip(self.events, self.events[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


def _mark(timer: Optional[PhaseTimer], name: str) -> None:
    if timer is not None:
        timer.mark(name)


class PeerExchange:
    """Exchange buffer of a row-sharded layer, mapped into every rank of the node, plus this rank's scratch.

    Layout of the shared buffer (identical on every rank, byte offsets):
        [0, 4096)      barrier flags: one uint64 per peer, written only by that peer (epochs only grow)
        z_full         [T, R] bf16   z = x C^T, every rank stores its token slice into all ranks' copies
        g_parts        [G, t_r, R] bf16   slot s = rank s's partial g = dY_s S_s for MY token slice
        g_full         [T, R] bf16   the summed g, every rank stores its reduced token slice into all ranks' copies
    Local (not shared): S [n_local, R] bf16 (this rank's noise rows, refilled in every forward and backward) and
    g_loc [t_r, R].

    The buffer comes from ``torch.distributed._symmetric_memory`` (its NVLink multicast binding switched off: the kernels
    use plain stores to the peers' mappings) or, failing that, from CUDA IPC handles of an ordinary allocation.  Needs one
    GPU per rank, equal token shards in multiples of 32, at most 8 ranks; ``PeerExchange.create`` returns None otherwise and
    the NCCL path is used.
    """
    FLAG_BYTES = 4096

    def __init__(self, plan: "ShardedLayerPlan", R: int, buf: torch.Tensor, ptrs: Sequence[int], how: str, keep=None):
        from . import kernels as K
        self.plan, self.R, self.buf, self.how, self._keep = plan, R, buf, how, keep
        self.world, self.rank, self.dev = plan.world, plan.rank, buf.device
        T = sum(plan.tok_sizes)
        self.T, self.t_r = T, plan.tok_sizes[0]
        self.z_off = self.FLAG_BYTES
        self.parts_off = self.z_off + T * R * 2
        self.gfull_off = self.parts_off + T * R * 2
        self.ptrs = K._ptr_array(ptrs)

        def view(off, rows):
            return buf[off:off + rows * R * 2].view(torch.bfloat16).view(rows, R)
        self.z_full, self.g_full = view(self.z_off, T), view(self.gfull_off, T)
        self.g_parts = view(self.parts_off, T).view(self.world, self.t_r, R)
        n_local = plan.row_hi - plan.row_lo
        self.S = torch.empty((n_local, R), dtype=torch.bfloat16, device=self.dev)
        self.g_loc = torch.empty((self.t_r, R), dtype=torch.bfloat16, device=self.dev)
        self.side = torch.cuda.Stream(device=self.dev)
        self.epoch = 0
        self.forward_pending = False      # a forward whose y product no later barrier has been seen to follow
        self.noise_key = None             # (seed, row_lo, row_hi) of the noise rows self.S holds

    @staticmethod
    def total_bytes(T: int, R: int) -> int:
        return PeerExchange.FLAG_BYTES + 3 * T * R * 2

    @classmethod
    def create(cls, plan: "ShardedLayerPlan", R: int, device: torch.device, group=None) -> Optional["PeerExchange"]:
        sizes = plan.tok_sizes
        if (plan.world < 2 or plan.world > _lib.MAX_PEERS or not dist.is_initialized() or dist.get_backend(group) != "nccl"
                or any(n != sizes[0] for n in sizes) or sizes[0] % 32 or R % 8):
            return None
        # one GPU per rank: ranks that share a GPU must not wait for each other inside kernels
        seen = [None] * plan.world
        dist.all_gather_object(seen, str(torch.cuda.get_device_properties(device).uuid), group=group)
        if len(set(seen)) != plan.world:
            return None
        nbytes = cls.total_bytes(sum(sizes), R)
        ex = None
        try:
            ex = cls._from_symmetric_memory(plan, R, device, nbytes, group)
        except Exception as e_symm:          # not available in this build / on this box: try plain CUDA IPC
            try:
                ex = cls._from_ipc(plan, R, device, nbytes, group)
            except Exception as e_ipc:
                if os.environ.get("RANDUMB_B200_DEBUG"):
                    print(f"PeerExchange unavailable: symmetric memory: {e_symm!r}; IPC: {e_ipc!r}", flush=True)
                ex = None
        # every rank must take the same path
        ok = torch.tensor([1 if ex is not None else 0], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            return None
        torch.cuda.synchronize(device)
        dist.barrier(group=group)            # every rank's flags are zero before anybody signals
        return ex

    @classmethod
    def _from_symmetric_memory(cls, plan, R, device, nbytes, group):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        grp = group if group is not None else dist.group.WORLD
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        torch.cuda.synchronize(device)
        hdl = symm_mem.rendezvous(buf, grp)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        if len(ptrs) != plan.world or ptrs[plan.rank] != buf.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe this buffer")
        return cls(plan, R, buf, ptrs, "torch symmetric memory", keep=hdl)

    @classmethod
    def _from_ipc(cls, plan, R, device, nbytes, group):
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        handle = buf.untyped_storage()._share_cuda_()
        handles = [None] * plan.world
        dist.all_gather_object(handles, handle, group=group)
        ptrs, keep = [], []
        for r, h in enumerate(handles):
            if r == plan.rank:
                ptrs.append(buf.data_ptr())
                continue
            st = torch.UntypedStorage._new_shared_cuda(*h)
            keep.append(st)
            ptrs.append(st.data_ptr())
        return cls(plan, R, buf, ptrs, "CUDA IPC", keep=keep)

    def barrier(self) -> None:
        """Enqueue this rank's barrier kernel on the current stream (same sequence of calls on every rank)."""
        from . import kernels as K
        self.epoch += 1
        K.peer_barrier(self.ptrs, self.rank, self.world, self.epoch, self.dev)

    def slice_offset(self, base: int, row: int) -> int:
        return base + row * self.R * 2


class PeerAllReduce:
    """Sum of a bf16 tensor over the ranks of one node through peer memory, with this library's kernels: every rank stores
    chunk j of its tensor into rank j's slot array, after a barrier rank j adds the G contributions to its chunk in rank order
    (float32 accumulation: the result does not depend on arrival order and is the same on every rank), stores the sum into
    every rank's result buffer, and a second barrier publishes it.  For the 8 MB coefficient gradient of the headline layer
    on 8 GPUs this takes about half as long as the NCCL all-reduce it replaces.  Same requirements as ``PeerExchange`` (one
    GPU per rank, at most 8 ranks); ``create`` returns None otherwise.

    Buffer (identical on every rank): [0, 4096) barrier flags | parts [G, chunk] | full [G * chunk], bf16."""
    FLAG_BYTES = 4096

    def __init__(self, numel: int, rank: int, world: int, buf: torch.Tensor, ptrs: Sequence[int], how: str, keep=None):
        from . import kernels as K
        self.numel, self.rank, self.world, self.buf, self.how, self._keep = numel, rank, world, buf, how, keep
        self.dev = buf.device
        self.chunk = self.chunk_elems(numel, world)
        self.parts_off = self.FLAG_BYTES
        self.full_off = self.parts_off + world * self.chunk * 2
        self.ptrs = K._ptr_array(ptrs)
        self.parts = buf[self.parts_off:self.full_off].view(torch.bfloat16).view(world, self.chunk)
        self.full = buf[self.full_off:self.full_off + world * self.chunk * 2].view(torch.bfloat16)
        self.red = torch.empty(self.chunk, dtype=torch.bfloat16, device=self.dev)
        self.pad = torch.zeros(world * self.chunk, dtype=torch.bfloat16, device=self.dev) if world * self.chunk != numel else None
        self.epoch = 0

    @staticmethod
    def chunk_elems(numel: int, world: int) -> int:
        per = -(-numel // world)
        return -(-per // 8) * 8                      # whole 16-byte units

    @classmethod
    def total_bytes(cls, numel: int, world: int) -> int:
        return cls.FLAG_BYTES + 2 * world * cls.chunk_elems(numel, world) * 2

    @classmethod
    def create(cls, numel: int, device: torch.device, group=None) -> Optional["PeerAllReduce"]:
        if not dist.is_initialized() or dist.get_backend(group) != "nccl":
            return None
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world < 2 or world > _lib.MAX_PEERS or numel <= 0:
            return None
        mapped = _map_peer_buffer(cls.total_bytes(numel, world), device, world, rank, group)
        if mapped is None:
            return None
        buf, ptrs, how, keep = mapped
        return cls(numel, rank, world, buf, ptrs, how, keep)

    def _barrier(self) -> None:
        from . import kernels as K
        self.epoch += 1
        K.peer_barrier(self.ptrs, self.rank, self.world, self.epoch, self.dev)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In place: ``t`` (contiguous bf16, ``numel`` elements) becomes the sum over the ranks.  Same sequence of calls on
        every rank; everything is enqueued on the current stream."""
        from . import kernels as K
        assert t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() == self.numel and t.device == self.dev
        src = t.view(-1)
        if self.pad is not None:
            self.pad[:self.numel].copy_(src)
            src = self.pad
        G, c = self.world, self.chunk
        K.peer_scatter(self.ptrs, G, self.parts_off + self.rank * c * 2, src.view(G, c))     # my chunk j -> rank j, slot `rank`
        self._barrier()
        K.reduce_slots(self.red, self.parts)                                               # rank order, float32
        K.peer_copy(self.ptrs, G, self.full_off + self.rank * c * 2, self.red)
        self._barrier()
        t.view(-1).copy_(self.full[:self.numel])
        return t


def _map_peer_buffer(nbytes: int, device: torch.device, world: int, rank: int, group=None):
    """A zeroed buffer of ``nbytes`` on every rank, mapped into all of them: (buffer, peer pointers, how, keep-alive) or None
    when the ranks share a GPU or neither symmetric memory nor CUDA IPC is available (the same answer on every rank)."""
    seen = [None] * world
    dist.all_gather_object(seen, str(torch.cuda.get_device_properties(device).uuid), group=group)
    mapped = None
    if len(set(seen)) == world:
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            grp = group if group is not None else dist.group.WORLD
            buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            buf.zero_()
            torch.cuda.synchronize(device)
            hdl = symm_mem.rendezvous(buf, grp)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if len(ptrs) != world or ptrs[rank] != buf.data_ptr():
                raise RuntimeError("symmetric memory handle does not describe this buffer")
            mapped = (buf, ptrs, "torch symmetric memory", hdl)
        except Exception as e_symm:
            try:
                buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
                torch.cuda.synchronize(device)
                handles = [None] * world
                dist.all_gather_object(handles, buf.untyped_storage()._share_cuda_(), group=group)
                ptrs, keep = [], []
                for r, h in enumerate(handles):
                    if r == rank:
                        ptrs.append(buf.data_ptr())
                        continue
                    st = torch.UntypedStorage._new_shared_cuda(*h)
                    keep.append(st)
                    ptrs.append(st.data_ptr())
                mapped = (buf, ptrs, "CUDA IPC", keep)
            except Exception as e_ipc:
                if os.environ.get("RANDUMB_B200_DEBUG"):
                    print(f"peer buffer unavailable: symmetric memory: {e_symm!r}; IPC: {e_ipc!r}", flush=True)
                mapped = None
    ok = torch.tensor([1 if mapped is not None else 0], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        return None
    torch.cuda.synchronize(device)
    dist.barrier(group=group)            # every rank's flags are zero before anybody signals
    return mapped


def sharded_forward_peer(x: torch.Tensor, coef: torch.Tensor, seed: int, plan: ShardedLayerPlan, ex: PeerExchange,
                         timer: Optional[PhaseTimer] = None) -> torch.Tensor:
    """``sharded_forward`` with the z all-gather done by this library's kernels: the tensor cores compute the local token
    slice of z straight into this rank's copy of ``z_full``; the slice is then stored into every peer's copy, and while those
    stores and the barrier are in flight (NVLink-bound, a few SMs) this rank's noise rows are hashed on a side stream (integer
    ALU on all SMs).  After both, every rank holds all of z and computes its columns of y.  (The hash is not started beside
    the z product: its two thousand resident threads per SM starve the product's single MMA-issuing thread.)"""
    from . import kernels as K
    cur = torch.cuda.current_stream(ex.dev)
    z_loc = ex.z_full[plan.tok_lo:plan.tok_hi]
    K.gemm_dense(x[plan.tok_lo:plan.tok_hi], coef, out=z_loc)                                  # [t_r, R], in place in z_full
    _mark(timer, "z product")
    if ex.forward_pending:
        # two forwards in a row (no backward, whose barriers would order them): a faster rank must not store its next z slice
        # into this rank's z_full while the previous y product still reads it
        ex.barrier()
    ex.forward_pending = True
    ex.side.wait_stream(cur)
    with torch.cuda.stream(ex.side):
        K.noise(ex.S.shape[0], ex.R, seed, plan.row_lo, 0, out=ex.S)
    ex.noise_key = (int(seed), plan.row_lo, plan.row_hi)         # what ex.S holds once the side stream has been waited for
    K.peer_copy(_others(ex), ex.world - 1, ex.slice_offset(ex.z_off, plan.tok_lo), z_loc)
    ex.barrier()
    cur.wait_stream(ex.side)
    _mark(timer, "z exchange + noise fill")
    y = K.gemm_dense(ex.z_full, ex.S)                                                           # [T, n_r] = z S_r^T
    _mark(timer, "y product")
    return y


def _others(ex: PeerExchange):
    """Pointer list of the other ranks' buffers (this rank's own copy is written by the local kernel)."""
    from . import kernels as K
    if not hasattr(ex, "_others"):
        ex._others = K._ptr_array([ex.ptrs[r] for r in range(ex.world) if r != ex.rank])
    return ex._others


def sharded_backward_peer(dy_local: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, plan: ShardedLayerPlan,
                          ex: PeerExchange, timer: Optional[PhaseTimer] = None, fused_scatter: bool = True,
                          keep_noise: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``sharded_backward(replicate=False)`` -- (dX[tok_lo:tok_hi, :], dC[:, k_lo:k_hi]) -- with the sum of g over the ranks
    done by this library's kernels.  The partial g = dY_r S_r leaves the product kernel's epilogue tile by tile straight into
    the owner of each token slice (``rdb_gemm_dense_scatter``: the scatter half of a reduce-scatter fused into the product);
    after a barrier every rank sums the G contributions to its slice in rank order; the reduced slice is stored into every
    rank's ``g_full`` on a side stream while the tensor cores compute dX from it; dC (all tokens, this rank's input
    features) follows the second barrier.

    ``keep_noise`` (off by default): the exchange object's noise rows are the ones ``sharded_forward_peer`` hashed for the same
    seed and rows, so a training step that calls forward and then backward may read them again instead of hashing them a
    second time -- one hash per element and step instead of two, at the price of keeping S_r (``n_r x R`` bf16) alive between
    the two calls, which the stateless C entry points never do."""
    from . import kernels as K
    R, G = ex.R, ex.world
    cur = torch.cuda.current_stream(ex.dev)
    if not (keep_noise and ex.noise_key == (int(seed), plan.row_lo, plan.row_hi)):
        K.noise(ex.S.shape[0], R, seed, plan.row_lo, 0, out=ex.S)
        ex.noise_key = (int(seed), plan.row_lo, plan.row_hi)
    _mark(timer, "noise fill")
    slot = ex.parts_off + ex.rank * ex.t_r * R * 2            # my slot in every owner's g_parts
    fused_scatter = fused_scatter and os.environ.get("RANDUMB_B200_FUSED_SCATTER", "1") != "0"
    done = fused_scatter and K.gemm_dense_scatter(ex.ptrs, G, slot, ex.t_r, dy_local, ex.S, b_kmajor=False)
    if not done:
        g = K.gemm_dense(dy_local, ex.S, True, False)                                        # partial [T, R]
        K.peer_scatter(ex.ptrs, G, slot, g)
    _mark(timer, "g product")
    ex.barrier()
    ex.forward_pending = False                                  # every rank is past its y product
    K.reduce_slots(ex.g_loc, ex.g_parts)                                                      # [t_r, R], summed in rank order
    _mark(timer, "g exchange")
    ex.side.wait_stream(cur)
    with torch.cuda.stream(ex.side):
        K.peer_copy(ex.ptrs, G, ex.slice_offset(ex.gfull_off, plan.tok_lo), ex.g_loc, max_blocks=64)
        ex.barrier()
    # the copy's 64 small blocks need somewhere to run while the persistent product holds one CTA per SM: leave them 20 SMs
    # (64 CTA pairs are still resident, one per 512 x 256 tile of a 512-token slice with 16384 input features)
    dx_loc = K.gemm_dense(ex.g_loc, coef, True, False, options=_lib.CallOptions(reserve_sms=20))   # [t_r, K]
    _mark(timer, "dX product")
    cur.wait_stream(ex.side)
    _mark(timer, "g all-gather tail")
    k_lo, k_hi = shard_range(x.shape[1], plan.world, plan.rank)
    dc_cols = K.gemm_dense(ex.g_full, x[:, k_lo:k_hi], False, False)                          # [R, k_r]
    _mark(timer, "dC product")
    return dx_loc, dc_cols


# ------------------------------------------------------------------------------------------------
# data-parallel backward: the layer's backward, then the all-reduce of dC (or the all-reduce hidden behind the dX product)
# ------------------------------------------------------------------------------------------------
def data_parallel_backward(dy: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, row0: int = 0, group=None,
                           average: bool = False, peer: Optional["PeerAllReduce"] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dX[T, K], dC[R, K] summed over the ranks) for a replicated bf16 layer and this rank's tokens.

    Default: the library's own backward (``rdb_linear_bwd``: dX beside dC on disjoint CTA pairs where their tiles pack),
    then the all-reduce of dC in the open.  ``RANDUMB_B200_DP_BACKWARD=hidden`` selects the older schedule -- dC first, its
    all-reduce started asynchronously behind the dX product, which is given fewer SMs so that the collective can run -- which
    hides the reduction but pays for it with the SMs taken from dX and with dX and dC no longer running side by side:
    0.597 against 0.587 ms per step of the headline layer at 2 GPUs, 0.619 against 0.596 at 4.  ``peer``: a ``PeerAllReduce``
    for dC's size does the reduction with this library's kernels over peer memory instead of NCCL (default schedule only).
    The returned dC is safe to use on the current stream.
    """
    from . import kernels as K
    R = coef.shape[0]
    if os.environ.get("RANDUMB_B200_DP_BACKWARD", "plain") != "hidden":
        dx, dc = K.linear_bwd(dy, x, coef, seed, row0)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            if peer is not None:
                peer.all_reduce(dc)           # this library's kernels over peer memory, sum in rank order
            else:
                dist.all_reduce(dc, op=dist.ReduceOp.SUM, group=group)
            if average:
                dc /= dist.get_world_size(group)
        return dx, dc
    g = K.noise_product(dy, R, seed, True, row0)                                              # [T, R]
    dc = K.gemm_dense(g, x, False, False)                                                     # [R, K]
    work = None
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(dc, op=dist.ReduceOp.SUM, group=group, async_op=True)
    # the product kernels are persistent, one CTA per SM: leave a few SMs to the collective or it waits for them to retire
    # (an option of this one launch: no process state changes, other threads' launches are not affected)
    dx = K.gemm_dense(g, coef, True, False,
                      options=_lib.CallOptions(reserve_sms=OVERLAP_SMS) if work is not None else None)   # [T, K]
    if work is not None:
        work.wait()                       # makes the current stream wait for the reduction; the host does not block
        if average:
            dc /= dist.get_world_size(group)
    return dx, dc


# ------------------------------------------------------------------------------------------------
# gradient exchange
# ------------------------------------------------------------------------------------------------
def allreduce_coef_grads(params: Sequence[torch.nn.Parameter], group=None, average: bool = True,
                         comm_dtype: Optional[torch.dtype] = None) -> int:
    """One flat all-reduce over the gradients of ``params``; returns the bytes sent per rank.

    The coefficient matrices are small (d_c x in_features each), so all of them are packed into a
    single bucket: one launch, one NVLink/NVSwitch reduction.
    """
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    dt = comm_dtype or grads[0].dtype
    flat = torch.cat([g.reshape(-1).to(dt) for g in grads])
    if world > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n
    return flat.numel() * flat.element_size()
