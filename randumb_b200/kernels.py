"""Tensor-level wrappers over the C ABI: torch supplies device memory and the current stream,
every number is produced by the library's own CUDA kernels.

All functions require CUDA tensors and raise ``RuntimeError`` otherwise -- there is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (BF16, F32, IMPL_AUTO, IMPL_SIMT, IMPL_UMMA, PATH_AUTO, PATH_FACTORED, PATH_WPATH)  # noqa: F401

_DT = {torch.float32: F32, torch.bfloat16: BF16}
_status_bufs: dict[int, torch.Tensor] = {}


def _dt(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise RuntimeError(f"randumb_b200 supports float32 and bfloat16, got {t}") from None


def _need_cuda(*ts: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("randumb_b200 kernels run on CUDA tensors only (no CPU implementation)")
        if dev is not None and t.device != dev:
            raise RuntimeError("all tensors must live on the same device")
        dev = t.device
    return dev


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _seed(seed: int) -> int:
    return int(seed) & 0xFFFFFFFF


def status_buffer(dev: torch.device) -> torch.Tensor:
    """Per-device int32[4] word the kernels write to when a bounded wait expires."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_bufs[idx] = buf
    return buf


def check_status(dev: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel launched so far gave up on a barrier wait."""
    devs = [dev.index if dev is not None and dev.index is not None else torch.cuda.current_device()] if dev is not None \
        else list(_status_bufs.keys())
    for idx in devs:
        buf = _status_bufs.get(idx)
        if buf is None:
            continue
        code = int(buf[0].item())
        if code != 0:
            buf.zero_()
            raise RuntimeError(f"randumb_b200 kernel gave up: {_lib.STATUS_NAMES.get(code, code)}")


def set_option(key: int, value: int) -> int:
    """Set the PROCESS DEFAULT of a tuning switch; returns the previous one.  Raises on an unknown key or a value out of
    range (nothing changes then).  Per-call values go through the ``options`` argument of the wrappers below."""
    prev = _lib.lib().rdb_set_option(key, value)
    _lib.check(min(prev, 0), f"rdb_set_option({key}, {value})")
    return prev


def _auto_impl(impl: int, *ts: Optional[torch.Tensor]) -> int:
    """IMPL_AUTO with an operand that does not start on a 16-byte boundary (a view at an odd storage offset) means the
    CUDA-core kernels: say so up front, so the workspace is sized for them."""
    if impl == IMPL_AUTO and any(t is not None and t.data_ptr() % 16 for t in ts):
        return IMPL_SIMT
    return impl


def _opts(options: Optional[_lib.CallOptions]):
    return ctypes.byref(options) if options is not None else None


# ------------------------------------------------------------------------------------------ noise
def noise_bits(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0, device="cuda") -> torch.Tensor:
    """uint32 hash words of S[row0:row0+rows, col0:col0+cols], returned as an int32 tensor (same bits)."""
    dev = torch.device(device)
    out = torch.empty((rows, cols), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_noise_bits(_ptr(out), rows, cols, cols, row0, col0, _seed(seed), _stream(out.device))
    _lib.check(rc, "rdb_noise_bits")
    return out


def noise(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0, dtype=torch.float32, device="cuda",
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """S[row0:row0+rows, col0:col0+cols] as float32 or bfloat16; ``out``: a contiguous [rows, cols] tensor to fill instead."""
    if out is not None:
        if tuple(out.shape) != (rows, cols) or not out.is_contiguous() or not out.is_cuda:
            raise RuntimeError(f"noise: out must be a contiguous CUDA tensor of shape [{rows}, {cols}]")
        dev, dtype = out.device, out.dtype
    else:
        dev = torch.device(device)
        out = torch.empty((rows, cols), dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_noise(_ptr(out), _dt(dtype), rows, cols, cols, row0, col0, _seed(seed), _stream(out.device))
    _lib.check(rc, "rdb_noise")
    return out


def noise_1d(n: int, seed: int, idx0: int = 0, device="cuda") -> torch.Tensor:
    dev = torch.device(device)
    out = torch.empty((n,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_noise_1d(_ptr(out), n, idx0, _seed(seed), _stream(out.device))
    _lib.check(rc, "rdb_noise_1d")
    return out


# ------------------------------------------------------------------------------------------ layer
def _workspace(nbytes: int, dev: torch.device) -> torch.Tensor:
    return torch.empty((max(int(nbytes), 256),), dtype=torch.uint8, device=dev)


def linear_fwd(x: torch.Tensor, coef: torch.Tensor, seed: int, out_features: int, row0: int = 0,
               path: int = PATH_AUTO, impl: int = IMPL_AUTO, options: Optional[_lib.CallOptions] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] @ (S[row0:row0+N] @ coef[R, K]).T  -- x, coef contiguous, same dtype."""
    dev = _need_cuda(x, coef)
    if x.dim() != 2 or coef.dim() != 2 or x.shape[1] != coef.shape[1]:
        raise RuntimeError(f"linear_fwd: x {tuple(x.shape)} and coef {tuple(coef.shape)} do not match [T,K] / [R,K]")
    if x.dtype != coef.dtype:
        raise RuntimeError("linear_fwd: x and coef must have the same dtype")
    assert x.is_contiguous() and coef.is_contiguous(), "linear_fwd expects contiguous x and coef"
    T, K = x.shape
    R = coef.shape[0]
    N = int(out_features)
    dt = _dt(x.dtype)
    L = _lib.lib()
    y = torch.empty((T, N), dtype=x.dtype, device=dev)
    impl = _auto_impl(impl, x, coef, y)
    with torch.cuda.device(dev):
        nbytes = L.rdb_linear_workspace_bytes_ex(0, T, K, N, R, dt, path, impl, _opts(options))
        ws = _workspace(nbytes, dev)
        rc = L.rdb_linear_fwd_ex(_ptr(y), _ptr(x), _ptr(coef), _ptr(ws), ws.numel(), T, K, N, R, row0, _seed(seed), dt, path,
                                 impl, _opts(options), _ptr(status_buffer(dev)), _stream(dev))
    _lib.check(rc, "rdb_linear_fwd")
    return y


def linear_bwd(dy: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, row0: int = 0, need_dx: bool = True,
               need_dc: bool = True, path: int = PATH_AUTO, impl: int = IMPL_AUTO, options: Optional[_lib.CallOptions] = None
               ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(dx[T,K], dc[R,K]) for dy[T,N]; either may be skipped."""
    dev = _need_cuda(dy, x, coef)
    if dy.dim() != 2 or x.dim() != 2 or coef.dim() != 2 or dy.shape[0] != x.shape[0] or x.shape[1] != coef.shape[1]:
        raise RuntimeError("linear_bwd: shapes must be dy[T,N], x[T,K], coef[R,K]")
    if not (dy.dtype == x.dtype == coef.dtype):
        raise RuntimeError("linear_bwd: dy, x and coef must have the same dtype")
    assert dy.is_contiguous() and x.is_contiguous() and coef.is_contiguous(), "linear_bwd expects contiguous inputs"
    T, N = dy.shape
    K = x.shape[1]
    R = coef.shape[0]
    dt = _dt(x.dtype)
    L = _lib.lib()
    dx = torch.empty((T, K), dtype=x.dtype, device=dev) if need_dx else None
    dc = torch.empty((R, K), dtype=x.dtype, device=dev) if need_dc else None
    impl = _auto_impl(impl, dy, x, coef, dx, dc)
    with torch.cuda.device(dev):
        nbytes = L.rdb_linear_workspace_bytes_ex(1, T, K, N, R, dt, path, impl, _opts(options))
        ws = _workspace(nbytes, dev)
        rc = L.rdb_linear_bwd_ex(_ptr(dx), _ptr(dc), _ptr(dy), _ptr(x), _ptr(coef), _ptr(ws), ws.numel(), T, K, N, R, row0,
                                 _seed(seed), dt, path, impl, _opts(options), _ptr(status_buffer(dev)), _stream(dev))
    _lib.check(rc, "rdb_linear_bwd")
    return dx, dc


def linear_weight(coef: torch.Tensor, seed: int, out_features: int, row0: int = 0) -> torch.Tensor:
    """Dense W[N, K] = S[row0:row0+N] @ coef (debugging / ops without a fused kernel)."""
    dev = _need_cuda(coef)
    assert coef.dim() == 2 and coef.is_contiguous()
    R, K = coef.shape
    w = torch.empty((int(out_features), K), dtype=coef.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_linear_weight(_ptr(w), _ptr(coef), K, int(out_features), R, row0, _seed(seed), _dt(coef.dtype),
                                          _stream(dev))
    _lib.check(rc, "rdb_linear_weight")
    return w


def gemv_fwd(x: torch.Tensor, coef: torch.Tensor, seed: int, out_features: int, row0: int = 0) -> torch.Tensor:
    dev = _need_cuda(x, coef)
    assert x.dtype == torch.float32 and coef.dtype == torch.float32 and x.is_contiguous() and coef.is_contiguous()
    R, K = coef.shape
    assert x.numel() == K
    y = torch.empty((int(out_features),), dtype=torch.float32, device=dev)
    ws = torch.empty((max(R, 1),), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_gemv_fwd(_ptr(y), _ptr(x), _ptr(coef), _ptr(ws), K, int(out_features), R, row0, _seed(seed),
                                     _stream(dev))
    _lib.check(rc, "rdb_gemv_fwd")
    return y


def gemv_bwd(dy: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, row0: int = 0, need_dx: bool = True,
             need_dc: bool = True):
    dev = _need_cuda(dy, x, coef)
    assert dy.dtype == torch.float32 and x.dtype == torch.float32 and coef.dtype == torch.float32
    assert dy.is_contiguous() and x.is_contiguous() and coef.is_contiguous()
    R, K = coef.shape
    N = dy.numel()
    dx = torch.empty((K,), dtype=torch.float32, device=dev) if need_dx else None
    dc = torch.empty((R, K), dtype=torch.float32, device=dev) if need_dc else None
    ws = _workspace(_lib.lib().rdb_gemv_bwd_workspace_bytes(K, N, R), dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_gemv_bwd(_ptr(dx), _ptr(dc), _ptr(dy), _ptr(x), _ptr(coef), _ptr(ws), K, N, R, row0,
                                     _seed(seed), _stream(dev))
    _lib.check(rc, "rdb_gemv_bwd")
    return dx, dc


# ------------------------------------------------------------------------------------------ building blocks
def gemm_noise(a: torch.Tensor, n: int, seed: int, transposed: bool = False, row0: int = 0, col0: int = 0,
               impl: int = IMPL_AUTO, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """D[M, n] = a[M, Kc] @ G.T with G generated (see rdb_gemm_noise)."""
    dev = _need_cuda(a)
    assert a.dim() == 2 and a.is_contiguous()
    M, Kc = a.shape
    out_dtype = out_dtype or a.dtype
    d = torch.empty((M, n), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_gemm_noise(_ptr(d), _ptr(a), M, n, Kc, Kc, n, _dt(a.dtype), _dt(out_dtype),
                                       1 if transposed else 0, row0, col0, _seed(seed), impl, _ptr(status_buffer(dev)),
                                       _stream(dev))
    _lib.check(rc, "rdb_gemm_noise")
    return d


def linear_stages_noise(T: int, K: int, N: int, R: int, dtype: torch.dtype, path: int = PATH_AUTO, impl: int = IMPL_AUTO,
                        options: Optional[_lib.CallOptions] = None, backward: bool = False) -> bool:
    """Whether linear_fwd (or, with ``backward``, linear_bwd) would write S once into the workspace for this problem (see
    rdb_linear_stages_noise)."""
    rc = _lib.lib().rdb_linear_stages_noise_ex(int(T), int(K), int(N), int(R), _dt(dtype), path, impl, _opts(options))
    _lib.check(min(rc, 0), "rdb_linear_stages_noise")
    return bool(rc & (2 if backward else 1))


def linear_plan(T: int, K: int, N: int, R: int, dtype: torch.dtype, path: int = PATH_AUTO, impl: int = IMPL_AUTO) -> Tuple[int, int]:
    """(association, kernels) the linear entry points would use: (PATH_FACTORED | PATH_WPATH, IMPL_SIMT | IMPL_UMMA)."""
    rc = _lib.lib().rdb_linear_path(int(T), int(K), int(N), int(R), _dt(dtype), path, impl)
    _lib.check(min(rc, 0), "rdb_linear_path")
    return rc & 0xFF, rc >> 8


def noise_product(a: torch.Tensor, n: int, seed: int, transposed: bool = False, row0: int = 0,
                  options: Optional[_lib.CallOptions] = None) -> torch.Tensor:
    """``a @ S[row0:row0+n].T`` (``transposed=False``, a is [M, R]) or ``a @ S[row0:row0+Kc]`` (``transposed=True``, a is
    [M, Kc], result [M, n]) with the same rule as the linear entry points: bf16 problems hash S once into a temporary and run
    the plain tensor-core product -- the transposed product (the backward's g = dY S) always, the other one for more than 1024
    rows of ``a``; everything else regenerates S inside the kernel."""
    M, Kc = a.shape
    rows, cols = (Kc, n) if transposed else (n, Kc)          # extent of the noise block S[rows, cols]
    ok8 = rows % 8 == 0 and cols % 8 == 0
    if a.dtype == torch.bfloat16 and ok8 and linear_stages_noise(M, 8, rows, cols, a.dtype, PATH_FACTORED, options=options,
                                                                       backward=transposed):
        S = noise(rows, cols, seed, row0, 0, torch.bfloat16, a.device)
        return gemm_dense(a, S, True, not transposed, options=options)
    return gemm_noise(a, n, seed, transposed, row0)


def _rows_ok(t: torch.Tensor) -> bool:
    return t.shape[0] <= 1 or t.shape[1] == 0 or (t.stride(1) == 1 and t.stride(0) >= t.shape[1]) or t.is_contiguous()


def _pitch(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 and t.shape[1] > 0 else t.shape[1]


def gemm_dense(a: torch.Tensor, b: torch.Tensor, a_kmajor: bool = True, b_kmajor: bool = True,
               out_dtype: Optional[torch.dtype] = None, impl: int = IMPL_AUTO, options: Optional[_lib.CallOptions] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """D[M, N] = op(a) @ op(b).T; a is [M,Kc] (a_kmajor) or [Kc,M]; b is [N,Kc] (b_kmajor) or [Kc,N].
    ``options``: per-call tuning switches (e.g. ``CallOptions(reserve_sms=32)`` for a launch that should leave SMs to a
    collective); ``out``: a contiguous [M, N] tensor to write into instead of a fresh one."""
    dev = _need_cuda(a, b)
    # rows may be further apart than their length (a column slice of a wider matrix): the row pitch is passed on
    assert a.dim() == 2 and b.dim() == 2 and _rows_ok(a) and _rows_ok(b), "gemm_dense: operands need unit stride along rows"
    M, Kc = (a.shape[0], a.shape[1]) if a_kmajor else (a.shape[1], a.shape[0])
    N, Kb = (b.shape[0], b.shape[1]) if b_kmajor else (b.shape[1], b.shape[0])
    if Kc != Kb:
        raise RuntimeError("gemm_dense: contraction extents differ")
    if out is not None:
        if tuple(out.shape) != (M, N) or not out.is_contiguous() or out.device != dev:
            raise RuntimeError(f"gemm_dense: out must be a contiguous [{M}, {N}] tensor on {dev}")
        d, out_dtype = out, out.dtype
    else:
        out_dtype = out_dtype or a.dtype
        d = torch.empty((M, N), dtype=out_dtype, device=dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        # few output tiles and a long contraction: scratch for split-K (float32 partial products, ordered sum)
        nbytes = L.rdb_gemm_dense_workspace_bytes(M, N, Kc) if impl != IMPL_SIMT and a.dtype == torch.bfloat16 else 0
        ws = _workspace(nbytes, dev) if nbytes else None
        rc = L.rdb_gemm_dense_ex(_ptr(d), _ptr(a), _ptr(b), _ptr(ws), nbytes, M, N, Kc, _pitch(a), _pitch(b), N, _dt(a.dtype),
                                 _dt(b.dtype), _dt(out_dtype), 1 if a_kmajor else 0, 1 if b_kmajor else 0, impl, _opts(options),
                                 _ptr(status_buffer(dev)), _stream(dev))
    _lib.check(rc, "rdb_gemm_dense_ex")
    return d


# ------------------------------------------------------------------------------------------ 1-D coefficient form
def materialize_fwd(coef: torch.Tensor, size, strides, seed: int, scale_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scale_bias``: None, or a one-element float32 device tensor; adds ``scale_bias * noise1d(sq(n))``."""
    dev = _need_cuda(coef)
    if scale_bias is not None:
        assert scale_bias.numel() == 1 and scale_bias.dtype == torch.float32 and scale_bias.device == dev
    assert coef.dim() == 1 and coef.dtype == torch.float32 and coef.is_contiguous()
    size = list(size)
    strides = list(strides)
    if len(size) == 1:
        P, Q, sP, sQ = 1, size[0], 0, strides[0]
    elif len(size) == 2:
        P, Q, sP, sQ = size[0], size[1], strides[0], strides[1]
    else:
        # more dimensions: only the contiguous layout, which is the flat 1-D case (element n uses noise row n)
        expect, acc = [], 1
        for d in reversed(size):
            expect.append(acc)
            acc *= d
        if strides != list(reversed(expect)):
            raise RuntimeError("materialize_fwd handles 1-D and 2-D outputs, and contiguous outputs of more dimensions")
        P, Q, sP, sQ = 1, acc, 0, 1
    out = torch.empty(size, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_materialize_fwd(_ptr(out), _ptr(coef), coef.numel(), P, Q, sP, sQ,
                                            _ptr(scale_bias) if scale_bias is not None else None, _seed(seed), _stream(dev))
    _lib.check(rc, "rdb_materialize_fwd")
    return out


def materialize_bwd(dout: torch.Tensor, dcoefs_size: int, seed: int) -> torch.Tensor:
    dev = _need_cuda(dout)
    assert dout.is_contiguous(), "dout is not contiguous, backwards pass might give incorrect results."
    dout = dout.reshape(-1).to(torch.float32)
    L = _lib.lib()
    dcoef = torch.empty((int(dcoefs_size),), dtype=torch.float32, device=dev)
    nbytes = L.rdb_materialize_bwd_workspace_bytes(dout.numel(), int(dcoefs_size))
    ws = torch.empty((max(nbytes // 4, 1),), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = L.rdb_materialize_bwd(_ptr(dcoef), _ptr(dout), _ptr(ws), dout.numel(), int(dcoefs_size), _seed(seed),
                                   _stream(dev))
    _lib.check(rc, "rdb_materialize_bwd")
    return dcoef


def scale_bias_bwd(dout: torch.Tensor, seed: int) -> torch.Tensor:
    """``sum_n dout[n] * noise1d(n)`` over the flattened contiguous gradient; one-element float32 tensor."""
    dev = _need_cuda(dout)
    assert dout.is_contiguous(), "dout is not contiguous, backwards pass might give incorrect results."
    dout = dout.reshape(-1).to(torch.float32)
    L = _lib.lib()
    dbias = torch.empty((1,), dtype=torch.float32, device=dev)
    ws = torch.empty((max(L.rdb_scale_bias_bwd_workspace_bytes(dout.numel()) // 4, 1),), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = L.rdb_scale_bias_bwd(_ptr(dbias), _ptr(dout), _ptr(ws), dout.numel(), _seed(seed), _stream(dev))
    _lib.check(rc, "rdb_scale_bias_bwd")
    return dbias


# ------------------------------------------------------------------------------------------ embedding rows
def embed_fwd(idx: torch.Tensor, coef: torch.Tensor, rowsize: int, seed: int) -> torch.Tensor:
    """Rows ``idx`` of the virtual (vocab, rowsize) matrix: float32 ``[*idx.shape, rowsize]``."""
    dev = _need_cuda(coef)
    assert coef.dim() == 1 and coef.dtype == torch.float32 and coef.is_contiguous()
    assert idx.device == dev and not idx.is_floating_point(), "idx must be an integer tensor on the device of coef"
    flat = idx.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((flat.numel(), int(rowsize)), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_embed_fwd(_ptr(out), _ptr(flat), _ptr(coef), flat.numel(), int(rowsize), coef.numel(),
                                      int(rowsize), _seed(seed), _stream(dev))
    _lib.check(rc, "rdb_embed_fwd")
    return out.reshape(*idx.shape, int(rowsize))


def embed_bwd(idx: torch.Tensor, dout: torch.Tensor, dcoefs_size: int, rowsize: int, seed: int) -> torch.Tensor:
    dev = _need_cuda(dout)
    assert idx.device == dev and not idx.is_floating_point()
    flat = idx.reshape(-1).to(torch.int64).contiguous()
    dout = dout.reshape(-1).to(torch.float32).contiguous()
    assert dout.numel() == flat.numel() * int(rowsize), "dout must hold one row of rowsize values per index"
    L = _lib.lib()
    dcoef = torch.empty((int(dcoefs_size),), dtype=torch.float32, device=dev)
    nbytes = L.rdb_materialize_bwd_workspace_bytes(dout.numel(), int(dcoefs_size))
    ws = torch.empty((max(nbytes // 4, 1),), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = L.rdb_embed_bwd(_ptr(dcoef), _ptr(dout), _ptr(flat), _ptr(ws), flat.numel(), int(rowsize), int(dcoefs_size),
                             _seed(seed), _stream(dev))
    _lib.check(rc, "rdb_embed_bwd")
    return dcoef


# ------------------------------------------------------------------------------------------ exchange over peer memory
def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr


def peer_barrier(flag_ptrs, rank: int, world: int, epoch: int, dev: torch.device) -> None:
    """Enqueue the barrier kernel of this rank (see rdb_peer_barrier); ``flag_ptrs``: a ctypes array from ``_ptr_array``."""
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_peer_barrier(flag_ptrs, rank, world, epoch, _ptr(status_buffer(dev)), _stream(dev))
    _lib.check(rc, "rdb_peer_barrier")


def peer_copy(dst_ptrs, ndst: int, dst_offset: int, src: torch.Tensor, max_blocks: int = 0) -> None:
    dev = _need_cuda(src)
    assert src.is_contiguous()
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_peer_copy(dst_ptrs, ndst, dst_offset, _ptr(src), src.numel() * src.element_size(), max_blocks, _stream(dev))
    _lib.check(rc, "rdb_peer_copy")


def peer_scatter(dst_ptrs, ndst: int, dst_offset: int, src: torch.Tensor, max_blocks: int = 0) -> None:
    """Row block j of the contiguous ``src`` (``src.shape[0] / ndst`` rows each) -> destination j."""
    dev = _need_cuda(src)
    assert src.is_contiguous() and src.shape[0] % ndst == 0
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_peer_scatter(dst_ptrs, ndst, dst_offset, _ptr(src), src.numel() * src.element_size() // ndst, max_blocks,
                                         _stream(dev))
    _lib.check(rc, "rdb_peer_scatter")


def reduce_slots(out: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """``out = slots.sum(0)`` for bf16 ``slots[nslots, ...]``, float32 accumulation in slot order."""
    dev = _need_cuda(out, slots)
    assert out.dtype == torch.bfloat16 and slots.dtype == torch.bfloat16 and out.is_contiguous() and slots.is_contiguous()
    assert slots.shape[1:] == out.shape
    nb = out.numel() * 2
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_reduce_slots_bf16(_ptr(out), _ptr(slots), nb, slots.shape[0], nb, _stream(dev))
    _lib.check(rc, "rdb_reduce_slots_bf16")
    return out


def gemm_dense_scatter(dst_ptrs, ndst: int, dst_offset: int, rows_per_dst: int, a: torch.Tensor, b: torch.Tensor,
                       b_kmajor: bool = True, options: Optional[_lib.CallOptions] = None) -> bool:
    """``a @ op(b).T`` on the CTA-pair kernel with row block j of the result stored into destination j by the kernel's
    epilogue (see rdb_gemm_dense_scatter).  Returns False, having launched nothing, when the shape does not qualify."""
    dev = _need_cuda(a, b)
    assert a.dim() == 2 and b.dim() == 2 and _rows_ok(a) and _rows_ok(b) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    M, Kc = a.shape
    N = b.shape[0] if b_kmajor else b.shape[1]
    with torch.cuda.device(dev):
        rc = _lib.lib().rdb_gemm_dense_scatter(dst_ptrs, ndst, dst_offset, rows_per_dst, _ptr(a), _ptr(b), M, N, Kc, _pitch(a), _pitch(b),
                                               1 if b_kmajor else 0, _opts(options), _ptr(status_buffer(dev)), _stream(dev))
    if rc == -6:
        return False
    _lib.check(rc, "rdb_gemm_dense_scatter")
    return True
