"""torch.library operator boundary.

Keeps the reference's operator names and schemas so existing call sites bind unchanged:

  rten::materialize_fwd / rten::materialize_bwd     src/rten_cpp/RandumbTensor.py:371-390
  rten::scale_bias_bwd                              src/rten_cpp/RandumbTensor.py:414-420
  rten::embed_fwd / rten::embed_bwd                 src/rten_cpp/RandumbTensor.py:1121-1134
  rten_cpp::sq5_gen_2d / rten_cpp::materialize_fwd  src/rten_cpp/csrc/rten.cpp:36-39, ops.py:8-13

and adds the operators of the matrix-coefficient layer ``W = S @ C`` that fill the slot the
reference left to ``fakeMM`` (RandumbTensor.py:771-791, 942-946):

  rten::rlinear_fwd(x, coef, seed, out_features, row0=0) -> y
  rten::rlinear_bwd(dy, x, coef, seed, row0, need_dx, need_dc) -> (dx, dc)
  rten::noise(rows, cols, seed, row0, dtype, device) -> S

Every operator is functional (fresh outputs, current stream), has a fake (meta) kernel so
FakeTensor / torch.compile tracing works, and -- like the reference (RandumbTensor.py:438-448) --
a CPU registration that raises ``NotImplementedError``: there is no CPU implementation.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch.library import custom_op

from . import kernels as K


def _cpu_raises(name):
    def _impl(*args, **kwargs):
        raise NotImplementedError(f"Unsupported CPU implementation of {name} called.")
    return _impl


# ------------------------------------------------------------------------------------------------
# matrix-coefficient layer
# ------------------------------------------------------------------------------------------------
@custom_op("rten::rlinear_fwd", mutates_args=(), device_types="cuda")
def rlinear_fwd(x: torch.Tensor, coef: torch.Tensor, seed: int, out_features: int, row0: int = 0) -> torch.Tensor:
    assert x.dim() == 2, "rlinear_fwd expects x flattened to [T, K]"
    return K.linear_fwd(x.contiguous(), coef.contiguous(), seed, out_features, row0)


@rlinear_fwd.register_fake
def _(x, coef, seed, out_features, row0=0):
    return x.new_empty((x.shape[0], out_features))


rlinear_fwd.register_kernel("cpu")(_cpu_raises("rlinear_fwd"))


@custom_op("rten::rlinear_bwd", mutates_args=(), device_types="cuda")
def rlinear_bwd(dy: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, seed: int, row0: int, need_dx: bool,
                need_dc: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    dx, dc = K.linear_bwd(dy.contiguous(), x.contiguous(), coef.contiguous(), seed, row0, need_dx, need_dc)
    # custom ops cannot return None: an empty tensor stands for "not requested"
    if dx is None:
        dx = x.new_empty((0,))
    if dc is None:
        dc = coef.new_empty((0,))
    return dx, dc


@rlinear_bwd.register_fake
def _(dy, x, coef, seed, row0, need_dx, need_dc):
    return (x.new_empty(x.shape) if need_dx else x.new_empty((0,)),
            coef.new_empty(coef.shape) if need_dc else coef.new_empty((0,)))


rlinear_bwd.register_kernel("cpu")(_cpu_raises("rlinear_bwd"))


def _rlinear_setup(ctx, inputs, output):
    x, coef, seed, out_features, row0 = inputs
    ctx.save_for_backward(x, coef)
    ctx.seed = seed
    ctx.row0 = row0


def _rlinear_backward(ctx, dy):
    x, coef = ctx.saved_tensors
    need_dx, need_dc = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    dx, dc = rlinear_bwd(dy, x, coef, ctx.seed, ctx.row0, need_dx, need_dc)
    return (dx if need_dx else None), (dc if need_dc else None), None, None, None


rlinear_fwd.register_autograd(_rlinear_backward, setup_context=_rlinear_setup)


def rlinear(x: torch.Tensor, coef: torch.Tensor, seed: int, out_features: int, row0: int = 0,
            bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ (S @ coef).T (+ bias) for x of shape [..., K]; differentiable in x and coef."""
    lead = x.shape[:-1]
    y = rlinear_fwd(x.reshape(-1, x.shape[-1]), coef, seed, out_features, row0)
    y = y.reshape(*lead, out_features)
    if bias is not None:
        y = y + bias
    return y


@custom_op("rten::noise", mutates_args=(), device_types="cuda")
def noise(rows: int, cols: int, seed: int, row0: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    return K.noise(rows, cols, seed, row0, 0, dtype, device)


@noise.register_fake
def _(rows, cols, seed, row0, dtype, device):
    return torch.empty((rows, cols), dtype=dtype, device=device)


# ------------------------------------------------------------------------------------------------
# reference operators (1-D coefficient vector)
# ------------------------------------------------------------------------------------------------
@custom_op("rten::materialize_fwd", mutates_args=(), device_types="cuda")
def materialize_fwd(coefs: torch.Tensor, size: List[int], strides: List[int], seed: int,
                    scale_bias: Optional[torch.Tensor], fused_bias: bool) -> torch.Tensor:
    assert not (fused_bias and scale_bias is None), "scale_bias not initialized but fused_bias is True"
    sb = scale_bias.detach().reshape(1).float().contiguous() if fused_bias else None
    return K.materialize_fwd(coefs.float().contiguous(), size, strides, seed, sb)


@materialize_fwd.register_fake
def _(coefs, size, strides, seed, scale_bias, fused_bias):
    return coefs.new_empty(size, dtype=torch.float32)


materialize_fwd.register_kernel("cpu")(_cpu_raises("materialize_fwd"))


@custom_op("rten::materialize_bwd", mutates_args=(), device_types="cuda")
def materialize_bwd(dout: torch.Tensor, dcoefs_size: int, seed: int) -> torch.Tensor:
    assert dout.is_contiguous(), "dout is not contiguous, backwards pass might give incorrect results."
    return K.materialize_bwd(dout, dcoefs_size, seed)


@materialize_bwd.register_fake
def _(dout, dcoefs_size, seed):
    return dout.new_empty((dcoefs_size,), dtype=torch.float32)


materialize_bwd.register_kernel("cpu")(_cpu_raises("materialize_bwd"))


@custom_op("rten::scale_bias_bwd", mutates_args=(), device_types="cuda")
def scale_bias_bwd(dout: torch.Tensor, seed: int) -> torch.Tensor:
    assert dout.is_contiguous(), "dout is not contiguous, backwards pass might give incorrect results."
    return K.scale_bias_bwd(dout, seed)


@scale_bias_bwd.register_fake
def _(dout, seed):
    return dout.new_empty((1,), dtype=torch.float32)


scale_bias_bwd.register_kernel("cpu")(_cpu_raises("scale_bias_bwd"))


def _mat_setup(ctx, inputs, output):
    coefs, size, strides, seed, scale_bias, fused_bias = inputs
    ctx.dcoefs_size = coefs.numel()
    ctx.seed = seed
    ctx.coef_dtype = coefs.dtype
    ctx.fused_bias = fused_bias
    ctx.bias_dtype = scale_bias.dtype if scale_bias is not None else None
    ctx.bias_shape = scale_bias.shape if scale_bias is not None else None
    ctx.view_size, ctx.view_strides = list(size), list(strides)


def _natural_order(grad: torch.Tensor, size: List[int], strides: List[int]) -> torch.Tensor:
    """Gradient of a strided view, laid out in the order of the virtual tensor's own elements.

    Element ``n`` of the virtual tensor always uses noise row ``n``; a view (a transpose, say) only changes which ``n`` sits
    at which output position: ``sq = sum_d index_d * stride_d`` (src/rten_cpp/RandumbTensor.py:264).  The backward kernels
    walk the noise rows in order (:304-359), so the incoming gradient is scattered back to ``flat[sq]`` first; positions
    the view does not reach keep a zero gradient."""
    expect, acc = [], 1
    for d in reversed(size):
        expect.append(acc)
        acc *= d
    if list(strides) == list(reversed(expect)):
        return grad.contiguous()
    extent = 1 + sum((d - 1) * st for d, st in zip(size, strides)) if all(d > 0 for d in size) else 0
    flat = grad.new_zeros((extent,))
    flat.as_strided(size, strides).copy_(grad)
    return flat


def _mat_backward(ctx, grad):
    grad = _natural_order(grad, ctx.view_size, ctx.view_strides)
    dcoefs = materialize_bwd(grad, ctx.dcoefs_size, ctx.seed).to(ctx.coef_dtype)
    dscale_bias = None
    if ctx.fused_bias:
        dscale_bias = scale_bias_bwd(grad, ctx.seed).to(ctx.bias_dtype).reshape(ctx.bias_shape)
    return dcoefs, None, None, None, dscale_bias, None


materialize_fwd.register_autograd(_mat_backward, setup_context=_mat_setup)


# ------------------------------------------------------------------------------------------------
# embedding rows of a virtual (vocab, rowsize) matrix (reference: RandumbTensor.py:1121-1160)
# ------------------------------------------------------------------------------------------------
@custom_op("rten::embed_fwd", mutates_args=(), device_types="cuda")
def embed_fwd(idx: torch.Tensor, coefs: torch.Tensor, rowsize: int, seed: int) -> torch.Tensor:
    return K.embed_fwd(idx, coefs.float().contiguous(), rowsize, seed)


@embed_fwd.register_fake
def _(idx, coefs, rowsize, seed):
    return coefs.new_empty((*idx.shape, rowsize), dtype=torch.float32)


embed_fwd.register_kernel("cpu")(_cpu_raises("embed_fwd"))


@custom_op("rten::embed_bwd", mutates_args=(), device_types="cuda")
def embed_bwd(idx: torch.Tensor, dout: torch.Tensor, dcoefs_size: int, rowsize: int, seed: int) -> torch.Tensor:
    return K.embed_bwd(idx, dout.contiguous(), dcoefs_size, rowsize, seed)


@embed_bwd.register_fake
def _(idx, dout, dcoefs_size, rowsize, seed):
    return dout.new_empty((dcoefs_size,), dtype=torch.float32)


embed_bwd.register_kernel("cpu")(_cpu_raises("embed_bwd"))


def _embed_setup(ctx, inputs, output):
    idx, coefs, rowsize, seed = inputs
    ctx.save_for_backward(idx)
    ctx.dcoefs_size = coefs.numel()
    ctx.rowsize = rowsize
    ctx.seed = seed
    ctx.coef_dtype = coefs.dtype


def _embed_backward(ctx, grad):
    (idx,) = ctx.saved_tensors
    dcoefs = embed_bwd(idx, grad.contiguous(), ctx.dcoefs_size, ctx.rowsize, ctx.seed).to(ctx.coef_dtype)
    return None, dcoefs, None, None


embed_fwd.register_autograd(_embed_backward, setup_context=_embed_setup)


def rt_mm(mat1: torch.Tensor, coefs: torch.Tensor, size: List[int], strides: List[int], seed: int,
          scale_bias: Optional[torch.Tensor] = None, fused_bias: bool = False) -> torch.Tensor:
    """``mat1[L, P] @ RT[P, Q]`` for a RandumbTensor in the 1-D coefficient form, same call as the reference's
    experimental ``rt_mm`` / ``rt_mm_grouped`` (src/rten_cpp/RandumbTensor.py:634-645, 758-769).

    Every element of RT costs ``M`` hashes, so regenerating RT tiles inside a product would repeat that work once
    per row block of ``mat1``; RT is materialised once (``rten::materialize_fwd``, differentiable in ``coefs`` and
    ``scale_bias``) and multiplied by the library's own product kernels (differentiable in ``mat1``).
    """
    P, Q = size
    assert mat1.dim() == 2 and mat1.size(1) == P, f"mm shape mismatch, received mat1 shape {tuple(mat1.size())} and rt shape {size}"
    rt = materialize_fwd(coefs, list(size), list(strides), seed, scale_bias, fused_bias)
    return _DenseMM.apply(mat1, rt.to(mat1.dtype))


class _DenseMM(torch.autograd.Function):
    """a[L, P] @ b[P, Q] on the library's product kernels (tensor cores for bf16, CUDA cores for float32)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return K.gemm_dense(a.contiguous(), b.contiguous(), True, False)

    @staticmethod
    def backward(ctx, grad):
        a, b = ctx.saved_tensors
        grad = grad.contiguous()
        da = K.gemm_dense(grad, b.contiguous(), True, True) if ctx.needs_input_grad[0] else None      # grad @ b^T
        db = K.gemm_dense(a.contiguous(), grad, False, False) if ctx.needs_input_grad[1] else None   # a^T @ grad
        return da, db


# C++-namespace twins of the reference (rten.cpp:36-39); registered from Python onto the same C ABI.
@custom_op("rten_cpp::sq5_gen_2d", mutates_args=())
def sq5_gen_2d(M: int, N: int, seed: int) -> torch.Tensor:
    return K.noise(M, N, seed, 0, 0, torch.float32, torch.device("cuda", torch.cuda.current_device()))


@sq5_gen_2d.register_fake
def _(M, N, seed):
    return torch.empty((M, N), dtype=torch.float32, device="cuda")


@custom_op("rten_cpp::materialize_fwd", mutates_args=(), device_types="cuda")
def materialize_fwd_cpp(coef: torch.Tensor, seed: int, P: int, Q: int, stride_P: int, stride_Q: int) -> torch.Tensor:
    assert coef.dim() == 1 and coef.is_contiguous()
    return K.materialize_fwd(coef.float(), [P, Q], [stride_P, stride_Q], seed)


@materialize_fwd_cpp.register_fake
def _(coef, seed, P, Q, stride_P, stride_Q):
    return coef.new_empty((P, Q), dtype=torch.float32)
