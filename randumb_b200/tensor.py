"""``RandumbTensor``: a storage-less tensor whose values are ``noise @ coef``.

Same surface as the reference class (src/rten_cpp/RandumbTensor.py:794-954) and its differentiable
constructor (:959-994):

* 1-D ``coef`` of length M  -- the reference's form: element n of the (strided) tensor is
  ``sum_m S[sq(n), m] * coef[m]``; materialised by ``rten::materialize_fwd``.
* 2-D ``coef`` of shape [R, K] -- the matrix-coefficient form ``W[N, K] = S[N, R] @ coef``.  Used as
  the weight of ``F.linear`` it never materialises: the call is routed to the fused
  ``rten::rlinear_fwd`` operator, whose backward returns the coefficient gradient directly.

View ops (``view, transpose, t, permute, _to_copy``) return a new RandumbTensor with updated
shape/stride metadata, ``aten.mm``/``aten.addmm`` with a matrix-form weight go to the fused kernels,
and any other op materialises the operand, runs, and drops the dense copy again
(:916-954 of the reference).
"""
from __future__ import annotations

from collections.abc import Iterable
from typing import Optional, Union

import torch
from torch.autograd import Function
from torch.utils._pytree import tree_map
from torch._subclasses.fake_tensor import FakeTensorMode
from torch._guards import detect_fake_mode

from . import kernels as K
from . import ops


class RandumbTensor(torch.Tensor):
    """Wrapper subclass holding ``_coef``, ``seed`` and shape/stride metadata only.

    Register ``_coef`` as the module parameter and the RandumbTensor itself as a buffer, and always
    build it through :func:`CreateRandumbTensor` so gradients reach ``_coef``.
    """

    @staticmethod
    def __new__(cls, data: torch.Tensor, seed: int, shape: Union[tuple, torch.Size], scale_bias: Optional[torch.Tensor] = None,
                fused_bias: bool = False, strides: Optional[tuple] = None, row0: int = 0):
        assert not data.requires_grad or not torch.is_grad_enabled()
        kwargs = {}
        if strides is not None:
            kwargs["strides"] = strides
        return torch.Tensor._make_wrapper_subclass(cls, torch.Size(shape), device=data.device, dtype=data.dtype,
                                                   requires_grad=False, **kwargs)

    def __init__(self, data: torch.Tensor, seed: int, shape: Union[tuple, torch.Size], scale_bias: Optional[torch.Tensor] = None,
                 fused_bias: bool = False, strides: Optional[tuple] = None, row0: int = 0):
        self.seed = int(seed)
        self.scale_bias = scale_bias
        self.fused_bias = fused_bias
        self.row0 = int(row0)
        self._coef = data
        size = self._coef.size()
        assert len(size) in (1, 2), f"Coefficient tensor must be 1D or 2D but received tensor of shape {tuple(size)}"
        self.is_matrix_form = len(size) == 2
        self.int_dim = size[0]
        self._tensor: Optional[torch.Tensor] = None
        if self.is_matrix_form:
            assert len(self.shape) == 2, "a 2-D coefficient describes a 2-D weight [out_features, in_features]"
            n_out, k_in = self._natural_shape()
            assert k_in == size[1], f"coef has {size[1]} columns but the weight has {k_in} input features"
            self.noise_matrix_shape = torch.Size((n_out, self.int_dim))
        else:
            self.noise_matrix_shape = torch.Size((self.shape.numel(), self.int_dim))

    # ---- matrix form helpers ---------------------------------------------------------------
    def _is_natural(self) -> bool:
        """[N, K] with unit stride along K (the layout of a Linear weight)."""
        return self.dim() == 2 and self.stride(1) == 1 and self.stride(0) == self.shape[1]

    def _is_transposed(self) -> bool:
        """[K, N] view of the natural weight (what ``weight.t()`` produces)."""
        return self.dim() == 2 and self.stride(0) == 1 and self.stride(1) == self.shape[0]

    def _natural_shape(self):
        if self._is_natural():
            return self.shape[0], self.shape[1]
        if self._is_transposed():
            return self.shape[1], self.shape[0]
        raise AssertionError(f"matrix-form RandumbTensor with unsupported strides {self.stride()} for shape {tuple(self.shape)}")

    def __repr__(self):
        with torch._C._DisableTorchDispatch():
            return (f"RandumbTensor(seed={self.seed}, int_dim={self.int_dim}, shape={self.shape}, stride={self.stride()}, "
                    f"noise_matrix_shape={self.noise_matrix_shape}, dtype={self.dtype}, device='{self.device}')")

    # ---- debugging helpers kept from the reference -----------------------------------------
    def get_materialized(self) -> torch.Tensor:
        self.materialize()
        ref = self._tensor
        self.dematerialize()
        return ref

    def get_noise_matrix(self) -> torch.Tensor:
        return K.noise(self.noise_matrix_shape[0], self.noise_matrix_shape[1], self.seed, self.row0, 0, torch.float32,
                       self.device)

    def print_memory(self):
        noise_mem = self.element_size() * self.noise_matrix_shape.numel() / 2**20
        coeff_mem = self._coef.element_size() * self._coef.numel() / 2**20
        out_mem = self.element_size() * self.shape.numel() / 2**20
        total_mem = noise_mem + coeff_mem + out_mem
        print(f"unmaterialized noise matrix: {noise_mem}MiB\ncoefficient matrix: {coeff_mem}MiB\noutput matrix: {out_mem}MiB")
        print(f"% 'saved' memory: {noise_mem / total_mem * 100}%")

    @torch.compiler.disable(recursive=False)
    def materialize(self):
        with torch.no_grad():
            if self.is_matrix_form:
                n_out, _ = self._natural_shape()
                w = K.linear_weight(self._coef.detach().contiguous(), self.seed, n_out, self.row0)
                self._tensor = w if self._is_natural() else w.t()
            else:
                self._tensor = ops.materialize_fwd(self._coef, list(self.size()), list(self.stride()), self.seed,
                                                   self.scale_bias, self.fused_bias).to(self.dtype)

    def dematerialize(self):
        self._tensor = None

    # ---- F.linear with a matrix-form weight goes straight to the fused operator -------------
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.nn.functional.linear:
            x = args[0]
            w = args[1] if len(args) > 1 else kwargs.get("weight")
            b = args[2] if len(args) > 2 else kwargs.get("bias")
            # The shortcut differentiates through w._coef itself, so it is only taken when that is the
            # tensor autograd should reach (a dtype-cast view holds a detached copy instead).
            if (isinstance(w, RandumbTensor) and w.is_matrix_form and w._is_natural() and not isinstance(x, RandumbTensor)
                    and (w._coef.requires_grad or not w.requires_grad)):
                coef = w._coef if w._coef.dtype == x.dtype else w._coef.to(x.dtype)
                y = ops.rlinear(x, coef, w.seed, w.shape[0], w.row0)
                if b is not None:
                    y = y + b
                return y
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    OVERRIDE_VIEW_OPS = [torch.ops.aten.view.default, torch.ops.aten.transpose.int, torch.ops.aten._to_copy.default,
                         torch.ops.aten.t.default, torch.ops.aten.permute.default]

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        materialized: list[RandumbTensor] = []

        def _materialize(e):
            if isinstance(e, RandumbTensor):
                e.materialize()
                materialized.append(e)
                return e._tensor
            return e

        if func in cls.OVERRIDE_VIEW_OPS:
            instance: RandumbTensor = args[0]
            with torch.no_grad():
                fake_mode = detect_fake_mode(args)
                if fake_mode is None:
                    fake_mode = FakeTensorMode()
                with fake_mode:
                    fake = torch.empty_strided(instance.shape, instance.stride(), dtype=instance.dtype)
                    fake = func(fake, *args[1:], **kwargs)
                coef = instance._coef
                if func is torch.ops.aten._to_copy.default and fake.dtype != coef.dtype:
                    coef = coef.detach().to(fake.dtype)
                rt = RandumbTensor(coef, instance.seed, fake.shape, instance.scale_bias, instance.fused_bias, fake.stride(),
                                   instance.row0)
                del fake
            return rt

        # x @ W^T and dY @ W with a matrix-form weight: fused kernels, W never written to memory
        if func in (torch.ops.aten.mm.default, torch.ops.aten.addmm.default):
            off = 1 if func is torch.ops.aten.addmm.default else 0
            a, w = args[off], args[off + 1]
            if isinstance(w, RandumbTensor) and w.is_matrix_form and not isinstance(a, RandumbTensor) and a.dim() == 2:
                out = None
                if w._is_transposed():        # [T,K] @ [K,N]
                    out = K.linear_fwd(a.contiguous(), w._coef.detach().contiguous(), w.seed, w.shape[1], w.row0)
                elif w._is_natural():         # [T,N] @ [N,K]  (the dX product of the backward pass)
                    out = K.linear_bwd(a.contiguous(), a.new_empty((a.shape[0], w.shape[1])), w._coef.detach().contiguous(),
                                       w.seed, w.row0, need_dx=True, need_dc=False)[0]
                if out is not None:
                    if off:
                        alpha, beta = kwargs.get("alpha", 1), kwargs.get("beta", 1)
                        out = out * alpha + _materialize(args[0]) * beta if (alpha != 1 or beta != 1) else out + _materialize(args[0])
                        for t in materialized:
                            t.dematerialize()
                    return out

        ret = func(*tree_map(_materialize, args), **tree_map(_materialize, kwargs))
        for t in materialized:
            t.dematerialize()
        return ret


class RandumbTensorConstructor(Function):
    """Differentiable ``coefs -> RandumbTensor`` edge (reference: RandumbTensor.py:959-990).

    backward receives the dense gradient of the virtual tensor and contracts it with the noise:
    1-D coef -> ``rten::materialize_bwd``; 2-D coef -> ``dC = S^T dW`` through the generated-operand
    product (only reached when the weight was used by something other than ``F.linear``, whose fused
    backward produces dC without ever forming dW).
    """

    @staticmethod
    def forward(ctx, coefs: torch.Tensor, seed: int, shape: Iterable, scale_bias: Optional[torch.Tensor], fused_bias: bool,
                row0: int = 0) -> RandumbTensor:
        if not isinstance(coefs, torch.Tensor):
            raise AssertionError(f"Expected coefs to be of type torch.Tensor, found {type(coefs)} instead.")
        assert coefs.dim() in (1, 2), f"Coefficient tensor must be 1D or 2D but received tensor of shape {coefs.size()}"
        out = RandumbTensor(coefs, seed, shape, scale_bias, fused_bias, None, row0)
        ctx.coef_shape = tuple(coefs.shape)
        ctx.seed = seed
        ctx.row0 = row0
        ctx.dtype = out.dtype
        assert not (fused_bias and coefs.dim() == 2), "the fused random bias belongs to the 1-D coefficient form"
        ctx.fused_bias = fused_bias and scale_bias is not None
        ctx.bias_dtype = scale_bias.dtype if scale_bias is not None else None
        ctx.bias_shape = scale_bias.shape if scale_bias is not None else None
        return out

    @staticmethod
    def backward(ctx, grad):
        dscale_bias = None
        if len(ctx.coef_shape) == 1:
            grad = grad.flatten().contiguous()
            dcoefs = ops.materialize_bwd(grad, ctx.coef_shape[0], ctx.seed).to(ctx.dtype)
            if ctx.fused_bias:
                dscale_bias = ops.scale_bias_bwd(grad, ctx.seed).to(ctx.bias_dtype).reshape(ctx.bias_shape)
        else:
            R, _ = ctx.coef_shape
            # dC^T[K, R] = dW^T[K, N] @ S[N, R]: contraction over noise rows, dW^T as the streamed operand
            dwt = grad.t().contiguous()
            dct = K.gemm_noise(dwt, R, ctx.seed, transposed=True, row0=ctx.row0, impl=K.IMPL_SIMT if dwt.dtype == torch.float32
                               else K.IMPL_AUTO)
            dcoefs = dct.t().contiguous().to(ctx.dtype)
        return dcoefs, None, None, dscale_bias, None, None


def CreateRandumbTensor(coefs: torch.Tensor, seed: int, shape: Iterable, scale_bias: Optional[torch.Tensor] = None,
                        fused_bias: bool = False, row0: int = 0) -> RandumbTensor:
    """``rt = CreateRandumbTensor(coefs, seed, shape)`` -- same call as the reference (:993-994)."""
    return RandumbTensorConstructor.apply(coefs, seed, shape, scale_bias, fused_bias, row0)
