"""Modules whose weights are RandumbTensors.

``RandumbLinear`` is the matrix-coefficient layer (coef ``[d_c, in_features]``); ``SillyLinear`` keeps
the reference constructor conventions (src/rten_cpp/SillyLayers.py:142-227): ``int_dim`` and ``seed``
are lists of two values or generators, parameters are ``weight_coef`` / ``bias_coef``, the virtual
tensors are registered as buffers ``weight`` / ``bias``.  ``stepgen`` / ``listgen`` are the reference's
seed and int_dim sequences (SillyLayers.py:25-34).
"""
from __future__ import annotations

import math
from types import GeneratorType
from typing import Generator, Optional, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .tensor import CreateRandumbTensor, RandumbTensor


def stepgen(offset, step):
    """offset, offset+step, offset+2*step, ... -- a whole model's seeds are then two integers."""
    i = 0
    while True:
        yield offset + step * i
        i += 1


def listgen(lst):
    for i in lst:
        yield i


def kaiming_out_std(fan_in: int, a: float = math.sqrt(5)) -> float:
    """Standard deviation nn.Linear's default init gives its weight: gain / sqrt(fan_in)."""
    gain = math.sqrt(2.0 / (1 + a * a))
    return gain / math.sqrt(fan_in)


def coef_std_for(out_std: float, int_dim: int) -> float:
    """var(W) = int_dim * var(S) * var(coef) with var(S) = 1/3  =>  std(coef) = sqrt(3/int_dim) * std(W)
    (reference: SillyLayers.py:62-71, README.md:20-29)."""
    return math.sqrt(3.0 / int_dim) * out_std


class RandumbModuleMixin(nn.Module):
    """``.to()/.cuda()/.float()`` rebuild the RandumbTensor buffers around the moved parameters, because a
    wrapper subclass cannot change device or dtype in place (reference: SillyLayers.py:89-113)."""

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        self._rebuild_virtual_buffers()
        return self

    def _rebuild_virtual_buffers(self):
        for name, buf in list(self._buffers.items()):
            if isinstance(buf, RandumbTensor):
                coef = getattr(self, f"{name}_coef")
                scale_bias = getattr(self, f"{name}_scale_bias", buf.scale_bias)
                self._buffers[name] = CreateRandumbTensor(coef, buf.seed, buf.shape, scale_bias, buf.fused_bias, buf.row0)

    def init_rt_scale_bias(self, val: float = 0.0) -> None:
        """One trainable scale per 1-D-form virtual buffer for the fused random bias, registered as
        ``<buffer>_scale_bias`` (reference: SillyLayers.py:116-120)."""
        for name, buf in list(self._buffers.items()):
            if isinstance(buf, RandumbTensor) and not buf.is_matrix_form:
                coef = getattr(self, f"{name}_coef")
                p = nn.Parameter(torch.tensor([val], dtype=coef.dtype, device=coef.device))
                self.register_parameter(f"{name}_scale_bias", p)
                self._buffers[name] = CreateRandumbTensor(coef, buf.seed, buf.shape, p, buf.fused_bias, buf.row0)

    def _fan_in_std(self) -> float:
        w = self._buffers["weight"]
        fan_in = w.shape[1] if w.dim() == 2 else int(w.shape[1:].numel())
        return kaiming_out_std(fan_in)

    def init_zero_coef_uniform_bias(self) -> None:
        """The reference layers' default start (SillyLayers.py:122-133): coefficient vectors zero, every
        ``<buffer>_scale_bias`` equal to nn.Linear's uniform bound ``sqrt(3) * gain / sqrt(fan_in)``."""
        self.init_rt_scale_bias(math.sqrt(3.0) * self._fan_in_std())
        with torch.no_grad():
            for name, buf in self._buffers.items():
                if isinstance(buf, RandumbTensor) and not buf.is_matrix_form:
                    getattr(self, f"{name}_coef").zero_()

    def init_uniform_coef_zero_bias(self) -> None:
        """The reference's alternative start (SillyLayers.py:135-138, 37-79): uniform coefficients whose variance
        gives the virtual weight nn.Linear's default std, random-bias scales zero.  One generator seeded with the
        layer's first seed draws the weight coefficients, then the bias coefficients."""
        self.init_rt_scale_bias(0.0)
        out_std = self._fan_in_std()
        seed0 = self.seed[0] if isinstance(self.seed, (list, tuple)) else self.seed
        coef_w = getattr(self, "weight_coef")
        gen = torch.Generator(device=coef_w.device).manual_seed(int(seed0))
        with torch.no_grad():
            for name in ("weight", "bias"):
                buf = self._buffers.get(name)
                if isinstance(buf, RandumbTensor) and not buf.is_matrix_form:
                    coef = getattr(self, f"{name}_coef")
                    bound = math.sqrt(3.0) * coef_std_for(out_std, coef.shape[0])
                    coef.uniform_(-bound, bound, generator=gen)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # The reference registers its virtual tensors as persistent buffers, so its checkpoints carry a dense copy of
        # every weight and bias beside the coefficients (SillyLayers.py:207, 212).  Those copies are redundant here
        # (the buffers are regenerated from seed + coefficients): drop them instead of failing on unexpected keys.
        for name, buf in self._buffers.items():
            if isinstance(buf, RandumbTensor):
                state_dict.pop(prefix + name, None)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class RandumbLinear(RandumbModuleMixin, nn.Module):
    """``y = x @ (S @ C).T (+ b)`` with ``S = noise(out_features, d_c; seed)`` regenerated inside the kernels.

    Args:
        in_features, out_features: as nn.Linear.
        d_c: coefficient (intrinsic) dimension; the trainable state is ``coef[d_c, in_features]``.
        seed: noise seed of this layer.
        bias: ordinary dense bias vector (not pseudorandom).
        row0: global index of this module's first output row -- a rank that owns rows
            ``[row0, row0 + out_features)`` of a larger virtual layer regenerates exactly those rows.
        init_std: target std of the virtual weight; default is nn.Linear's Kaiming-uniform equivalent.
            ``coef ~ N(0, 3 * init_std**2 / d_c)``.
    """

    def __init__(self, in_features: int, out_features: int, d_c: int, seed: int, bias: bool = False, device=None,
                 dtype=None, row0: int = 0, init_std: Optional[float] = None):
        super().__init__()
        self.in_features, self.out_features, self.d_c, self.seed, self.row0 = in_features, out_features, d_c, int(seed), int(row0)
        self.init_std = init_std if init_std is not None else kaiming_out_std(in_features)
        self.weight_coef = nn.Parameter(torch.empty((d_c, in_features), device=device, dtype=dtype))
        self.register_buffer("weight", CreateRandumbTensor(self.weight_coef, self.seed, (out_features, in_features), row0=self.row0),
                             persistent=False)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        gen = torch.Generator(device=self.weight_coef.device).manual_seed(self.seed & 0x7FFFFFFFFFFFFFFF)
        with torch.no_grad():
            self.weight_coef.normal_(0.0, coef_std_for(self.init_std, self.d_c), generator=gen)
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        coef = self.weight_coef if self.weight_coef.dtype == input.dtype else self.weight_coef.to(input.dtype)
        return ops.rlinear(input, coef, self.seed, self.out_features, self.row0, self.bias)

    def get_extra_state(self):
        return {"seed": self.seed, "d_c": self.d_c, "out_features": self.out_features, "row0": self.row0}

    def set_extra_state(self, state):
        if state["d_c"] != self.d_c or state["out_features"] != self.out_features:
            raise RuntimeError(f"checkpoint describes a different layer: {state}")
        self.seed, self.row0 = int(state["seed"]), int(state["row0"])
        self._rebuild_virtual_buffers_with_seed()

    def _rebuild_virtual_buffers_with_seed(self):
        self._buffers["weight"] = CreateRandumbTensor(self.weight_coef, self.seed, (self.out_features, self.in_features),
                                                      row0=self.row0)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, d_c={self.d_c}, seed={self.seed}, "
                f"row0={self.row0}, bias={self.bias is not None}")


class SillyLinear(RandumbModuleMixin, nn.Module):
    """The reference's linear layer (src/rten_cpp/SillyLayers.py:142-227): weight and bias are both RandumbTensors.

    ``int_dim`` / ``seed``: list of two values or a generator (first for the weight, second for the bias).
    With the default ``coef_form="vector"`` an unchanged reference call site gets the reference's layer: ``weight_coef``
    is ``[int_dim[0]]``, ``bias_coef`` ``[int_dim[1]]``, one ``<name>_scale_bias`` parameter per virtual tensor, all
    coefficients zero at the start and the scales equal to nn.Linear's uniform bound (``init_zero_coef_uniform_bias``,
    SillyLayers.py:122-133, 218-221); ``rt_bias`` decides whether the fused random bias ``scale_bias * noise1d`` is
    added when the tensors are materialised.  The forward is ``mat1 @ RT`` on the library's own kernels (``ops.rt_mm``).
    A reference checkpoint loads into it (its dense ``weight`` / ``bias`` entries are ignored).

    ``coef_form="matrix"`` is this library's extension: the weight takes the matrix-coefficient form
    (``weight_coef`` is ``[int_dim[0], in_features]``, fused tensor-core operator, uniform start with the variance of
    ``init_kaiming_uniform``, SillyLayers.py:37-79); the bias keeps the 1-D form.  ``RandumbLinear`` is the plain
    module for that form.
    """
    num_seeds = 2

    def __init__(self, in_features: int, out_features: int, int_dim: Union[list, Generator], seed: Union[list, Generator],
                 bias: bool = True, rt_bias: bool = False, device=None, dtype=None, coef_form: str = "vector") -> None:
        super().__init__()
        if coef_form not in ("matrix", "vector"):
            raise ValueError(f"coef_form must be 'matrix' or 'vector', got {coef_form!r}")
        self.in_features, self.out_features, self.rt_bias, self.coef_form = in_features, out_features, rt_bias, coef_form
        self.int_dim = [next(int_dim) for _ in range(self.num_seeds)] if isinstance(int_dim, GeneratorType) else list(int_dim)
        self.seed = [next(seed) for _ in range(self.num_seeds)] if isinstance(seed, GeneratorType) else list(seed)
        vector = coef_form == "vector"
        wshape = (self.int_dim[0],) if vector else (self.int_dim[0], in_features)
        self.weight_coef = nn.Parameter(torch.empty(wshape, dtype=dtype, device=device))
        self.register_buffer("weight", CreateRandumbTensor(self.weight_coef, self.seed[0], (out_features, in_features),
                                                           fused_bias=rt_bias and vector), persistent=False)
        if bias:
            self.bias_coef = nn.Parameter(torch.empty(self.int_dim[1], dtype=dtype, device=device))
            self.register_buffer("bias", CreateRandumbTensor(self.bias_coef, self.seed[1], (out_features,), fused_bias=rt_bias),
                                 persistent=False)
        else:
            self.bias = None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        self.init_zero_coef_uniform_bias()           # every 1-D-form tensor: zero coefficients, scale = uniform bound
        if self.coef_form == "matrix":
            out_std = kaiming_out_std(self.in_features)
            gen = torch.Generator(device=self.weight_coef.device).manual_seed(self.seed[0] & 0x7FFFFFFFFFFFFFFF)
            bound = math.sqrt(3.0) * coef_std_for(out_std, self.int_dim[0])
            with torch.no_grad():
                self.weight_coef.uniform_(-bound, bound, generator=gen)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if self.coef_form == "vector" and input.is_cuda:
            # x @ W^T with W materialised by the library's kernel and multiplied by the library's own product kernels
            # (the reference ends in a library GEMM here: RandumbTensor.py:942-946, 771-791)
            lead = input.shape[:-1]
            x2 = input.reshape(-1, self.in_features)
            y = ops.rt_mm(x2, w._coef, [self.in_features, self.out_features], [1, self.in_features], w.seed, w.scale_bias,
                          w.fused_bias).reshape(*lead, self.out_features)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        return F.linear(input, w, self.bias)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, int_dim={self.int_dim}, "
                f"seeds={self.seed}, bias={self.bias is not None}, coef_form={self.coef_form}, rt_bias={self.rt_bias}")


class SillyEmbedding(RandumbModuleMixin, nn.Module):
    """Embedding table that is a RandumbTensor in the 1-D coefficient form (reference:
    SillyLayers.py:301-366; same constructor arguments in the same order): ``forward(idx)`` regenerates only the
    looked-up rows, ``rten::embed_fwd``.  ``padding_idx``, ``max_norm``, ``scale_grad_by_freq`` and ``sparse`` are
    accepted and, as in the reference, not applied; ``rt_bias`` only registers the (zero) ``weight_scale_bias``
    parameter -- the reference's lookup kernel does not add the random bias either (RandumbTensor.py:998-1057)."""
    num_seeds = 1

    def __init__(self, num_embeddings: int, embedding_dim: int, int_dim: Union[list, Generator], seed: Union[list, Generator],
                 rt_bias: bool = False, padding_idx: Optional[int] = None, max_norm: Optional[float] = None,
                 norm_type: float = 2.0, scale_grad_by_freq: bool = False, sparse: bool = False,
                 _weight: Optional[RandumbTensor] = None, _freeze: bool = False, device="cuda", dtype=None) -> None:
        super().__init__()
        assert padding_idx is None, "padding_idx not supported"
        self.num_embeddings, self.embedding_dim, self.rt_bias = num_embeddings, embedding_dim, rt_bias
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        self.int_dim = [next(int_dim) for _ in range(self.num_seeds)] if isinstance(int_dim, GeneratorType) else list(int_dim)
        self.seed = [next(seed) for _ in range(self.num_seeds)] if isinstance(seed, GeneratorType) else list(seed)
        if _weight is None:
            self.weight_coef = nn.Parameter(torch.empty(self.int_dim[0], dtype=dtype, device=device), requires_grad=not _freeze)
            self.register_buffer("weight", CreateRandumbTensor(self.weight_coef, self.seed[0], (num_embeddings, embedding_dim)),
                                 persistent=False)
            self.reset_parameters()
        else:
            assert list(_weight.shape) == [num_embeddings, embedding_dim], \
                f"Shape of weight {_weight.shape} does not match num_embeddings and embedding_dim"
            self.register_buffer("weight", _weight, persistent=False)
            self.weight_coef = _weight._coef

    def reset_parameters(self) -> None:
        # reference: init_kaiming_uniform on the coefficient vector, generator seeded with the layer's seed
        # (SillyLayers.py:362-365, 37-79); the (unused) scale starts at zero
        if self.rt_bias:
            self.init_rt_scale_bias(0.0)
        out_std = kaiming_out_std(self.embedding_dim)
        gen = torch.Generator(device=self.weight_coef.device).manual_seed(int(self.seed[0]))
        with torch.no_grad():
            bound = math.sqrt(3.0) * coef_std_for(out_std, self.int_dim[0])
            self.weight_coef.uniform_(-bound, bound, generator=gen)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return ops.embed_fwd(input, self.weight_coef, self.embedding_dim, self.weight.seed).to(self.weight_coef.dtype)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}, int_dim={self.int_dim}, seeds={self.seed}"


class SillyConv2d(RandumbModuleMixin, nn.Conv2d):
    """``nn.Conv2d`` whose weight ``[out, in/groups, kh, kw]`` and bias are RandumbTensors in the 1-D coefficient
    form (reference: SillyLayers.py:230-297); the convolution itself is PyTorch's, on the weight materialised for the
    call by ``rten::materialize_fwd`` and dropped afterwards.  Starts like the reference: zero coefficients, one
    ``<name>_scale_bias`` per virtual tensor equal to the uniform bound; ``rt_bias`` switches the fused random bias on."""
    num_seeds = 2

    def __init__(self, in_channels: int, out_channels: int, int_dim: Union[list, Generator], seed: Union[list, Generator],
                 kernel_size, stride=1, padding=0, dilation=1, groups: int = 1, bias: bool = True, rt_bias: bool = False,
                 padding_mode: str = "zeros", device=None, dtype=None) -> None:
        self.int_dim = [next(int_dim) for _ in range(self.num_seeds)] if isinstance(int_dim, GeneratorType) else list(int_dim)
        self.seed = [next(seed) for _ in range(self.num_seeds)] if isinstance(seed, GeneratorType) else list(seed)
        self.rt_bias = rt_bias
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode,
                         device=device, dtype=dtype)

    def reset_parameters(self) -> None:
        # nn.Conv2d.__init__ has created dense parameters: keep their shapes, replace them by coefficient vectors
        w = self.weight
        self.weight_coef = nn.Parameter(torch.empty(self.int_dim[0], dtype=w.dtype, device=w.device))
        wshape = tuple(w.shape)
        del self.weight
        self.register_buffer("weight", CreateRandumbTensor(self.weight_coef, self.seed[0], wshape, fused_bias=self.rt_bias),
                             persistent=False)
        if self.bias is not None:
            b = self.bias
            self.bias_coef = nn.Parameter(torch.empty(self.int_dim[1], dtype=b.dtype, device=b.device))
            bshape = tuple(b.shape)
            del self.bias
            self.register_buffer("bias", CreateRandumbTensor(self.bias_coef, self.seed[1], bshape, fused_bias=self.rt_bias),
                                 persistent=False)
        self.init_zero_coef_uniform_bias()

    def extra_repr(self) -> str:
        return super().extra_repr() + f", int_dim={self.int_dim}, seeds={self.seed}"
