"""randumb_b200 -- B200-native (sm_100a) pseudorandom-weight linear layer.

The weight of a layer is never stored: ``W = S @ C`` with ``S`` Squirrel5 noise regenerated inside the
kernels from a seed and ``C`` a small trainable coefficient matrix.  Public surface (mirrors the
reference package ``rten_cpp``):

* ``ops``      torch.library operators (``rten::rlinear_fwd`` ..., ``rten::materialize_fwd`` ...)
* ``RandumbTensor`` / ``CreateRandumbTensor``   storage-less tensor subclass + differentiable constructor
* ``RandumbLinear`` / ``SillyLinear`` / ``SillyEmbedding`` / ``SillyConv2d`` / ``stepgen`` / ``listgen``   modules
* ``parallel`` row sharding over GPUs and the dC all-reduce
* ``kernels``  tensor-level wrappers over the C ABI (``include/randumb_b200.h``)

Importing the package does not need a GPU; running any kernel does, and there is no CPU fallback.
"""
from . import kernels, ops, parallel  # noqa: F401
from .layers import RandumbLinear, SillyConv2d, SillyEmbedding, SillyLinear, listgen, stepgen  # noqa: F401
from .ops import rlinear  # noqa: F401
from .tensor import CreateRandumbTensor, RandumbTensor  # noqa: F401

__all__ = ["kernels", "ops", "parallel", "RandumbLinear", "SillyLinear", "SillyEmbedding", "SillyConv2d", "listgen", "stepgen", "rlinear",
           "CreateRandumbTensor", "RandumbTensor"]
