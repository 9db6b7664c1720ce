"""ctypes binding of librandumb_b200.so (the C ABI declared in include/randumb_b200.h).

There is no fallback: if the shared library is missing the import of any compute entry raises,
and every wrapper raises ``RuntimeError`` carrying ``rdb_strerror`` on a non-zero return code.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# RANDUMB_B200_LIB points at a library built elsewhere (same C ABI); default is the in-tree build.
LIB_PATH = os.environ.get("RANDUMB_B200_LIB") or os.path.join(_HERE, "lib", "librandumb_b200.so")

# constants mirrored from include/randumb_b200.h
F32, BF16 = 0, 1
PATH_AUTO, PATH_FACTORED, PATH_WPATH = 0, 1, 2
IMPL_AUTO, IMPL_SIMT, IMPL_UMMA = 0, 1, 2
OPT_NOISE_TILE = 1
OPT_DENSE_PAIR = 2
OPT_STAGE_NOISE = 3
OPT_RESERVE_SMS = 4
OPT_FILL_OVERLAP = 5
OPT_GEMV_FUSED = 6
OPT_GRADS_BESIDE = 7
MAX_RESERVE_SMS = 64
MAX_PEERS = 8
STATUS_NAMES = {0: "ok", 1: "producer wait expired", 2: "mma wait expired", 3: "epilogue wait expired",
                4: "generator wait expired", 5: "peer wait expired"}

_i64, _u32, _i32, _vp, _sz = ctypes.c_int64, ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t


class CallOptions(ctypes.Structure):
    """``rdb_call_options``: per-call values of the tuning switches; a field < 0 keeps the process default."""
    _fields_ = [("noise_tile", ctypes.c_int32), ("dense_pair", ctypes.c_int32), ("stage_noise", ctypes.c_int32),
                ("reserve_sms", ctypes.c_int32), ("fill_overlap", ctypes.c_int32), ("grads_beside", ctypes.c_int32)]

    def __init__(self, noise_tile: int = -1, dense_pair: int = -1, stage_noise: int = -1, reserve_sms: int = -1,
                 fill_overlap: int = -1, grads_beside: int = -1):
        super().__init__(noise_tile, dense_pair, stage_noise, reserve_sms, fill_overlap, grads_beside)


_op = ctypes.POINTER(CallOptions)

# name -> (restype, argtypes); one entry per declaration in the header
PROTOTYPES = {
    "rdb_version": (_i32, []),
    "rdb_strerror": (ctypes.c_char_p, [_i32]),
    "rdb_set_option": (_i32, [_i32, _i32]),
    "rdb_set_profile_buffer": (_i32, [_vp, _sz]),
    "rdb_noise_bits": (_i32, [_vp, _i64, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_noise": (_i32, [_vp, _i32, _i64, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_noise_1d": (_i32, [_vp, _i64, _i64, _u32, _vp]),
    "rdb_linear_workspace_bytes": (_sz, [_i32, _i64, _i64, _i64, _i64, _i32, _i32, _i32]),
    "rdb_linear_workspace_bytes_ex": (_sz, [_i32, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _op]),
    "rdb_linear_stages_noise": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32]),
    "rdb_linear_stages_noise_ex": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32, _op]),
    "rdb_linear_path": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32]),
    "rdb_linear_bwd_plan": (_i32, [_i64, _i64, _i64, _i64, _i32, _i32, _i32, _op, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "rdb_linear_fwd_ex": (_i32, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _u32, _i32, _i32, _i32, _op, _vp, _vp]),
    "rdb_linear_bwd_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _u32, _i32, _i32, _i32,
                                 _op, _vp, _vp]),
    "rdb_gemm_dense_ex": (_i32, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _op,
                                 _vp, _vp]),
    "rdb_linear_fwd": (_i32, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _u32, _i32, _i32, _i32, _vp, _vp]),
    "rdb_linear_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _u32, _i32, _i32, _i32,
                              _vp, _vp]),
    "rdb_linear_weight": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _u32, _i32, _vp]),
    "rdb_gemv_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_gemv_fwd_static": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_gemv_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "rdb_gemv_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_gemm_noise": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i64, _i64, _u32, _i32, _vp, _vp]),
    "rdb_gemm_dense": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp,
                              _vp]),
    "rdb_gemm_dense_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "rdb_gemm_dense_ws": (_i32, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp,
                          _vp]),
    "rdb_peer_barrier": (_i32, [_vp, _i32, _i32, ctypes.c_uint64, _vp, _vp]),
    "rdb_peer_copy": (_i32, [_vp, _i32, _sz, _vp, _sz, _i32, _vp]),
    "rdb_peer_scatter": (_i32, [_vp, _i32, _sz, _vp, _sz, _i32, _vp]),
    "rdb_reduce_slots_bf16": (_i32, [_vp, _vp, _sz, _i32, _sz, _vp]),
    "rdb_gemm_dense_scatter": (_i32, [_vp, _i32, _sz, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _op, _vp, _vp]),
    "rdb_materialize_fwd": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _u32, _vp]),
    "rdb_materialize_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "rdb_materialize_bwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _u32, _vp]),
    "rdb_scale_bias_bwd_workspace_bytes": (_sz, [_i64]),
    "rdb_scale_bias_bwd": (_i32, [_vp, _vp, _vp, _i64, _u32, _vp]),
    "rdb_embed_fwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _u32, _vp]),
    "rdb_embed_bwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _u32, _vp]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once; raise loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m randumb_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for the kernels)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def strerror(code: int) -> str:
    return lib().rdb_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: [{code}] {strerror(code)}")
