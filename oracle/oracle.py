"""TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.

CPU restatement (numpy + torch on the host) of the randumb pseudorandom-weight
path.  Only ``tests/``, the smoke test and the benchmark's CPU-baseline legs may
import this module; nothing under ``randumb_b200/`` does.

Parity pin: ``noise_bits`` / ``noise_f32`` are compared bit-for-bit with the
outputs of the reference's own Triton kernels run under the Triton interpreter
(``tests/golden/make_golden.py`` wrote ``tests/golden/*.npz``); the C twin in
``sq5_oracle.c`` is checked against the same vectors.

Reference locations restated here (paths inside the reference project):
  * hash: ``src/rten_cpp/RandumbTensor.py:130-164`` and ``csrc/cuda/rten.cu:28-48``
  * 1-D hash: ``src/rten_cpp/RandumbTensor.py:204-232``
  * noise matrix orientation (row index first): ``RandumbTensor.py:78-99``
  * materialise fwd / bwd with a 1-D coefficient vector: ``RandumbTensor.py:235-290, 304-359``
  * "explicit noise matrix, then torch matmul and autograd" -- the reference's own
    cross-check: ``benchmark.py:144-148, 379-383``.  The matrix-coefficient layer
    ``W = S @ C`` (S: [N, R] noise, C: [R, K] trainable) is evaluated that way.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

N1 = np.uint32(0xD2A80A3F)
N2 = np.uint32(0xA884F197)
N3 = np.uint32(0x6C736F4B)
N4 = np.uint32(0xB79F3ABB)
N5 = np.uint32(0x1B56C4F5)
PRIME = np.uint32(198491317)

_HERE = os.path.dirname(os.path.abspath(__file__))


def _mix(pos: np.ndarray, seed: int) -> np.ndarray:
    """The eleven mixing steps on uint32 positions (wrap-around arithmetic)."""
    with np.errstate(over="ignore"):
        b = pos.astype(np.uint32, copy=True)
        b *= N1
        b += np.uint32(seed & 0xFFFFFFFF)
        b ^= b >> np.uint32(9)
        b += N2
        b ^= b >> np.uint32(11)
        b *= N3
        b ^= b >> np.uint32(13)
        b += N4
        b ^= b >> np.uint32(15)
        b *= N5
        b ^= b >> np.uint32(17)
    return b


def noise_bits(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0) -> np.ndarray:
    """uint32 hash words of S[row0:row0+rows, col0:col0+cols]; position = PRIME*row + col mod 2^32."""
    with np.errstate(over="ignore"):
        r = (np.arange(row0, row0 + rows, dtype=np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        c = (np.arange(col0, col0 + cols, dtype=np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        pos = (PRIME * r)[:, None] + c[None, :]
    return _mix(pos, seed)


def bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """float32(int32(bits)) * float32(1/0x7FFFFFFF) (that float32 constant is exactly 2**-31)."""
    scale = np.float32(1.0) / np.float32(0x7FFFFFFF)
    return bits.view(np.int32).astype(np.float32) * scale


def noise_f32(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0) -> np.ndarray:
    return bits_to_f32(noise_bits(rows, cols, seed, row0, col0))


def noise_bits_1d(n: int, seed: int, idx0: int = 0) -> np.ndarray:
    idx = (np.arange(idx0, idx0 + n, dtype=np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    return _mix(idx, seed)


def noise_bf16(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0) -> torch.Tensor:
    """Canonical bf16 noise: round-to-nearest-even of the float32 value."""
    return torch.from_numpy(noise_f32(rows, cols, seed, row0, col0)).to(torch.bfloat16)


# ----------------------------------------------------------------------------------------------
# 1-D coefficient form of the reference (materialise forward / backward)
# ----------------------------------------------------------------------------------------------
def _rows_dot(rows: np.ndarray, coef: np.ndarray, seed: int) -> np.ndarray:
    """sum_m S[rows[n], m] * coef[m] for a vector of noise row numbers (float64 accumulation)."""
    with np.errstate(over="ignore"):
        pos = (PRIME * (rows & 0xFFFFFFFF).astype(np.uint32))[:, None] + np.arange(coef.size, dtype=np.uint32)[None, :]
    S = bits_to_f32(_mix(pos, seed)).astype(np.float64)
    return S @ coef.astype(np.float64)


def materialize_fwd(coef: np.ndarray, P: int, Q: int, stride_P: int, stride_Q: int, seed: int,
                    scale_bias: float | None = None) -> np.ndarray:
    """out[n] = sum_m S[sq(n), m] * coef[m] (+ scale_bias * noise1d(sq(n)));  sq(n) = (n % Q)*stride_Q + (n // Q)*stride_P.
    Reference: src/rten_cpp/RandumbTensor.py:235-290 (bias branch :283-286)."""
    n = np.arange(P * Q, dtype=np.int64)
    sq = (n % Q) * stride_Q + (n // Q) * stride_P
    out = _rows_dot(sq, coef, seed)
    if scale_bias is not None:
        out = out + float(scale_bias) * bits_to_f32(_mix((sq & 0xFFFFFFFF).astype(np.uint32), seed)).astype(np.float64)
    return out.reshape(P, Q)


def materialize_bwd(dout: np.ndarray, M: int, seed: int) -> np.ndarray:
    """dcoef[m] = sum_n S[n, m] * dout_flat[n]."""
    d = dout.reshape(-1).astype(np.float64)
    S = noise_f32(d.size, M, seed).astype(np.float64)
    return S.T @ d


def scale_bias_bwd(dout: np.ndarray, seed: int) -> float:
    """sum_n dout_flat[n] * noise1d(n).  Reference: src/rten_cpp/RandumbTensor.py:400-407."""
    d = dout.reshape(-1).astype(np.float64)
    return float(bits_to_f32(noise_bits_1d(d.size, seed)).astype(np.float64) @ d)


def _embed_rows(idx: np.ndarray, rowsize: int) -> np.ndarray:
    i = idx.reshape(-1).astype(np.int64)
    return (i[:, None] * rowsize + np.arange(rowsize, dtype=np.int64)[None, :]).reshape(-1)


def embed_fwd(idx: np.ndarray, coef: np.ndarray, rowsize: int, seed: int) -> np.ndarray:
    """out[i, j] = sum_m S[idx[i]*rowsize + j, m] * coef[m].  Reference: src/rten_cpp/RandumbTensor.py:999-1056."""
    return _rows_dot(_embed_rows(idx, rowsize), coef, seed).reshape(idx.size, rowsize)


def embed_bwd(idx: np.ndarray, dout: np.ndarray, M: int, rowsize: int, seed: int) -> np.ndarray:
    """dcoef[m] = sum_{i,j} S[idx[i]*rowsize + j, m] * dout[i, j].  Reference: src/rten_cpp/RandumbTensor.py:1060-1107."""
    rows = _embed_rows(idx, rowsize)
    with np.errstate(over="ignore"):
        pos = (PRIME * (rows & 0xFFFFFFFF).astype(np.uint32))[:, None] + np.arange(M, dtype=np.uint32)[None, :]
    S = bits_to_f32(_mix(pos, seed)).astype(np.float64)
    return S.T @ dout.reshape(-1).astype(np.float64)


# ----------------------------------------------------------------------------------------------
# matrix-coefficient layer  W = S @ C,  y = x @ W.T   (explicit S, torch matmul, autograd)
# ----------------------------------------------------------------------------------------------
def linear_reference(x: torch.Tensor, coef: torch.Tensor, seed: int, out_features: int, row0: int = 0,
                     dy: torch.Tensor | None = None, dtype: torch.dtype = torch.float64):
    """Returns (y, dx, dc) computed in ``dtype`` from the given (already rounded) inputs.

    S is the unrounded float32 noise.  Mirrors materialise -> mm -> MmBackward ->
    constructor backward of the reference (RandumbTensor.py:892, 946, 986).
    """
    R, K = coef.shape
    S = torch.from_numpy(noise_f32(out_features, R, seed, row0=row0)).to(dtype)
    xd = x.detach().to(dtype).reshape(-1, K).requires_grad_(dy is not None)
    cd = coef.detach().to(dtype).requires_grad_(dy is not None)
    W = S @ cd
    y = torch.nn.functional.linear(xd, W)
    if dy is None:
        return y.detach(), None, None
    y.backward(dy.detach().to(dtype).reshape(-1, out_features))
    return y.detach(), xd.grad, cd.grad


# ----------------------------------------------------------------------------------------------
# comparison helpers (the two tests every parity check applies)
# ----------------------------------------------------------------------------------------------
def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    den = float(torch.linalg.norm(b))
    return float(torch.linalg.norm(a - b)) / (den if den > 0 else 1.0)


def close(a: torch.Tensor, b: torch.Tensor, tol: float) -> bool:
    """rel-Frobenius <= tol and allclose(rtol=tol, atol=tol*rms(b))."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    rms = float(torch.sqrt(torch.mean(b * b))) if b.numel() else 0.0
    return rel_fro(a, b) <= tol and bool(torch.allclose(a, b, rtol=tol, atol=tol * max(rms, 1e-30)))


# ----------------------------------------------------------------------------------------------
# C twin
# ----------------------------------------------------------------------------------------------
def build_c(quiet: bool = True) -> str:
    """Compile sq5_oracle.c into oracle/_build/liborc.so (gcc) and return its path."""
    out = os.path.join(_HERE, "_build", "liborc.so")
    src = os.path.join(_HERE, "sq5_oracle.c")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True,
                       stdout=subprocess.DEVNULL if quiet else None)
    return out


_C = None


def c_lib():
    global _C
    if _C is None:
        lib = ctypes.CDLL(build_c())
        i64, u32, vp = ctypes.c_int64, ctypes.c_uint32, ctypes.c_void_p
        lib.orc_sq5_bits.restype = u32
        lib.orc_sq5_bits.argtypes = [u32, u32, u32]
        lib.orc_sq5_bits_1d.restype = u32
        lib.orc_sq5_bits_1d.argtypes = [u32, u32]
        lib.orc_sq5_float.restype = ctypes.c_float
        lib.orc_sq5_float.argtypes = [u32, u32, u32]
        lib.orc_noise_bits.argtypes = [vp, i64, i64, i64, i64, i64, u32]
        lib.orc_noise_f32.argtypes = [vp, i64, i64, i64, i64, i64, u32]
        lib.orc_noise_1d_f32.argtypes = [vp, i64, i64, u32]
        lib.orc_materialize_fwd.argtypes = [vp, vp, i64, i64, i64, i64, i64, u32]
        lib.orc_materialize_bwd.argtypes = [vp, vp, i64, i64, u32]
        lib.orc_linear_fwd.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, u32]
        lib.orc_linear_bwd.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, u32]
        _C = lib
    return _C


def c_noise_bits(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.uint32)
    c_lib().orc_noise_bits(out.ctypes.data, rows, cols, cols, row0, col0, seed & 0xFFFFFFFF)
    return out


def c_noise_f32(rows: int, cols: int, seed: int, row0: int = 0, col0: int = 0) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float32)
    c_lib().orc_noise_f32(out.ctypes.data, rows, cols, cols, row0, col0, seed & 0xFFFFFFFF)
    return out


def c_linear_fwd(x: np.ndarray, C: np.ndarray, N: int, seed: int, row0: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    C = np.ascontiguousarray(C, dtype=np.float32)
    T, K = x.shape
    R = C.shape[0]
    y = np.empty((T, N), dtype=np.float64)
    c_lib().orc_linear_fwd(y.ctypes.data, x.ctypes.data, C.ctypes.data, T, K, N, R, row0, seed & 0xFFFFFFFF)
    return y


def c_linear_bwd(dy: np.ndarray, x: np.ndarray, C: np.ndarray, seed: int, row0: int = 0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    C = np.ascontiguousarray(C, dtype=np.float32)
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    T, K = x.shape
    R = C.shape[0]
    N = dy.shape[1]
    dx = np.empty((T, K), dtype=np.float64)
    dc = np.empty((R, K), dtype=np.float64)
    c_lib().orc_linear_bwd(dx.ctypes.data, dc.ctypes.data, dy.ctypes.data, x.ctypes.data, C.ctypes.data,
                           T, K, N, R, row0, seed & 0xFFFFFFFF)
    return dx, dc
