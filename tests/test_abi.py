"""The C-ABI library loads without a GPU, exports every symbol the header declares, and rejects bad
arguments on the host before any launch.  (No compute call is made here.)"""
import ctypes
import os
import re

import pytest

from randumb_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "randumb_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rdb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(built_lib):
    declared = _declared_symbols()
    assert declared, "no declarations parsed from the header"
    assert sorted(_lib.PROTOTYPES.keys()) == declared


def test_every_declared_symbol_is_exported(built_lib):
    handle = ctypes.CDLL(built_lib)
    for name in _declared_symbols():
        assert hasattr(handle, name), f"{name} declared in include/randumb_b200.h but not exported"


def test_version_and_strerror(built_lib):
    L = _lib.lib()
    assert L.rdb_version() == 100
    assert _lib.strerror(0) == "ok"
    for code in range(-8, 0):
        assert _lib.strerror(code) not in ("ok", "unknown error")


def test_argument_errors_are_caught_on_host(built_lib):
    L = _lib.lib()
    assert L.rdb_noise_bits(None, -1, 4, 4, 0, 0, 0, None) == -2            # negative rows
    assert L.rdb_noise_bits(None, 4, 4, 2, 0, 0, 0, None) == -2             # ld < cols
    assert L.rdb_noise_bits(None, 4, 4, 4, 0, 0, 0, None) == -1             # null output
    assert L.rdb_noise(None, 7, 4, 4, 4, 0, 0, 0, None) == -1               # null output checked first
    assert L.rdb_noise_bits(None, 0, 4, 4, 0, 0, 0, None) == 0              # empty is fine
    assert L.rdb_linear_fwd(None, None, None, None, 0, 4, 4, 4, 4, 0, 0, 5, 0, 0, None, None) == -3   # dtype
    assert L.rdb_linear_fwd(None, None, None, None, 0, 4, 4, 4, 4, 0, 0, 0, 0, 0, None, None) == -1   # null y
    assert L.rdb_linear_fwd(None, None, None, None, 0, 0, 4, 4, 4, 0, 0, 0, 0, 0, None, None) == 0    # T == 0
    assert L.rdb_linear_bwd(None, None, None, None, None, None, 0, 4, 4, 4, 4, 0, 0, 0, 0, 0, None, None) == 0  # nothing asked
    assert L.rdb_gemm_noise(None, None, 4, 4, 4, 2, 4, 0, 0, 0, 0, 0, 0, 0, None, None) == -2  # lda < Kc
    assert L.rdb_gemm_dense(None, None, None, 4, 4, 4, 4, 4, 2, 0, 0, 0, 1, 1, 0, None, None) == -2     # ldd < N
    assert L.rdb_set_option(99, 1) == -6


def test_workspace_sizes(built_lib):
    L = _lib.lib()
    # bf16 factored on tensor cores: z or g, bf16 [T, R], plus S bf16 [N, R] when the noise operand is staged
    zg, S = 8192 * 1024 * 2, 16384 * 1024 * 2
    assert L.rdb_linear_stages_noise(8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == 1
    assert L.rdb_linear_workspace_bytes(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg + S
    assert L.rdb_linear_workspace_bytes(1, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg + S
    assert L.rdb_set_option(_lib.OPT_STAGE_NOISE, 1) == 0          # regenerate inside the kernel: nothing of S in memory
    try:
        assert L.rdb_linear_stages_noise(8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == 0
        assert L.rdb_linear_workspace_bytes(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg
    finally:
        assert L.rdb_set_option(_lib.OPT_STAGE_NOISE, 0) == 1
    # few tokens: one 512-token tile regenerates S once anyway; a noise block above 1 GiB is never staged
    assert L.rdb_linear_stages_noise(512, 4096, 16384, 1024, _lib.BF16, 0, 0) == 0
    assert L.rdb_linear_stages_noise(8192, 4096, 1 << 20, 1024, _lib.BF16, 0, 0) == 0
    assert L.rdb_linear_stages_noise(8192, 4096, 16384, 1024, _lib.F32, 0, 0) == 0
    # fp32 factored: f32 [T, R]
    assert L.rdb_linear_workspace_bytes(0, 64, 784, 256, 64, _lib.F32, 0, 0) == 64 * 64 * 4
    # a 256 -> 10 head is cheaper through W: f32 [N, K] (+ dW in backward)
    assert L.rdb_linear_workspace_bytes(0, 64, 256, 10, 64, _lib.F32, 0, 0) == 10 * 256 * 4
    assert L.rdb_linear_workspace_bytes(1, 64, 256, 10, 64, _lib.F32, 0, 0) == 2 * 10 * 256 * 4
    # tensor-core kernels refuse shapes they cannot take
    assert L.rdb_linear_workspace_bytes(0, 64, 250, 10, 64, _lib.BF16, 1, _lib.IMPL_UMMA) == 0


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
