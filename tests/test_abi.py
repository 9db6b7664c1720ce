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


def test_options_are_validated_and_per_call(built_lib):
    L = _lib.lib()
    # process defaults: a value out of range is refused and nothing changes
    assert L.rdb_set_option(_lib.OPT_RESERVE_SMS, 16) == 0
    assert L.rdb_set_option(_lib.OPT_RESERVE_SMS, _lib.MAX_RESERVE_SMS + 1) == -6
    assert L.rdb_set_option(_lib.OPT_RESERVE_SMS, 0) == 16
    assert L.rdb_set_option(_lib.OPT_FILL_OVERLAP, 3) == -6 and L.rdb_set_option(_lib.OPT_FILL_OVERLAP, 1) == 1
    assert L.rdb_set_option(_lib.OPT_GRADS_BESIDE, 3) == -6 and L.rdb_set_option(_lib.OPT_GRADS_BESIDE, 1) == 1
    # per-call options override the default for that call only, and are validated the same way
    stage_off = _lib.CallOptions(stage_noise=1)
    zg, S = 8192 * 1024 * 2, 16384 * 1024 * 2
    assert L.rdb_linear_workspace_bytes_ex(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0, ctypes.byref(stage_off)) == zg
    assert L.rdb_linear_workspace_bytes(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg + S
    assert L.rdb_linear_stages_noise_ex(8192, 4096, 16384, 1024, _lib.BF16, 0, 0, ctypes.byref(stage_off)) == 0
    bad = _lib.CallOptions(reserve_sms=1000)
    assert L.rdb_linear_stages_noise_ex(8192, 4096, 16384, 1024, _lib.BF16, 0, 0, ctypes.byref(bad)) == -6
    assert L.rdb_linear_fwd_ex(None, None, None, None, 0, 4, 4, 4, 4, 0, 0, 0, 0, 0, ctypes.byref(bad), None, None) == -6
    assert L.rdb_gemm_dense_ex(None, None, None, None, 0, 4, 4, 4, 4, 4, 4, 0, 0, 0, 1, 1, 0, ctypes.byref(bad), None, None) == -6


def test_unaligned_operands_are_caught_on_host(built_lib):
    """The tensor-core kernels address their operands through TMA, which needs 16-byte aligned bases.  With RDB_IMPL_UMMA an
    operand at an odd offset is an alignment error; with RDB_IMPL_AUTO the call goes to the CUDA-core kernels, which then ask
    for their own (larger) workspace.  Both answers come from the host checks: the pointers are never dereferenced."""
    L = _lib.lib()
    T, K, N, R = 64, 128, 256, 64
    ok, odd, ws = 0x7F0000001000, 0x7F0000001000 + 8, 0x7F0000100000
    big = 1 << 30
    args = (ws, big, T, K, N, R, 0, 0, _lib.BF16, _lib.PATH_FACTORED)
    assert L.rdb_linear_fwd(ok, odd, ok, *args, _lib.IMPL_UMMA, None, None) == -4
    assert L.rdb_linear_fwd(odd, ok, ok, *args, _lib.IMPL_UMMA, None, None) == -4
    assert L.rdb_linear_fwd(ok, ok, odd, *args, _lib.IMPL_UMMA, None, None) == -4
    assert L.rdb_linear_bwd(ok, ok, odd, ok, ok, *args, _lib.IMPL_UMMA, None, None) == -4
    assert L.rdb_linear_bwd(odd, None, ok, ok, ok, *args, _lib.IMPL_UMMA, None, None) == -4
    assert "16-byte" in _lib.strerror(-4)
    # AUTO: falls back to the CUDA-core layout (float32 z: T*R*4 bytes), so a workspace that holds only a bf16 z is refused
    umma_ws = L.rdb_linear_workspace_bytes(0, T, K, N, R, _lib.BF16, _lib.PATH_FACTORED, _lib.IMPL_AUTO)
    simt_ws = L.rdb_linear_workspace_bytes(0, T, K, N, R, _lib.BF16, _lib.PATH_FACTORED, _lib.IMPL_SIMT)
    assert umma_ws == T * R * 2 and simt_ws == T * R * 4
    assert L.rdb_linear_fwd(ok, odd, ok, ws, T * R * 2, T, K, N, R, 0, 0, _lib.BF16, _lib.PATH_FACTORED, _lib.IMPL_AUTO, None, None) == -5


def test_association_and_kernel_decision_table(built_lib):
    """rdb_linear_path: FLOP rule for the association, tcgen05 kernels for every bf16 problem with extents in multiples of 8
    -- both associations run on them, so a large-d_c problem that prefers the W path keeps the tensor cores."""
    L = _lib.lib()
    F, W, SIMT, UMMA = _lib.PATH_FACTORED, _lib.PATH_WPATH, _lib.IMPL_SIMT, _lib.IMPL_UMMA
    plan = lambda T, K, N, R, dt, path=0, impl=0: (lambda rc: (rc & 0xFF, rc >> 8) if rc >= 0 else rc)(L.rdb_linear_path(T, K, N, R, dt, path, impl))
    assert plan(8192, 4096, 16384, 1024, _lib.BF16) == (F, UMMA)          # headline layer
    assert plan(4096, 16384, 65536, 2048, _lib.BF16) == (F, UMMA)         # row-sharded layer
    assert plan(8192, 768, 3072, 128, _lib.BF16) == (F, UMMA)             # GPT-2-small MLP
    assert plan(64, 784, 256, 64, _lib.F32) == (F, SIMT) and plan(64, 256, 10, 64, _lib.F32) == (W, SIMT)   # MNIST-shaped
    assert plan(8192, 4096, 4096, 4096, _lib.BF16) == (W, UMMA)           # large d_c: fewer FLOPs through W, still tensor cores
    assert plan(4096, 1024, 1024, 1024, _lib.BF16) == (W, UMMA)
    assert plan(4096, 1024, 1024, 1024, _lib.BF16, F) == (F, UMMA) and plan(4096, 1024, 1024, 1024, _lib.BF16, 0, SIMT) == (W, SIMT)
    assert plan(64, 250, 10, 64, _lib.BF16) == (W, SIMT)                  # extents not in multiples of 8
    assert plan(64, 250, 10, 64, _lib.BF16, 0, UMMA) == -6
    # W-path workspace on the tensor cores: S and W (and dW in backward), bf16
    n, k, r = 4096, 4096, 4096
    assert L.rdb_linear_workspace_bytes(0, 8192, k, n, r, _lib.BF16, 0, 0) == n * r * 2 + n * k * 2
    assert L.rdb_linear_workspace_bytes(1, 8192, k, n, r, _lib.BF16, 0, 0) == n * r * 2 + 2 * n * k * 2


def test_backward_plan_puts_the_two_gradients_side_by_side_only_where_their_tiles_pack(built_lib):
    """rdb_linear_bwd_plan: dX (256 tiles of 16 k-blocks) and dC (32 tiles of 128 k-blocks) of the headline layer share the
    74 CTA pairs 42 : 32; a dX that fills the pairs by itself, or a dC with at most 128 rows, stays in sequence."""
    L = _lib.lib()

    def plan(T, K, N, R, dt=_lib.BF16, opts=None):
        a, b = ctypes.c_int(-1), ctypes.c_int(-1)
        rc = L.rdb_linear_bwd_plan(T, K, N, R, dt, 0, 0, ctypes.byref(opts) if opts is not None else None, ctypes.byref(a), ctypes.byref(b))
        return rc, a.value, b.value

    assert plan(8192, 4096, 16384, 1024) == (1, 42, 32)                    # headline layer
    assert plan(4096, 16384, 65536, 2048) == (0, 0, 0)                     # row-sharded layer on one GPU
    assert plan(8192, 768, 3072, 128) == (0, 0, 0)                         # GPT-2-small MLP: dC has 128 rows
    assert plan(64, 784, 256, 64, _lib.F32) == (0, 0, 0)
    assert plan(8192, 4096, 16384, 1024, opts=_lib.CallOptions(grads_beside=0)) == (0, 0, 0)
    assert plan(8192, 4096, 16384, 1024, opts=_lib.CallOptions(dense_pair=0)) == (0, 0, 0)
    rc, a, b = plan(4096, 16384, 65536, 2048, opts=_lib.CallOptions(grads_beside=2))
    assert rc == 1 and a + b == 74 and a > 0 and b > 0
    rc, a, b = plan(8192, 4096, 16384, 1024, opts=_lib.CallOptions(reserve_sms=20, grads_beside=2))   # 20 SMs left to a collective
    assert rc == 1 and a + b == 64
    assert plan(8192, 4096, 16384, 1024, opts=_lib.CallOptions(grads_beside=7))[0] == -6
    assert L.rdb_linear_bwd_plan(8192, 4096, 16384, 1024, _lib.BF16, 0, 0, None, None, None) == 1


def test_peer_exchange_arguments_are_checked_on_host(built_lib):
    L = _lib.lib()
    ok = 0x7F0000001000
    two = (ctypes.c_void_p * 2)(ok, ok + 4096)
    bad = (ctypes.c_void_p * 2)(ok, ok + 8)                                 # second pointer not 16-byte aligned
    nul = (ctypes.c_void_p * 2)(ok, None)
    assert L.rdb_peer_barrier(None, 0, 2, 1, None, None) == -9
    assert L.rdb_peer_barrier(two, 2, 2, 1, None, None) == -9              # rank out of range
    assert L.rdb_peer_barrier(two, 0, 2, 0, None, None) == -9              # epochs start at 1
    assert L.rdb_peer_barrier(two, 0, 9, 1, None, None) == -9              # more than RDB_MAX_PEERS
    assert L.rdb_peer_barrier(nul, 0, 2, 1, None, None) == -9
    assert L.rdb_peer_copy(bad, 2, 0, ok, 64, 0, None) == -9
    assert L.rdb_peer_copy(two, 2, 8, ok, 64, 0, None) == -4               # offset not a multiple of 16
    assert L.rdb_peer_copy(two, 2, 0, ok, 0, 0, None) == 0                 # nothing to copy
    assert L.rdb_peer_scatter(two, 2, 0, ok + 4, 64, 0, None) == -4
    assert L.rdb_reduce_slots_bf16(ok, ok, 64, 0, 64, None) == -9
    assert L.rdb_reduce_slots_bf16(ok, ok, 64, 2, 0, None) == 0
    # fused product + scatter: destinations, block size and shape are validated before anything is launched
    assert L.rdb_gemm_dense_scatter(two, 2, 0, 500, ok, ok, 1024, 256, 264, 264, 256, 0, None, None, None) == -9   # 500 % 32
    assert L.rdb_gemm_dense_scatter(two, 2, 0, 256, ok, ok, 1024, 256, 264, 264, 256, 0, None, None, None) == -9   # 4 blocks, 2 destinations
    assert L.rdb_gemm_dense_scatter(two, 2, 0, 512, ok, ok, 1024, 72, 264, 264, 72, 0, None, None, None) == -6     # too narrow for the pair kernel
    assert L.rdb_gemm_dense_scatter(two, 2, 0, 512, ok, ok, 1024, 256, 264, 100, 256, 0, None, None, None) == -2   # lda < Kc
    assert "peer" in _lib.strerror(-9)


def test_workspace_sizes(built_lib):
    L = _lib.lib()
    # bf16 factored on tensor cores: z or g, bf16 [T, R], plus S bf16 [N, R] when the noise operand is staged
    zg, S = 8192 * 1024 * 2, 16384 * 1024 * 2
    assert L.rdb_linear_stages_noise(8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == 3          # forward | backward
    assert L.rdb_linear_workspace_bytes(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg + S
    assert L.rdb_linear_workspace_bytes(1, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg + S
    assert L.rdb_set_option(_lib.OPT_STAGE_NOISE, 1) == 0          # regenerate inside the kernel: nothing of S in memory
    try:
        assert L.rdb_linear_stages_noise(8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == 0
        assert L.rdb_linear_workspace_bytes(0, 8192, 4096, 16384, 1024, _lib.BF16, 0, 0) == zg
    finally:
        assert L.rdb_set_option(_lib.OPT_STAGE_NOISE, 0) == 1
    # few tokens: the forward's one 512-token tile regenerates S once anyway, the backward still hashes it once on every SM
    # (its g = dY S has four work units to do it in otherwise); a noise block above 1 GiB is never staged
    assert L.rdb_linear_stages_noise(512, 4096, 16384, 1024, _lib.BF16, 0, 0) == 2
    assert L.rdb_linear_workspace_bytes_ex(0, 512, 4096, 16384, 1024, _lib.BF16, 0, 0, None) == \
        L.rdb_linear_workspace_bytes_ex(0, 512, 4096, 16384, 1024, _lib.BF16, 0, 0, ctypes.byref(_lib.CallOptions(stage_noise=1)))
    assert L.rdb_linear_workspace_bytes(1, 512, 4096, 16384, 1024, _lib.BF16, 0, 0) >= 512 * 1024 * 2 + S
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
