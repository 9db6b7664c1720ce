"""rdb_gemv_fwd_static: the batch-1 forward for callers that cannot allocate device memory (a serving
loop whose memory is fully handed out at start-up, a runtime that forbids allocation on its request
path).  Its scratch is a fixed array inside the library, so the test calls it through the C ABI with
inputs and outputs only, twice in a row with different data, and compares with rdb_gemv_fwd, which takes
a caller-provided workspace.  Collected last on purpose (file name), so a failure here cannot hide other
results when the run stops at the first failure."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(L, x, C, N, seed, row0):
    R, K = C.shape
    stream = torch.cuda.current_stream().cuda_stream
    y_ws = torch.empty(N, device="cuda")
    ws = torch.empty(max(R, 1), device="cuda")
    assert L.rdb_gemv_fwd(y_ws.data_ptr(), x.data_ptr(), C.data_ptr(), ws.data_ptr(), K, N, R, row0, seed, stream) == 0
    y_st = torch.empty(N, device="cuda")
    assert L.rdb_gemv_fwd_static(y_st.data_ptr(), x.data_ptr(), C.data_ptr(), K, N, R, row0, seed, stream) == 0
    torch.cuda.synchronize()
    return y_ws, y_st


def test_static_scratch_forward_matches_workspace_forward():
    from randumb_b200 import _lib
    from oracle import oracle as O
    assert torch.cuda.is_available()
    L = _lib.lib()
    g = torch.Generator().manual_seed(77)
    # first call: the headline batch-1 shape; second call right after it: different sizes and data, with a
    # smaller R so that entries of the shared array beyond it still hold the first call's values
    for (K, N, R, seed, row0) in [(4096, 4096, 256, 42, 0), (1000, 777, 96, 5, 31)]:
        x = torch.randn(K, generator=g)
        C = torch.randn(R, K, generator=g) * 0.02
        y_ws, y_st = _call_pair(L, x.cuda(), C.cuda(), N, seed, row0)
        # same kernels, same order of operations: the tolerance of the float32 tests (1e-5) is met exactly
        assert torch.equal(y_st, y_ws)
        torch.testing.assert_close(y_st, y_ws, rtol=1e-5, atol=1e-5)
        # ... and both are the layer: float64 oracle on the same float32 inputs
        y_ref, _, _ = O.linear_reference(x[None, :], C, seed, N, row0, dtype=torch.float64)
        assert O.close(y_st[None, :], y_ref, 1e-5), f"rel {O.rel_fro(y_st[None, :], y_ref):.2e}"


def test_static_scratch_call_allocates_nothing_and_takes_the_maximum_r():
    """The point of the entry point: no device memory changes hands during the call.  Free memory as the driver reports it
    is the same before and after a call (inputs and outputs allocated beforehand), also at the largest coefficient dimension
    the built-in array holds, where the result still equals the workspace variant's."""
    from randumb_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(78)
    K, N, R, seed = 64, 40, 16384, 9                     # R == RDB_GEMV_STATIC_MAX_R
    x = torch.randn(K, generator=g).cuda()
    C = (torch.randn(R, K, generator=g) * 0.02).cuda()
    y_ws, y_st = _call_pair(L, x, C, N, seed, 0)         # also the first call on this device (address look-up) if run alone
    assert torch.equal(y_st, y_ws)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    reserved_before = torch.cuda.memory_reserved()
    assert L.rdb_gemv_fwd_static(y_st.data_ptr(), x.data_ptr(), C.data_ptr(), K, N, R, 0, seed, stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before
    assert torch.equal(y_st, y_ws)


def test_static_scratch_rejects_oversized_r():
    from randumb_b200 import _lib
    L = _lib.lib()
    y = torch.empty(8, device="cuda")
    x = torch.empty(8, device="cuda")
    C = torch.empty(8, device="cuda")
    rc = L.rdb_gemv_fwd_static(y.data_ptr(), x.data_ptr(), C.data_ptr(), 8, 8, 16384 + 1, 0, 0, None)
    assert rc == -8 and "exceeds" in _lib.strerror(rc)
