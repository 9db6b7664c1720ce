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
    assert torch.cuda.is_available()
    L = _lib.lib()
    g = torch.Generator().manual_seed(77)
    # first call: the headline batch-1 shape; second call right after it: different sizes and data, with a
    # smaller R so that entries of the shared array beyond it still hold the first call's values
    for (K, N, R, seed, row0) in [(4096, 4096, 256, 42, 0), (1000, 777, 96, 5, 31)]:
        x = torch.randn(K, generator=g).cuda()
        C = (torch.randn(R, K, generator=g) * 0.02).cuda()
        y_ws, y_st = _call_pair(L, x, C, N, seed, row0)
        # same kernels, same order of operations: the tolerance of the float32 tests (1e-5) is met exactly
        assert torch.equal(y_st, y_ws)
        torch.testing.assert_close(y_st, y_ws, rtol=1e-5, atol=1e-5)


def test_static_scratch_rejects_oversized_r():
    from randumb_b200 import _lib
    L = _lib.lib()
    y = torch.empty(8, device="cuda")
    x = torch.empty(8, device="cuda")
    C = torch.empty(8, device="cuda")
    rc = L.rdb_gemv_fwd_static(y.data_ptr(), x.data_ptr(), C.data_ptr(), 8, 8, 16384 + 1, 0, 0, None)
    assert rc == -8 and "exceeds" in _lib.strerror(rc)
