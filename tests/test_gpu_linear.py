"""Parity of the layer's CUDA kernels (through the C ABI) with the CPU oracle.

Tolerances: float32 -- rel-Frobenius <= 1e-5 and allclose(rtol=1e-5, atol=1e-5*rms) against a float64
oracle on the same float32 inputs; bf16 -- the same two tests with 2e-2 against a float32 oracle on the
bf16-rounded inputs and the unrounded float32 noise.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def K():
    from randumb_b200 import kernels
    assert torch.cuda.is_available()
    return kernels


def _inputs(T, Kin, N, R, dtype, seed=0, coef_scale=None):
    g = torch.Generator().manual_seed(1000 + seed)
    x = torch.randn(T, Kin, generator=g)
    scale = coef_scale if coef_scale is not None else (3.0 / (R * Kin)) ** 0.5
    C = torch.randn(R, Kin, generator=g) * scale
    dy = torch.randn(T, N, generator=g)
    return x.to(dtype), C.to(dtype), dy.to(dtype)


def _check(K, T, Kin, N, R, dtype, seed, row0, path, impl, tol):
    x, C, dy = _inputs(T, Kin, N, R, dtype, seed)
    odt = torch.float64 if dtype == torch.float32 else torch.float32
    y, dx, dc = O.linear_reference(x, C, seed, N, row0, dy, dtype=odt)
    yg = K.linear_fwd(x.cuda(), C.cuda(), seed, N, row0, path=path, impl=impl)
    dxg, dcg = K.linear_bwd(dy.cuda(), x.cuda(), C.cuda(), seed, row0, path=path, impl=impl)
    torch.cuda.synchronize()
    K.check_status()
    assert yg.dtype == dtype and dxg.dtype == dtype and dcg.dtype == dtype
    assert O.close(yg, y, tol), f"y rel {O.rel_fro(yg, y):.3e}"
    assert O.close(dxg, dx, tol), f"dx rel {O.rel_fro(dxg, dx):.3e}"
    assert O.close(dcg, dc, tol), f"dc rel {O.rel_fro(dcg, dc):.3e}"


# ---- float32 (CUDA cores) -------------------------------------------------------------------------
@pytest.mark.parametrize("T,Kin,N,R,seed,row0,path", [
    (64, 784, 256, 64, 0, 0, 0),      # MNIST-shaped layer 1 (factored)
    (64, 256, 10, 64, 1, 0, 0),       # MNIST-shaped head: the W path is cheaper and is chosen
    (64, 256, 10, 64, 1, 0, 1),       # same, forced factored
    (33, 70, 45, 9, 5, 7, 2), (33, 70, 45, 9, 5, 7, 1),   # ragged everything, both associations
    (5, 8, 300, 16, 3, 0, 0), (1, 1, 1, 1, 2, 0, 0), (2, 3, 5, 1, 2, 4, 2)])
def test_f32_layer(K, T, Kin, N, R, seed, row0, path):
    _check(K, T, Kin, N, R, torch.float32, seed, row0, path, K.IMPL_AUTO, F32_TOL)


@pytest.mark.parametrize("Kin,N,R,seed", [(4096, 4096, 256, 42), (100, 37, 5, 1), (4098, 513, 33, 9)])
def test_f32_gemv(K, Kin, N, R, seed):
    """Batch-1: the matrix-vector kernels (also what rdb_linear_* dispatches to for T == 1)."""
    x, C, dy = _inputs(1, Kin, N, R, torch.float32, seed)
    y, dx, dc = O.linear_reference(x, C, seed, N, 0, dy)
    yg = K.gemv_fwd(x.cuda().view(-1), C.cuda(), seed, N)
    dxg, dcg = K.gemv_bwd(dy.cuda().view(-1), x.cuda().view(-1), C.cuda(), seed)
    assert O.close(yg.view(1, -1), y, F32_TOL) and O.close(dxg.view(1, -1), dx, F32_TOL) and O.close(dcg, dc, F32_TOL)
    y2 = K.linear_fwd(x.cuda(), C.cuda(), seed, N)
    dx2, dc2 = K.linear_bwd(dy.cuda(), x.cuda(), C.cuda(), seed)
    assert torch.equal(y2.view(-1), yg) and torch.equal(dx2.view(-1), dxg) and torch.equal(dc2, dcg)
    dx3, none = K.gemv_bwd(dy.cuda().view(-1), x.cuda().view(-1), C.cuda(), seed, need_dc=False)
    assert none is None and torch.equal(dx3, dxg)


@pytest.mark.parametrize("Kin,N,R,seed", [(4096, 4096, 256, 42), (4098, 513, 33, 9), (640, 4099, 1024, 3)])
def test_gemv_single_launch_equals_one_kernel_per_step(K, Kin, N, R, seed):
    """RDB_OPT_GEMV_FUSED: forward and backward as one cooperative launch each (grid-wide barriers between the steps) against
    one kernel per step chained with programmatic dependent launch -- the same device functions in the same order, so the
    same bits; and both replay from a CUDA graph."""
    from randumb_b200 import _lib
    x, C, dy = _inputs(1, Kin, N, R, torch.float32, seed)
    xg, Cg, dyg = x.cuda().view(-1), C.cuda(), dy.cuda().view(-1)
    res = {}
    for fused in (1, 0):
        prev = K.set_option(_lib.OPT_GEMV_FUSED, fused)
        try:
            y = K.gemv_fwd(xg, Cg, seed, N)
            dx, dc = K.gemv_bwd(dyg, xg, Cg, seed)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y_g = K.gemv_fwd(xg, Cg, seed, N)
                dx_g, dc_g = K.gemv_bwd(dyg, xg, Cg, seed)
            y_g.zero_(); dx_g.zero_(); dc_g.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y_g, y) and torch.equal(dx_g, dx) and torch.equal(dc_g, dc)
            res[fused] = (y, dx, dc)
        finally:
            K.set_option(_lib.OPT_GEMV_FUSED, prev)
    for a, b in zip(res[1], res[0]):
        assert torch.equal(a, b)
    y_ref, dx_ref, dc_ref = O.linear_reference(x, C, seed, N, 0, dy)
    assert O.close(res[1][0].view(1, -1), y_ref, F32_TOL) and O.close(res[1][1].view(1, -1), dx_ref, F32_TOL) and O.close(res[1][2], dc_ref, F32_TOL)


# ---- bf16 on tensor cores --------------------------------------------------------------------------
@pytest.mark.parametrize("T,Kin,N,R,seed,row0", [
    (512, 256, 384, 128, 42, 0),
    (1000, 264, 520, 72, 7, 1000),     # nothing a multiple of the tile
    (8, 8, 8, 8, 3, 0),                # smallest shape the tensor-core path takes
    (130, 4096, 136, 1024, 5, 65530),  # long contractions, noise rows around 2^16
    (1024, 768, 3072, 128, 13, 0),     # GPT-2-small MLP up-projection shape (tokens reduced)
])
def test_bf16_layer_tensor_cores(K, T, Kin, N, R, seed, row0):
    _check(K, T, Kin, N, R, torch.bfloat16, seed, row0, K.PATH_FACTORED, K.IMPL_UMMA, BF16_TOL)


@pytest.mark.parametrize("tile", [1, 2, 3, 4, 5, 6, 7, 8, 9])
def test_bf16_layer_every_work_unit_shape(K, tile):
    """Every (cluster size, sub-tiles, generated rows) variant of the generated-operand kernel, on a shape
    with ragged tiles and an odd number of token tiles per cluster."""
    prev = K.set_option(1, tile)
    prev_stage = K.set_option(3, 1)          # regenerate S inside the kernel whatever the token count
    try:
        _check(K, 1500, 264, 520, 72, torch.bfloat16, 7, 10, K.PATH_FACTORED, K.IMPL_UMMA, BF16_TOL)
        _check(K, 100, 64, 136, 200, torch.bfloat16, 8, 0, K.PATH_FACTORED, K.IMPL_UMMA, BF16_TOL)
    finally:
        K.set_option(1, prev)
        K.set_option(3, prev_stage)


@pytest.mark.parametrize("T,Kin,N,R,seed,row0", [
    (1500, 264, 520, 72, 7, 10),        # ragged tiles
    (2048, 512, 1024, 256, 3, 65000),   # noise rows across 2^16
    (8, 8, 8, 8, 3, 0), (100, 64, 136, 200, 8, 0)])
def test_staged_noise_equals_regenerated_noise(K, T, Kin, N, R, seed, row0):
    """S written once per call and read back by the plain product gives the bits of the kernels that regenerate S per
    tile (same bf16 noise values, same accumulation order), and both agree with the oracle."""
    x, C, dy = _inputs(T, Kin, N, R, torch.bfloat16, seed)
    xg, Cg, dyg = x.cuda(), C.cuda(), dy.cuda()
    outs = {}
    for mode in (1, 2):
        prev = K.set_option(3, mode)
        try:
            assert K.linear_stages_noise(T, Kin, N, R, torch.bfloat16, K.PATH_FACTORED, K.IMPL_UMMA) == (mode == 2)
            y = K.linear_fwd(xg, Cg, seed, N, row0, path=K.PATH_FACTORED, impl=K.IMPL_UMMA)
            dx, dc = K.linear_bwd(dyg, xg, Cg, seed, row0, path=K.PATH_FACTORED, impl=K.IMPL_UMMA)
            outs[mode] = (y, dx, dc)
        finally:
            K.set_option(3, prev)
    K.check_status()
    assert torch.equal(outs[1][0], outs[2][0])                     # y: same bits
    for a, b in zip(outs[1][1:], outs[2][1:]):
        # dX and dC follow g, which the staged path may compute split-K (float32 partial sums over slices of the
        # contraction): equal up to the rounding of that re-association
        assert torch.equal(a, b) or O.close(a, b, 1e-2)
    y, dx, dc = O.linear_reference(x, C, seed, N, row0, dy, dtype=torch.float32)
    assert O.close(outs[2][0], y, BF16_TOL) and O.close(outs[2][1], dx, BF16_TOL) and O.close(outs[2][2], dc, BF16_TOL)
    # the building block used by the row-sharded layer follows the same rule
    z = torch.randn(T, R, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    prev = K.set_option(3, 2)
    try:
        for a, b in ((K.noise_product(z, N, seed, False, row0), K.gemm_noise(z, N, seed, False, row0)),
                     (K.noise_product(dyg, R, seed, True, row0), K.gemm_noise(dyg, R, seed, True, row0))):
            assert torch.equal(a, b) or O.close(a, b, 1e-2)       # equal bits unless the plain product ran split-K
    finally:
        K.set_option(3, prev)


@pytest.mark.parametrize("T,Kin,N,R,seed,row0,path", [(64, 80, 96, 16, 0, 0, 0), (33, 70, 45, 9, 5, 7, 2), (33, 70, 45, 9, 5, 7, 1)])
def test_bf16_layer_any_shape_path(K, T, Kin, N, R, seed, row0, path):
    """Shapes the tensor-core kernels refuse (odd extents) run on the CUDA-core kernels."""
    _check(K, T, Kin, N, R, torch.bfloat16, seed, row0, path, K.IMPL_AUTO, BF16_TOL)


def test_umma_refuses_unaligned_shapes(K):
    x, C, _ = _inputs(33, 70, 45, 9, torch.bfloat16)
    with pytest.raises(RuntimeError, match="not supported"):
        K.linear_fwd(x.cuda(), C.cuda(), 0, 45, impl=K.IMPL_UMMA)


# ---- building blocks ----------------------------------------------------------------------------------
def test_generated_operand_is_the_noise_matrix(K):
    """With A = I the product returns the generated tile itself: element-exact layout check."""
    A = torch.eye(128, 64).bfloat16().cuda()
    d = K.gemm_noise(A, 256, 11, False, 5, impl=K.IMPL_UMMA).cpu()
    G = O.noise_bf16(256, 64, 11, row0=5)
    assert torch.equal(d[:64], G.t().contiguous()) and float(d[64:].abs().max()) == 0.0
    dt = K.gemm_noise(A, 256, 11, True, 5, impl=K.IMPL_UMMA).cpu()        # G[n, k] = S[row0 + k, n]
    Gt = O.noise_bf16(64, 256, 11, row0=5)
    assert torch.equal(dt[:64], Gt)


@pytest.mark.parametrize("akm,bkm", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("out", [torch.bfloat16, torch.float32])
def test_dense_products_all_operand_layouts(K, akm, bkm, out):
    g = torch.Generator().manual_seed(4)
    M, N, Kc = 1000, 520, 328
    A = torch.randn(M, Kc, generator=g).bfloat16()
    B = torch.randn(N, Kc, generator=g).bfloat16()
    ref = A.float() @ B.float().t()
    a = (A if akm else A.t().contiguous()).cuda()
    b = (B if bkm else B.t().contiguous()).cuda()
    d = K.gemm_dense(a, b, akm, bkm, out_dtype=out, impl=K.IMPL_UMMA)
    K.check_status()
    assert O.close(d, ref, 1e-2 if out == torch.bfloat16 else 1e-5)
    d2 = K.gemm_dense(a, b, akm, bkm, out_dtype=out, impl=K.IMPL_SIMT)
    assert O.close(d2, ref, 1e-2 if out == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("M,N,Kc,out", [(1024, 520, 328, torch.float32), (256, 72, 200, torch.float32), (1000, 72, 200, torch.bfloat16),
                                         (128, 128, 4096, torch.bfloat16)])
def test_dense_products_whole_row_tiles_and_narrow_outputs(K, M, N, Kc, out):
    """float32 outputs with whole 128-row tiles (TMA-stored), outputs of at most 128 columns (128-column tiles)."""
    g = torch.Generator().manual_seed(6)
    A = torch.randn(M, Kc, generator=g).bfloat16()
    B = torch.randn(N, Kc, generator=g).bfloat16()
    ref = A.float() @ B.float().t()
    for akm, bkm in ((True, True), (False, False)):
        a = (A if akm else A.t().contiguous()).cuda()
        b = (B if bkm else B.t().contiguous()).cuda()
        d = K.gemm_dense(a, b, akm, bkm, out_dtype=out, impl=K.IMPL_UMMA)
        K.check_status()
        assert O.close(d, ref, 1e-2 if out == torch.bfloat16 else 1e-5)


def test_dense_products_random_shapes(K):
    """Seeded random extents (multiples of 8, ragged against every tile size), operand layouts and kernel choices."""
    import random
    rnd = random.Random(1234)
    g = torch.Generator().manual_seed(9)
    for case in range(16):
        M = 8 * rnd.randint(1, 160)
        N = 8 * rnd.randint(1, 160)
        Kc = 8 * rnd.randint(1, 300)
        akm, bkm = rnd.random() < 0.5, rnd.random() < 0.5
        pair = rnd.choice((0, 1, 2))
        A = torch.randn(M, Kc, generator=g).bfloat16()
        B = torch.randn(N, Kc, generator=g).bfloat16()
        a = (A if akm else A.t().contiguous()).cuda()
        b = (B if bkm else B.t().contiguous()).cuda()
        prev = K.set_option(2, pair)
        try:
            d = K.gemm_dense(a, b, akm, bkm, impl=K.IMPL_UMMA)
        finally:
            K.set_option(2, prev)
        K.check_status()
        assert O.close(d, A.float() @ B.float().t(), 1e-2), (case, M, N, Kc, akm, bkm, pair)


@pytest.mark.parametrize("M,N,Kc", [(512, 2048, 16384), (128, 768, 8192), (72, 264, 1504), (256, 128, 3072),
                                    (1024, 2048, 16384), (2048, 2048, 16384), (1056, 520, 16392)])
def test_dense_products_split_k(K, M, N, Kc):
    """Few output tiles and a long contraction: slices of the contraction as independent work items, float32 partial
    products, ordered sum -- within bf16 rounding of the unsplit kernel, identical from run to run.  The last three shapes run
    on CTA pairs (512 x 256 tiles, ragged in the last one), the others on single CTAs."""
    from randumb_b200 import _lib
    assert _lib.lib().rdb_gemm_dense_workspace_bytes(M, N, Kc) > 0
    g = torch.Generator().manual_seed(8)
    A = (torch.randn(M, Kc, generator=g) * 0.1).bfloat16()
    B = torch.randn(N, Kc, generator=g).bfloat16()
    ref = A.float() @ B.float().t()
    for akm, bkm in ((True, True), (False, False), (True, False)):
        a = (A if akm else A.t().contiguous()).cuda()
        b = (B if bkm else B.t().contiguous()).cuda()
        d1 = K.gemm_dense(a, b, akm, bkm)
        d2 = K.gemm_dense(a, b, akm, bkm)
        K.check_status()
        assert torch.equal(d1, d2)
        assert O.close(d1, ref, 1e-2)


@pytest.mark.parametrize("akm,bkm", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("M,N,Kc", [(1000, 520, 328), (2048, 264, 72), (136, 136, 8), (304, 1032, 4096)])
def test_dense_products_on_cta_pairs(K, akm, bkm, M, N, Kc):
    """The cta_group::2 kernel (512 x 256 pair tiles) against the single-CTA kernel."""
    g = torch.Generator().manual_seed(5)
    A = torch.randn(M, Kc, generator=g).bfloat16()
    B = torch.randn(N, Kc, generator=g).bfloat16()
    a = (A if akm else A.t().contiguous()).cuda()
    b = (B if bkm else B.t().contiguous()).cuda()
    outs = []
    for pair in (0, 2):                       # never / always the pair kernel
        prev = K.set_option(2, pair)
        try:
            outs.append(K.gemm_dense(a, b, akm, bkm, impl=K.IMPL_UMMA))
        finally:
            K.set_option(2, prev)
    K.check_status()
    # same bits, unless the single-CTA side ran split-K (few tiles, long contraction: 304 x 1032 x 4096)
    assert torch.equal(outs[0], outs[1]) or O.close(outs[0], outs[1], 1e-2)
    ref = A.float() @ B.float().t()
    assert O.close(outs[0], ref, 1e-2) and O.close(outs[1], ref, 1e-2)


# ---- edge cases ----------------------------------------------------------------------------------------
def test_empty_and_degenerate(K):
    dev = "cuda"
    C = torch.randn(4, 8, device=dev)
    assert K.linear_fwd(torch.empty(0, 8, device=dev), C, 0, 16).shape == (0, 16)
    assert K.linear_fwd(torch.randn(3, 8, device=dev), C, 0, 0).shape == (3, 0)
    y = K.linear_fwd(torch.randn(3, 8, device=dev), torch.empty(0, 8, device=dev), 0, 5)   # d_c == 0 -> W == 0
    assert float(y.abs().max()) == 0.0
    dx, dc = K.linear_bwd(torch.empty(0, 16, device=dev), torch.empty(0, 8, device=dev), C, 0)
    assert dx.shape == (0, 8) and dc.shape == (4, 8) and float(dc.abs().max()) == 0.0
    with pytest.raises(RuntimeError):
        K.linear_fwd(torch.randn(3, 7, device=dev), C, 0, 16)                                  # K mismatch
    with pytest.raises(RuntimeError):
        K.linear_fwd(torch.randn(3, 8, device=dev).double(), C.double(), 0, 16)                # dtype


def test_row_sharded_outputs_equal_the_unsharded_layer(K):
    """A rank that owns rows [row0, row0+n) computes exactly the same numbers as the full layer."""
    x, C, dy = _inputs(256, 128, 512, 64, torch.bfloat16, 3)
    xg, Cg, dyg = x.cuda(), C.cuda(), dy.cuda()
    y = K.linear_fwd(xg, Cg, 7, 512)
    parts = [K.linear_fwd(xg, Cg, 7, 128, row0=128 * r) for r in range(4)]
    assert torch.equal(torch.cat(parts, dim=1), y)
    dx, dc = K.linear_bwd(dyg, xg, Cg, 7)
    dxs = [K.linear_bwd(dyg[:, 128 * r:128 * (r + 1)].contiguous(), xg, Cg, 7, row0=128 * r) for r in range(4)]
    assert O.close(sum(p[0].float() for p in dxs), dx.float(), BF16_TOL)
    assert O.close(sum(p[1].float() for p in dxs), dc.float(), BF16_TOL)


def test_run_to_run_reproducible(K):
    x, C, dy = _inputs(700, 264, 520, 72, torch.bfloat16, 9)
    a = K.linear_fwd(x.cuda(), C.cuda(), 1, 520)
    b = K.linear_fwd(x.cuda(), C.cuda(), 1, 520)
    assert torch.equal(a, b)
    d1 = K.linear_bwd(dy.cuda(), x.cuda(), C.cuda(), 1)
    d2 = K.linear_bwd(dy.cuda(), x.cuda(), C.cuda(), 1)
    assert torch.equal(d1[0], d2[0]) and torch.equal(d1[1], d2[1])


@pytest.mark.parametrize("T,Kin,N,R", [(2048, 264, 520, 72), (300, 64, 136, 200)])
def test_partial_backward_and_graph_replay(K, T, Kin, N, R):
    """Asking for only dX or only dC gives the same tensors as asking for both; a forward + backward captured into a
    CUDA graph (no allocation, no synchronisation inside the entry points) replays to the eager results."""
    x, C, dy = _inputs(T, Kin, N, R, torch.bfloat16, 4)
    xg, Cg, dyg = x.cuda(), C.cuda(), dy.cuda()
    y = K.linear_fwd(xg, Cg, 3, N, 16)
    dx, dc = K.linear_bwd(dyg, xg, Cg, 3, 16)
    dx_only, none1 = K.linear_bwd(dyg, xg, Cg, 3, 16, need_dc=False)
    none2, dc_only = K.linear_bwd(dyg, xg, Cg, 3, 16, need_dx=False)
    assert none1 is None and none2 is None and torch.equal(dx_only, dx) and torch.equal(dc_only, dc)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_g = K.linear_fwd(xg, Cg, 3, N, 16)
        dx_g, dc_g = K.linear_bwd(dyg, xg, Cg, 3, 16)
    for _ in range(2):
        y_g.zero_(); dx_g.zero_(); dc_g.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y_g, y) and torch.equal(dx_g, dx) and torch.equal(dc_g, dc)
    K.check_status()


def test_noise_fill_beside_the_z_product_gives_the_same_bits(K):
    """RDB_OPT_FILL_OVERLAP: the staged noise operand hashed on the library's own stream beside z = x C^T (forced here; by
    default only large fills take that route) -- same result bit for bit, eagerly and replayed from a CUDA graph."""
    from randumb_b200 import _lib
    T, Kin, N, R = 2048, 264, 520, 72
    x, C, _ = _inputs(T, Kin, N, R, torch.bfloat16, 6)
    xg, Cg = x.cuda(), C.cuda()
    y_plain = K.linear_fwd(xg, Cg, 9, N, 8, options=_lib.CallOptions(fill_overlap=0))
    beside = _lib.CallOptions(fill_overlap=2)
    y_side = K.linear_fwd(xg, Cg, 9, N, 8, options=beside)          # also creates the stream and events, outside any capture
    torch.cuda.synchronize()
    assert torch.equal(y_side, y_plain)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_g = K.linear_fwd(xg, Cg, 9, N, 8, options=beside)
    for _ in range(2):
        y_g.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y_g, y_plain)
    K.check_status()


def test_input_and_coefficient_gradients_side_by_side_give_the_same_bits(K):
    """RDB_OPT_GRADS_BESIDE: dX on the library's own stream on some of the CTA pairs while dC runs on the caller's stream on the
    others -- the same bits as the two CTA-pair products one after the other, eagerly and replayed from a CUDA graph, with a
    ragged shape (forced) and with a shape the automatic rule itself sends that way."""
    from randumb_b200 import _lib
    for (T, Kin, N, R, beside) in ((1544, 776, 520, 264, _lib.CallOptions(grads_beside=2, dense_pair=2)),
                                   (4096, 4096, 1024, 1024, None)):
        g = torch.Generator().manual_seed(T)
        dy = (torch.randn(T, N, generator=g) * 0.1).bfloat16().cuda()
        x = torch.randn(T, Kin, generator=g).bfloat16().cuda()
        C = (torch.randn(R, Kin, generator=g) * 0.05).bfloat16().cuda()
        dx0, dc0 = K.linear_bwd(dy, x, C, 5, 16, options=_lib.CallOptions(grads_beside=0, dense_pair=2))
        dx1, dc1 = K.linear_bwd(dy, x, C, 5, 16, options=beside)      # also creates the stream and events, outside any capture
        torch.cuda.synchronize()
        assert torch.equal(dx1, dx0) and torch.equal(dc1, dc0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dx_g, dc_g = K.linear_bwd(dy, x, C, 5, 16, options=beside)
        for _ in range(2):
            dx_g.zero_()
            dc_g.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(dx_g, dx0) and torch.equal(dc_g, dc0)
        if T < 2048:
            _, dx_ref, dc_ref = O.linear_reference(x.cpu(), C.cpu(), 5, N, 16, dy.cpu(), dtype=torch.float32)
            assert O.close(dx1, dx_ref, BF16_TOL) and O.close(dc1, dc_ref, BF16_TOL)
    K.check_status()


def test_per_call_options_change_the_launch_not_the_result(K):
    """rdb_call_options: leaving SMs to a collective, or forcing one kernel family, for one call -- same bits as the default
    launch, and the process defaults are untouched afterwards."""
    from randumb_b200 import _lib
    g = torch.Generator().manual_seed(12)
    A = torch.randn(4096, 1024, generator=g).bfloat16().cuda()
    B = torch.randn(2048, 1024, generator=g).bfloat16().cuda()        # 256 single-CTA tiles / 64 pair tiles: no split-K
    ref = A.float() @ B.float().t()
    for family in (0, 2):
        base = K.gemm_dense(A, B, options=_lib.CallOptions(dense_pair=family))
        assert O.close(base, ref, BF16_TOL)
        for rs in (20, 32, 64):      # fewer CTAs walk the same tiles
            assert torch.equal(K.gemm_dense(A, B, options=_lib.CallOptions(reserve_sms=rs, dense_pair=family)), base)
    with pytest.raises(RuntimeError, match="options"):
        K.gemm_dense(A, B, options=_lib.CallOptions(reserve_sms=65))
    L = _lib.lib()
    assert L.rdb_set_option(_lib.OPT_RESERVE_SMS, 0) == 0 and L.rdb_set_option(_lib.OPT_DENSE_PAIR, 1) == 1
    K.check_status()


# ---- full benchmark sizes ------------------------------------------------------------------------------------------
def test_full_size_properties(K):
    """8192 x 4096 -> 16384, d_c = 1024 (the headline configuration): size-independent properties."""
    T, Kin, N, R, seed = 8192, 4096, 16384, 1024, 42
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(T, Kin, device="cuda", generator=g).bfloat16()
    C = (torch.randn(R, Kin, device="cuda", generator=g) * (3 * 0.02 ** 2 / R) ** 0.5).bfloat16()
    dy = torch.randn(T, N, device="cuda", generator=g).bfloat16()
    y = K.linear_fwd(x, C, seed, N)
    dx, dc = K.linear_bwd(dy, x, C, seed)
    torch.cuda.synchronize()
    K.check_status()
    # (1) a slab of output rows equals the same slab computed as its own (small) problem, against the oracle
    rows = slice(4096, 4096 + 24)
    y_ref, _, _ = O.linear_reference(x[:64].cpu(), C.cpu(), seed, 24, row0=4096, dtype=torch.float32)
    assert O.close(y[:64, rows], y_ref, BF16_TOL)
    # (2) <dy, y> == <dx, x> == <dc, C>  (adjoint identity of a linear map, up to bf16 rounding)
    ip_y = float((dy.float() * y.float()).sum())
    ip_x = float((dx.float() * x.float()).sum())
    ip_c = float((dc.float() * C.float()).sum())
    scale = float(dy.float().norm() * y.float().norm())
    assert abs(ip_y - ip_x) / scale < 2e-3 and abs(ip_y - ip_c) / scale < 2e-3
    # (3) token shards reproduce the full result exactly (tiles do not interact across tokens)
    y_half = K.linear_fwd(x[:4096].contiguous(), C, seed, N)
    assert torch.equal(y_half, y[:4096])


def _close_big(got, want, tol):
    """The two tests of O.close on tensors too large to hold several float64 copies of: rel-Frobenius <= tol and
    |a - b| <= tol * |b| + tol * rms(b) everywhere, evaluated in row chunks in float32 with float64 sums."""
    want = want.detach()
    got = got.detach().cpu()
    assert got.shape == want.shape
    num = den = 0.0
    for lo in range(0, want.shape[0], 1024):
        b = want[lo:lo + 1024].double()
        num += float(((got[lo:lo + 1024].double() - b) ** 2).sum())
        den += float((b ** 2).sum())
    rms = (den / want.numel()) ** 0.5
    worst = 0.0
    for lo in range(0, want.shape[0], 1024):
        b = want[lo:lo + 1024].float()
        excess = (got[lo:lo + 1024].float() - b).abs() - (tol * b.abs() + tol * rms)
        worst = max(worst, float(excess.max()))
    rel = (num / max(den, 1e-300)) ** 0.5
    return rel <= tol and worst <= 0.0, rel, worst


def test_headline_size_elementwise_against_the_oracle(K):
    """The headline configuration at full size (x[8192 x 4096] bf16, W[16384 x 4096], d_c = 1024, seed 42): every element of
    y, dX and dC against the float32 oracle on the same bf16-rounded inputs (both 2e-2 tests)."""
    T, Kin, N, R, seed = 8192, 4096, 16384, 1024, 42
    g = torch.Generator().manual_seed(1003)
    x = torch.randn(T, Kin, generator=g).bfloat16()
    C = (torch.randn(R, Kin, generator=g) * (3 * 0.02 ** 2 / R) ** 0.5).bfloat16()
    dy = torch.randn(T, N, generator=g).bfloat16()
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    S = torch.from_numpy(O.c_noise_f32(N, R, seed))
    W = S @ C.float()                                            # [N, K]
    xg, Cg, dyg = x.cuda(), C.cuda(), dy.cuda()
    y = K.linear_fwd(xg, Cg, seed, N)
    dx, dc = K.linear_bwd(dyg, xg, Cg, seed)
    torch.cuda.synchronize()
    K.check_status()
    ok, rel, worst = _close_big(y, x.float() @ W.t(), BF16_TOL)
    assert ok, f"y rel {rel:.3e} worst excess {worst:.3e}"
    ok, rel, worst = _close_big(dx, dy.float() @ W, BF16_TOL)
    assert ok, f"dx rel {rel:.3e} worst excess {worst:.3e}"
    dW = dy.float().t() @ x.float()                              # [N, K]
    ok, rel, worst = _close_big(dc, S.t() @ dW, BF16_TOL)
    assert ok, f"dc rel {rel:.3e} worst excess {worst:.3e}"


@pytest.mark.parametrize("stage", [2, 1])
def test_one_shard_of_the_row_sharded_layer_against_the_oracle(K, stage):
    """One rank's part of the 65536 x 16384 virtual layer split over 8 ranks (x[4096 x 16384] bf16, d_c = 2048, seed 7):
    rows [57344, 65536).  y, and this rank's contributions to dX and dC, element by element against the float32 oracle;
    once with S hashed into the workspace (2) and once regenerated inside the product kernels (1)."""
    from randumb_b200 import _lib
    T, Kin, N, R, seed, n_loc, row0 = 4096, 16384, 65536, 2048, 7, 8192, 57344
    g = torch.Generator().manual_seed(1005)
    x = torch.randn(T, Kin, generator=g).bfloat16()
    C = (torch.randn(R, Kin, generator=g) * (3 * 0.02 ** 2 / R) ** 0.5).bfloat16()
    dy = torch.randn(T, n_loc, generator=g).bfloat16()
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    S = torch.from_numpy(O.c_noise_f32(n_loc, R, seed, row0=row0))
    W = S @ C.float()                                            # [n_loc, K]
    opts = _lib.CallOptions(stage_noise=stage)
    assert K.linear_stages_noise(T, Kin, n_loc, R, torch.bfloat16, options=opts) == (stage == 2)
    xg, Cg, dyg = x.cuda(), C.cuda(), dy.cuda()
    y = K.linear_fwd(xg, Cg, seed, n_loc, row0, options=opts)
    dx, dc = K.linear_bwd(dyg, xg, Cg, seed, row0, options=opts)
    torch.cuda.synchronize()
    K.check_status()
    ok, rel, worst = _close_big(y, x.float() @ W.t(), BF16_TOL)
    assert ok, f"y rel {rel:.3e} worst excess {worst:.3e}"
    ok, rel, worst = _close_big(dx, dy.float() @ W, BF16_TOL)
    assert ok, f"dx rel {rel:.3e} worst excess {worst:.3e}"
    dW = dy.float().t() @ x.float()                              # [n_loc, K]
    ok, rel, worst = _close_big(dc, S.t() @ dW, BF16_TOL)
    assert ok, f"dc rel {rel:.3e} worst excess {worst:.3e}"


# ---- the W path on the tensor-core kernels ---------------------------------------------------------------------------
@pytest.mark.parametrize("T,Kin,N,R,seed,row0", [(4096, 1024, 1024, 1024, 3, 0), (1000, 264, 136, 520, 11, 40)])
def test_bf16_w_path_on_tensor_cores(K, T, Kin, N, R, seed, row0):
    """Large d_c: fewer FLOPs through W = S C.  AUTO picks that association and the tcgen05 kernels for it (S hashed once,
    W bf16 in the workspace, plain tensor-core products); the forced call and the CUDA-core W path agree."""
    from randumb_b200 import _lib
    assert K.linear_plan(T, Kin, N, R, torch.bfloat16) == (_lib.PATH_WPATH, _lib.IMPL_UMMA)
    _check(K, T, Kin, N, R, torch.bfloat16, seed, row0, K.PATH_AUTO, K.IMPL_AUTO, BF16_TOL)
    _check(K, T, Kin, N, R, torch.bfloat16, seed, row0, K.PATH_WPATH, K.IMPL_UMMA, BF16_TOL)
    _check(K, T, Kin, N, R, torch.bfloat16, seed, row0, K.PATH_WPATH, K.IMPL_SIMT, BF16_TOL)


def test_unaligned_views_fall_back_to_cuda_cores(K):
    """bf16 operands that start 8 bytes into an allocation cannot be addressed by TMA: AUTO runs the CUDA-core kernels
    (same results within tolerance), a forced tensor-core call is an alignment error."""
    T, Kin, N, R, seed = 96, 128, 256, 64, 5
    x, C, dy = _inputs(T, Kin, N, R, torch.bfloat16, seed)
    buf = torch.empty(T * Kin + 4, dtype=torch.bfloat16, device="cuda")
    xv = buf[4:].view(T, Kin)
    xv.copy_(x)
    assert xv.data_ptr() % 16 == 8 and xv.is_contiguous()
    y_ref, dx_ref, dc_ref = O.linear_reference(x, C, seed, N, 0, dy, dtype=torch.float32)
    y = K.linear_fwd(xv, C.cuda(), seed, N)
    dx, dc = K.linear_bwd(dy.cuda(), xv, C.cuda(), seed)
    torch.cuda.synchronize()
    assert O.close(y, y_ref, BF16_TOL) and O.close(dx, dx_ref, BF16_TOL) and O.close(dc, dc_ref, BF16_TOL)
    with pytest.raises(RuntimeError, match="16-byte"):
        K.linear_fwd(xv, C.cuda(), seed, N, impl=K.IMPL_UMMA)


# ---- the reference's 1-D coefficient form -------------------------------------------------------------------
def test_materialize_against_reference_kernel_outputs(K, golden):
    coef = torch.from_numpy(golden["matfwd_coef"]).cuda()
    got = K.materialize_fwd(coef, [18, 18], [18, 1], 1337).cpu().numpy()
    np.testing.assert_allclose(got, golden["matfwd_18x18_contig_seed1337"], atol=3e-6)
    got = K.materialize_fwd(coef, [18, 10], [1, 18], 5).cpu().numpy()
    np.testing.assert_allclose(got, golden["matfwd_18x10_transposed_seed5"], atol=3e-6)
    got = K.materialize_fwd(coef, [70], [1], 42).cpu().numpy()
    np.testing.assert_allclose(got, golden["matfwd_70x1_seed42"].ravel(), atol=3e-6)
    dout = torch.from_numpy(golden["matbwd_dout"]).cuda()
    got = K.materialize_bwd(dout, 24, 1337).cpu().numpy()
    np.testing.assert_allclose(got, golden["matbwd_333_M24_seed1337"], atol=2e-5)
    # larger, against the oracle
    coef2 = torch.randn(300, generator=torch.Generator().manual_seed(1))
    want = O.materialize_fwd(coef2.numpy(), 40, 50, 50, 1, 3)
    got = K.materialize_fwd(coef2.cuda(), [40, 50], [50, 1], 3).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    dout2 = torch.randn(20000, generator=torch.Generator().manual_seed(2))
    want = O.materialize_bwd(dout2.numpy(), 37, 8)
    got = K.materialize_bwd(dout2.cuda(), 37, 8).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-3)
