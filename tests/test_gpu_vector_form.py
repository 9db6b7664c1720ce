"""1-D-coefficient form on the GPU: fused random bias, its scale gradient, and embedding rows, against the
reference kernels' own outputs (golden fixtures) and the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    import randumb_b200
    assert torch.cuda.is_available()
    return randumb_b200


@pytest.fixture(scope="module")
def K(rb):
    return rb.kernels


def test_fused_random_bias_against_reference_kernel_outputs(K, golden):
    coef = torch.from_numpy(golden["matfwd_coef"]).cuda()
    sb = torch.tensor([0.25], device="cuda")
    got = K.materialize_fwd(coef, [18, 18], [18, 1], 1337, sb).cpu().numpy()
    np.testing.assert_allclose(got, golden["matfwd_18x18_bias0p25_seed1337"], atol=3e-6)
    sb = torch.tensor([-0.5], device="cuda")
    got = K.materialize_fwd(coef, [18, 10], [1, 18], 5, sb).cpu().numpy()
    np.testing.assert_allclose(got, golden["matfwd_18x10_transposed_bias_m0p5_seed5"], atol=3e-6)
    got = K.scale_bias_bwd(torch.from_numpy(golden["matbwd_dout"]).cuda(), 1337).cpu().numpy()
    np.testing.assert_allclose(got, golden["scale_bias_bwd_333_seed1337"], atol=1e-5)


def test_bias_term_is_bit_exact_noise(K):
    """Zero coefficients and scale 1: the output is the 1-D noise of the element index, bit for bit."""
    coef = torch.zeros(5, device="cuda")
    one = torch.ones(1, device="cuda")
    got = K.materialize_fwd(coef, [33, 47], [47, 1], 99, one).cpu().numpy().ravel()
    want = O.bits_to_f32(O.noise_bits_1d(33 * 47, 99))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_scale_bias_bwd_large_and_empty(K):
    g = torch.Generator().manual_seed(3)
    dout = torch.randn(3 * 8192 + 17, generator=g)          # several reduction spans and a ragged tail
    got = float(K.scale_bias_bwd(dout.cuda(), 21))
    want = O.scale_bias_bwd(dout.numpy(), 21)
    assert abs(got - want) <= 1e-4 * max(1.0, abs(want))
    again = float(K.scale_bias_bwd(dout.cuda(), 21))
    assert got == again                                       # fixed reduction order
    assert float(K.scale_bias_bwd(torch.empty(0, device="cuda"), 21)) == 0.0


def test_constructor_backward_returns_scale_gradient(rb, golden):
    coef = torch.nn.Parameter(torch.from_numpy(golden["matfwd_coef"]).cuda())
    scale = torch.nn.Parameter(torch.tensor([0.25], device="cuda"))
    rt = rb.CreateRandumbTensor(coef, 1337, (18, 18), scale, True)
    np.testing.assert_allclose(rt.get_materialized().cpu().numpy(), golden["matfwd_18x18_bias0p25_seed1337"], atol=3e-6)
    x = torch.randn(7, 18, device="cuda")
    F.linear(x, rt).sum().backward()
    dW = x.sum(0).repeat(18, 1).cpu().numpy()
    np.testing.assert_allclose(coef.grad.cpu().numpy(), O.materialize_bwd(dW, 24, 1337), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(float(scale.grad), O.scale_bias_bwd(dW, 1337), rtol=1e-4, atol=1e-4)


def test_silly_linear_vector_form_with_rt_bias(rb):
    """The reference's own layer: 1-D coefficients for weight and bias, zero coefficients and a random-bias
    scale at initialisation, so the layer starts as a fixed random projection."""
    m = rb.SillyLinear(32, 48, [16, 8], [13, 20], rt_bias=True).cuda()           # the default form is the reference's
    names = dict(m.named_parameters())
    assert set(names) == {"weight_coef", "bias_coef", "weight_scale_bias", "bias_scale_bias"}
    assert m.weight_coef.shape == (16,) and float(m.weight_coef.abs().sum()) == 0.0
    bound = float(m.weight_scale_bias)
    assert abs(bound - 1.0 / 32 ** 0.5) < 1e-6                 # nn.Linear's default uniform bound
    x = torch.randn(5, 32, device="cuda")
    y = m(x)
    W = bound * O.bits_to_f32(O.noise_bits_1d(48 * 32, 13)).astype("float64").reshape(48, 32)
    b = bound * O.bits_to_f32(O.noise_bits_1d(48, 20)).astype("float64")
    want = x.double().cpu().numpy() @ W.T + b
    assert O.close(y, torch.from_numpy(want), 1e-5)
    y.sum().backward()
    for p in names.values():
        assert p.grad is not None
    dW = x.sum(0).repeat(48, 1).cpu().numpy()
    assert abs(float(m.weight_scale_bias.grad) - O.scale_bias_bwd(dW, 13)) < 1e-3
    assert O.close(m.weight_coef.grad, torch.from_numpy(O.materialize_bwd(dW, 16, 13)), 1e-5)
    # moving the module keeps the scale parameters attached to the rebuilt buffers
    m = m.double().float()
    assert m.weight.scale_bias is m.weight_scale_bias and m.weight.fused_bias


def test_embedding_against_reference_kernel_outputs(K, golden):
    idx = torch.from_numpy(golden["embed_idx"]).cuda()
    coef = torch.from_numpy(golden["matfwd_coef"]).cuda()
    got = K.embed_fwd(idx, coef, 20, 77).cpu().numpy()
    np.testing.assert_allclose(got, golden["embed_fwd_13x20_seed77"], atol=3e-6)
    got = K.embed_bwd(idx, torch.from_numpy(golden["embed_dout"]).cuda(), 24, 20, 77).cpu().numpy()
    np.testing.assert_allclose(got, golden["embed_bwd_13x20_M24_seed77"], atol=1e-5)


def test_embedding_rows_equal_materialised_rows(K):
    """GPT-2-sized vocabulary: looked-up rows equal the same rows of the materialised matrix, for any index
    shape, int32 or int64, including the last row and repeats."""
    vocab, dim, M, seed = 50304, 96, 40, 4
    g = torch.Generator().manual_seed(5)
    coef = torch.randn(M, generator=g).cuda()
    idx = torch.randint(0, vocab, (3, 17), generator=g)
    idx[0, 0], idx[0, 1], idx[2, 16] = vocab - 1, vocab - 1, 0
    out = K.embed_fwd(idx.cuda(), coef, dim, seed)
    assert out.shape == (3, 17, dim)
    full = K.materialize_fwd(coef, [vocab, dim], [dim, 1], seed)
    assert torch.equal(out, full[idx.cuda()])
    assert torch.equal(K.embed_fwd(idx.int().cuda(), coef, dim, seed), out)
    want = O.embed_fwd(idx.numpy().ravel(), coef.cpu().numpy(), dim, seed)
    np.testing.assert_allclose(out.reshape(-1, dim).cpu().numpy(), want, atol=2e-5)
    assert K.embed_fwd(torch.empty(0, dtype=torch.int64, device="cuda"), coef, dim, seed).shape == (0, dim)


def test_silly_embedding_module_step(rb):
    torch.manual_seed(0)
    emb = rb.SillyEmbedding(1000, 64, [32], [9])
    idx = torch.randint(0, 1000, (4, 11), device="cuda")
    idx[1, 3] = idx[0, 0]                                     # a repeated token accumulates its gradient
    y = emb(idx)
    want = O.embed_fwd(idx.cpu().numpy().ravel(), emb.weight_coef.detach().cpu().numpy(), 64, 9)
    assert O.close(y.reshape(-1, 64), torch.from_numpy(want), 1e-5)
    # same rows through the storage-less weight buffer
    assert O.close(emb.weight.get_materialized()[idx.reshape(-1)], y.reshape(-1, 64), 1e-5)
    dout = torch.randn_like(y)
    (y * dout).sum().backward()
    want_g = O.embed_bwd(idx.cpu().numpy().ravel(), dout.cpu().numpy(), 32, 64, 9)
    assert O.close(emb.weight_coef.grad, torch.from_numpy(want_g), 1e-5)


def test_rt_mm_against_reference_kernel_output(rb, golden):
    """mat1 @ RT: the reference's fused rt_mm_grouped kernel output, and gradients against the oracle."""
    coef = torch.from_numpy(golden["matfwd_coef"]).cuda().requires_grad_(True)
    mat1 = torch.from_numpy(golden["rtmm_mat1"]).cuda().requires_grad_(True)
    out = rb.ops.rt_mm(mat1, coef, [40, 36], [36, 1], 9)
    np.testing.assert_allclose(out.detach().cpu().numpy(), golden["rtmm_33x40_40x36_seed9"], atol=5e-5)
    dout = torch.randn(33, 36, generator=torch.Generator().manual_seed(2))
    out.backward(dout.cuda())
    W = O.materialize_fwd(golden["matfwd_coef"], 40, 36, 36, 1, 9)
    np.testing.assert_allclose(mat1.grad.cpu().numpy(), dout.double().numpy() @ W.T, atol=5e-5)
    dW = golden["rtmm_mat1"].astype("float64").T @ dout.double().numpy()
    np.testing.assert_allclose(coef.grad.cpu().numpy(), O.materialize_bwd(dW.astype("float32"), 24, 9), rtol=1e-4, atol=1e-4)


def test_silly_conv2d_step(rb):
    """Convolution with a storage-less weight [out, in, kh, kw] and bias: forward and every gradient against the same
    convolution with the oracle's dense weight."""
    torch.manual_seed(0)
    m = rb.SillyConv2d(3, 8, [16, 4], [5, 6], 3, padding=1)
    m.init_uniform_coef_zero_bias()            # the default start is all-zero coefficients; use the reference's other scheme
    m = m.cuda()
    assert float(m.weight_coef.abs().sum()) > 0 and not m.weight.fused_bias
    x = torch.randn(2, 3, 10, 10, device="cuda", requires_grad=True)
    y = m(x)
    Wc = m.weight_coef.detach().double().cpu().requires_grad_(True)
    bc = m.bias_coef.detach().double().cpu().requires_grad_(True)
    S_w = torch.from_numpy(O.noise_f32(8 * 3 * 3 * 3, 16, 5)).double()
    S_b = torch.from_numpy(O.noise_f32(8, 4, 6)).double()
    xr = x.detach().double().cpu().requires_grad_(True)
    ref = F.conv2d(xr, (S_w @ Wc).reshape(8, 3, 3, 3), S_b @ bc, padding=1)
    assert O.close(y.reshape(2, -1), ref.reshape(2, -1), 1e-4)
    dout = torch.randn(2, 8, 10, 10, generator=torch.Generator().manual_seed(3))
    y.backward(dout.cuda())
    ref.backward(dout.double())
    assert O.close(m.weight_coef.grad, Wc.grad, 1e-4) and O.close(m.bias_coef.grad, bc.grad, 1e-4)
    assert O.close(x.grad.reshape(2, -1), xr.grad.reshape(2, -1), 1e-4)


def test_opcheck_vector_form_ops(rb):
    coef = torch.randn(12, device="cuda", requires_grad=True)
    idx = torch.randint(0, 30, (6,), device="cuda")
    torch.library.opcheck(torch.ops.rten.embed_fwd.default, (idx, coef, 8, 3))
    torch.library.opcheck(torch.ops.rten.scale_bias_bwd.default, (torch.randn(50, device="cuda"), 3))
    scale = torch.tensor([0.5], device="cuda", requires_grad=True)
    torch.library.opcheck(torch.ops.rten.materialize_fwd.default, (coef, [5, 6], [6, 1], 3, scale, True))
