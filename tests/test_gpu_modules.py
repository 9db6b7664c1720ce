"""The reference-facing layers on the GPU: torch.library operators with autograd, the RandumbTensor
subclass, the modules, and one training step of the MNIST-shaped MLP against the oracle."""
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


def test_rlinear_autograd_matches_oracle(rb):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 9, 40, generator=g)
    C = torch.randn(6, 40, generator=g) * 0.2
    dy = torch.randn(4, 9, 24, generator=g)
    y_ref, dx_ref, dc_ref = O.linear_reference(x.reshape(-1, 40), C, 5, 24, 3, dy.reshape(-1, 24))
    xg = x.cuda().requires_grad_(True)
    Cg = C.cuda().requires_grad_(True)
    y = rb.rlinear(xg, Cg, 5, 24, row0=3)
    assert y.shape == (4, 9, 24)
    y.backward(dy.cuda())
    assert O.close(y.reshape(-1, 24), y_ref, 1e-5)
    assert O.close(xg.grad.reshape(-1, 40), dx_ref, 1e-5)
    assert O.close(Cg.grad, dc_ref, 1e-5)
    # only the coefficient needs a gradient: dx is not computed
    x2 = x.cuda()
    C2 = C.cuda().requires_grad_(True)
    rb.rlinear(x2, C2, 5, 24, row0=3).backward(dy.cuda())
    assert O.close(C2.grad, dc_ref, 1e-5)


def test_opcheck_rlinear(rb):
    x = torch.randn(16, 24, device="cuda", requires_grad=True)
    C = torch.randn(8, 24, device="cuda", requires_grad=True)
    torch.library.opcheck(torch.ops.rten.rlinear_fwd.default, (x, C, 3, 32, 0),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_randumb_tensor_as_linear_weight(rb):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(10, 32, generator=g)
    C = torch.randn(8, 32, generator=g) * 0.2
    dy = torch.randn(10, 48, generator=g)
    y_ref, dx_ref, dc_ref = O.linear_reference(x, C, 9, 48, 0, dy)
    coef = torch.nn.Parameter(C.cuda())
    rt = rb.CreateRandumbTensor(coef, 9, (48, 32))
    xg = x.cuda().requires_grad_(True)
    y = F.linear(xg, rt)                       # fused operator, W never materialised
    y.backward(dy.cuda())
    assert O.close(y, y_ref, 1e-5) and O.close(xg.grad, dx_ref, 1e-5) and O.close(coef.grad, dc_ref, 1e-5)
    # explicit matmul with the transposed view: dispatch-level route (mm -> fused forward; backward through
    # the constructor edge with a dense dW, like the reference)
    coef.grad = None
    xg2 = x.cuda().requires_grad_(True)
    y2 = torch.mm(xg2, rt.t())
    y2.backward(dy.cuda())
    assert O.close(y2, y_ref, 1e-5) and O.close(xg2.grad, dx_ref, 1e-5) and O.close(coef.grad, dc_ref, 1e-5)
    # debugging helpers
    W = rt.get_materialized()
    S = rt.get_noise_matrix()
    assert W.shape == (48, 32) and S.shape == (48, 8)
    assert O.close(W, S.double().cpu() @ C.double(), 1e-5)
    # any other op materialises, runs, and drops the dense copy
    assert O.close((rt * 2.0), 2.0 * (S.double().cpu() @ C.double()), 1e-5)
    assert rt._tensor is None


def test_reference_form_tensor(rb, golden):
    import numpy as np
    coef = torch.nn.Parameter(torch.from_numpy(golden["matfwd_coef"]).cuda())
    rt = rb.CreateRandumbTensor(coef, 1337, (18, 18))
    np.testing.assert_allclose(rt.get_materialized().cpu().numpy(), golden["matfwd_18x18_contig_seed1337"], atol=3e-6)
    np.testing.assert_allclose(rb.CreateRandumbTensor(coef, 5, (10, 18)).t().get_materialized().cpu().numpy(),
                               golden["matfwd_18x10_transposed_seed5"], atol=3e-6)
    x = torch.randn(7, 18, device="cuda")
    y = F.linear(x, rt)
    y.sum().backward()
    dW = x.sum(0).repeat(18, 1)                # d(sum y)/dW[o, i] = sum_t x[t, i]
    want = O.materialize_bwd(dW.cpu().numpy(), 24, 1337)
    np.testing.assert_allclose(coef.grad.cpu().numpy(), want, rtol=1e-4, atol=1e-4)


def test_silly_linear_with_pseudorandom_bias(rb):
    torch.manual_seed(0)
    m = rb.SillyLinear(32, 48, rb.stepgen(8, 0), rb.stepgen(13, 7), coef_form="matrix")
    with torch.no_grad():
        m.bias_coef.uniform_(-0.3, 0.3)        # 1-D-form tensors start from zero coefficients
    m = m.cuda()
    assert m.weight.device.type == "cuda" and m.weight._coef is m.weight_coef
    x = torch.randn(5, 32, device="cuda")
    y = m(x)
    W = O.noise_f32(48, 8, 13).astype("float64") @ m.weight_coef.detach().double().cpu().numpy()
    b = O.materialize_fwd(m.bias_coef.detach().cpu().numpy(), 1, 48, 0, 1, 20).ravel()
    want = x.double().cpu().numpy() @ W.T + b
    assert O.close(y, torch.from_numpy(want), 1e-5)
    y.sum().backward()
    assert m.weight_coef.grad is not None and m.bias_coef.grad is not None
    want_db = O.materialize_bwd(torch.full((48,), 5.0).numpy(), 8, 20)
    assert O.close(m.bias_coef.grad, torch.from_numpy(want_db), 1e-5)


def test_mnist_shaped_mlp_step(rb):
    """784 -> 256 -> 10 with d_c = 64, seeds 0 and 1, float32, batch 64: loss and every gradient against
    explicit-noise autograd on the CPU in float64."""
    g = torch.Generator().manual_seed(1001)
    x = torch.rand(64, 784, generator=g)
    labels = torch.randint(0, 10, (64,), generator=g)
    seeds = rb.stepgen(0, 1)
    l1 = rb.RandumbLinear(784, 256, 64, next(seeds)).cuda()
    l2 = rb.RandumbLinear(256, 10, 64, next(seeds)).cuda()
    h = F.relu(l1(x.cuda()))
    loss = F.cross_entropy(l2(h), labels.cuda())
    loss.backward()
    C1 = l1.weight_coef.detach().double().cpu().requires_grad_(True)
    C2 = l2.weight_coef.detach().double().cpu().requires_grad_(True)
    W1 = torch.from_numpy(O.noise_f32(256, 64, 0)).double() @ C1
    W2 = torch.from_numpy(O.noise_f32(10, 64, 1)).double() @ C2
    ref = F.cross_entropy(F.linear(F.relu(F.linear(x.double(), W1)), W2), labels)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 1e-5
    assert abs(float(ref) - 2.3026) < 0.2        # ln 10 at initialisation
    assert O.close(l1.weight_coef.grad, C1.grad, 1e-5), O.rel_fro(l1.weight_coef.grad, C1.grad)
    assert O.close(l2.weight_coef.grad, C2.grad, 1e-5), O.rel_fro(l2.weight_coef.grad, C2.grad)


def test_gpt2_shaped_mlp_block_step(rb):
    """GPT-2-small MLP block (768 -> 3072 -> 768, d_c = 128, bf16, 2048 tokens, seeds from stepgen): forward, dX and both
    coefficient gradients against explicit-noise autograd in float32 on the CPU (bf16-rounded inputs and coefficients)."""
    g = torch.Generator().manual_seed(77)
    seeds = rb.stepgen(13, 7)
    c_fc = rb.RandumbLinear(768, 3072, 128, next(seeds), device="cuda", dtype=torch.bfloat16)
    c_proj = rb.RandumbLinear(3072, 768, 128, next(seeds), device="cuda", dtype=torch.bfloat16)
    x = torch.randn(2, 1024, 768, generator=g).bfloat16()
    dout = torch.randn(2, 1024, 768, generator=g).bfloat16()
    xg = x.cuda().requires_grad_(True)
    out = c_proj(F.gelu(c_fc(xg), approximate="tanh"))
    out.backward(dout.cuda())
    C1 = c_fc.weight_coef.detach().float().cpu().requires_grad_(True)
    C2 = c_proj.weight_coef.detach().float().cpu().requires_grad_(True)
    W1 = torch.from_numpy(O.noise_f32(3072, 128, 13)) @ C1
    W2 = torch.from_numpy(O.noise_f32(768, 128, 20)) @ C2
    xr = x.float().requires_grad_(True)
    ref = F.linear(F.gelu(F.linear(xr, W1), approximate="tanh"), W2)
    ref.backward(dout.float())
    assert O.close(out.reshape(-1, 768), ref.reshape(-1, 768), 2e-2), O.rel_fro(out.reshape(-1, 768), ref.reshape(-1, 768))
    assert O.close(xg.grad.reshape(-1, 768), xr.grad.reshape(-1, 768), 3e-2), O.rel_fro(xg.grad.reshape(-1, 768), xr.grad.reshape(-1, 768))
    # two bf16 layers and a nonlinearity deep: the gradients carry both layers' rounding
    assert O.rel_fro(c_fc.weight_coef.grad, C1.grad) < 3e-2 and O.rel_fro(c_proj.weight_coef.grad, C2.grad) < 3e-2


def test_bf16_module_and_state_roundtrip(rb):
    m = rb.RandumbLinear(256, 384, 64, seed=11, bias=True, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(4, 100, 256, device="cuda", dtype=torch.bfloat16)
    y = m(x)
    y_ref, _, _ = O.linear_reference(x.reshape(-1, 256).cpu(), m.weight_coef.detach().cpu(), 11, 384, dtype=torch.float32)
    assert O.close(y.reshape(-1, 384), y_ref, 2e-2)
    m2 = rb.RandumbLinear(256, 384, 64, seed=99, bias=True, device="cuda", dtype=torch.bfloat16)
    m2.load_state_dict(m.state_dict())
    assert torch.equal(m2(x), y)


def test_cpp_namespace_ops(rb):
    import numpy as np
    s = torch.ops.rten_cpp.sq5_gen_2d(6, 10, 3)      # non-square: rows x cols
    assert np.array_equal(s.cpu().numpy().view(np.uint32), O.noise_f32(6, 10, 3).view(np.uint32))
    coef = torch.randn(12, device="cuda")
    w = torch.ops.rten_cpp.materialize_fwd(coef, 3, 5, 7, 7, 1)
    np.testing.assert_allclose(w.cpu().numpy(), O.materialize_fwd(coef.cpu().numpy(), 5, 7, 7, 1, 3), atol=1e-5)
