"""Host-side mirror of the reference interface: operator schemas, the tensor subclass's metadata
handling, module conventions, sharding arithmetic.  CPU only -- no kernel runs here."""
import math
import os

import pytest
import torch

import randumb_b200 as rb
from randumb_b200 import parallel
from randumb_b200.tensor import RandumbTensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_operator_schemas_match_reference_names():
    s = str(torch.ops.rten.materialize_fwd.default._schema)
    assert s == ("rten::materialize_fwd(Tensor coefs, SymInt[] size, SymInt[] strides, SymInt seed, "
                 "Tensor? scale_bias, bool fused_bias) -> Tensor")
    assert str(torch.ops.rten.materialize_bwd.default._schema) == \
        "rten::materialize_bwd(Tensor dout, SymInt dcoefs_size, SymInt seed) -> Tensor"
    assert "rten::rlinear_fwd(Tensor x, Tensor coef, SymInt seed, SymInt out_features, SymInt row0=0) -> Tensor" == \
        str(torch.ops.rten.rlinear_fwd.default._schema)
    assert str(torch.ops.rten_cpp.sq5_gen_2d.default._schema) == "rten_cpp::sq5_gen_2d(SymInt M, SymInt N, SymInt seed) -> Tensor"
    assert str(torch.ops.rten_cpp.materialize_fwd.default._schema).startswith("rten_cpp::materialize_fwd(Tensor coef, SymInt seed, SymInt P")


def test_cpu_calls_raise_like_the_reference():
    with pytest.raises(NotImplementedError, match="Unsupported CPU implementation"):
        rb.ops.rlinear_fwd(torch.ones(2, 3), torch.ones(4, 3), 0, 5)
    with pytest.raises(NotImplementedError, match="Unsupported CPU implementation"):
        rb.ops.materialize_bwd(torch.ones(6), 3, 0)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        rb.kernels.linear_fwd(torch.ones(2, 3), torch.ones(4, 3), 0, 5)


def test_fake_tensor_tracing_gives_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(6, 5, 3, device="cuda")
        c = torch.empty(4, 3, device="cuda")
        assert rb.rlinear(x, c, 0, 7).shape == (6, 5, 7)
        dx, dc = rb.ops.rlinear_bwd(torch.empty(30, 7, device="cuda"), x.reshape(30, 3), c, 0, 0, True, False)
        assert dx.shape == (30, 3) and dc.numel() == 0


def test_randumb_tensor_metadata_and_views():
    coef = torch.zeros(8, 16)
    rt = rb.CreateRandumbTensor(coef, 5, (24, 16))
    assert isinstance(rt, RandumbTensor) and rt.is_matrix_form
    assert rt.noise_matrix_shape == (24, 8) and rt.int_dim == 8
    t = rt.t()
    assert isinstance(t, RandumbTensor) and t.shape == (16, 24) and t.stride() == (1, 16)
    assert t._is_transposed() and t.noise_matrix_shape == (24, 8)
    h = rt.to(torch.bfloat16)
    assert isinstance(h, RandumbTensor) and h.dtype == torch.bfloat16 and h._coef.dtype == torch.bfloat16
    with pytest.raises(AssertionError):
        rb.CreateRandumbTensor(torch.zeros(8, 15), 5, (24, 16))        # coef columns != in_features
    # reference form: 1-D coefficient, any shape, views keep working
    r1 = rb.CreateRandumbTensor(torch.zeros(6), 3, (4, 10))
    assert not r1.is_matrix_form and r1.noise_matrix_shape == (40, 6)
    v = r1.view(8, 5).transpose(0, 1)
    assert isinstance(v, RandumbTensor) and v.shape == (5, 8) and v.stride() == (1, 5)
    with pytest.raises(Exception):
        v.view(40)                                                       # incompatible view is refused


def test_constructor_edge_tracks_coef():
    coef = torch.nn.Parameter(torch.zeros(8, 16))
    rt = rb.CreateRandumbTensor(coef, 5, (24, 16))
    assert rt.requires_grad and rt.grad_fn is not None


def test_seed_generators():
    g = rb.stepgen(13, 7)
    assert [next(g) for _ in range(4)] == [13, 20, 27, 34]
    assert list(rb.listgen([3, 1, 2])) == [3, 1, 2]


def test_randumb_linear_init_and_state():
    m = rb.RandumbLinear(784, 256, 64, seed=0)
    assert m.weight_coef.shape == (64, 784)
    # coef ~ N(0, 3 std^2 / d_c) with std^2 = 1/(3 fan_in)
    want = math.sqrt(3.0 / 64) * math.sqrt(1.0 / (3 * 784))
    assert abs(float(m.weight_coef.detach().std()) - want) / want < 0.05
    m2 = rb.RandumbLinear(784, 256, 64, seed=0)
    assert torch.equal(m.weight_coef, m2.weight_coef)                    # init is a function of the seed
    sd = m.state_dict()
    assert set(sd.keys()) == {"weight_coef", "_extra_state"} and sd["_extra_state"]["seed"] == 0
    m3 = rb.RandumbLinear(784, 256, 64, seed=9)
    m3.load_state_dict(sd)
    assert m3.seed == 0 and torch.equal(m3.weight_coef, m.weight_coef) and m3.weight.seed == 0
    m3.to(torch.bfloat16)
    assert m3.weight.dtype == torch.bfloat16 and m3.weight._coef is m3.weight_coef


def test_silly_linear_conventions():
    # an unchanged reference call site: generators for int_dim and seed, 1-D coefficient vectors
    s = rb.SillyLinear(16, 24, rb.stepgen(8, 0), rb.stepgen(13, 7))
    assert s.int_dim == [8, 8] and s.seed == [13, 20] and s.coef_form == "vector"
    assert s.weight_coef.shape == (8,) and s.bias_coef.shape == (8,)
    assert s.weight.seed == 13 and s.bias.seed == 20 and not s.weight.is_matrix_form and not s.bias.is_matrix_form
    assert {n for n, _ in s.named_parameters()} == {"weight_coef", "bias_coef", "weight_scale_bias", "bias_scale_bias"}
    assert not s.weight.fused_bias and s.weight.scale_bias is s.weight_scale_bias
    s2 = rb.SillyLinear(16, 24, [4, 2], [1, 2], bias=False)
    assert s2.bias is None
    # the matrix-coefficient form is opt-in
    s3 = rb.SillyLinear(16, 24, [4, 2], [1, 2], coef_form="matrix")
    assert s3.weight_coef.shape == (4, 16) and s3.weight.is_matrix_form and float(s3.weight_coef.detach().abs().sum()) > 0
    assert {n for n, _ in s3.named_parameters()} == {"weight_coef", "bias_coef", "bias_scale_bias"}


def _build_from_case(cls_name, case):
    def gen(spec):
        if spec[0] == "list":
            return list(spec[1])
        if spec[0] == "listgen":
            return rb.listgen(list(spec[1]))
        return rb.stepgen(spec[1], spec[2])
    return getattr(rb, cls_name)(*case["args"], gen(case["int_dim"]), gen(case["seed"]), **case["kwargs"])


def test_modules_match_the_reference_classes_parameter_for_parameter():
    """tests/golden/ref_modules.json holds, for a list of constructor calls, what the reference's own classes create on
    CPU (written by tests/golden/make_golden.py): parameter names, shapes, initial values, buffer names, seeds.  The
    same calls on this library's classes must give the same state_dict keys and shapes, so a reference checkpoint
    loads, and the same initial values."""
    import json
    with open(os.path.join(ROOT, "tests", "golden", "ref_modules.json")) as f:
        records = json.load(f)
    assert len(records) >= 7
    for rec in records:
        m = _build_from_case(rec["cls"], rec["case"])
        ours = dict(m.named_parameters())
        assert set(ours) == set(rec["params"]), (rec["cls"], rec["case"], sorted(ours))
        assert list(m.seed) == rec["seed"] and list(m.int_dim) == rec["int_dim"]
        assert sorted(n for n, _ in m.named_buffers()) == sorted(rec["buffers"])
        for name, want in rec["params"].items():
            p = ours[name].detach()
            assert list(p.shape) == want["shape"], (rec["cls"], name)
            assert [float(v) for v in p.flatten()[:8]] == want["head"], (rec["cls"], name)
            assert abs(float(p.abs().sum()) - want["abs_sum"]) <= 1e-6 * max(1.0, want["abs_sum"])
        # a checkpoint written by the reference: the parameters plus a dense copy of every virtual tensor
        sd = {n: torch.full(want["shape"], 0.5) for n, want in rec["params"].items()}
        for b in rec["buffers"]:
            sd[b] = torch.zeros(tuple(getattr(m, b).shape))
        m.load_state_dict(sd)
        assert all(float(p.detach().flatten()[0]) == 0.5 for p in m.parameters())
        assert set(m.state_dict()) == set(rec["params"])            # virtual tensors are regenerated, never stored


@pytest.mark.parametrize("total,world", [(65536, 8), (16384, 4), (1000, 3), (8, 8), (10, 4), (0, 2)])
def test_shard_ranges_partition(total, world):
    rs = parallel.all_shard_ranges(total, world)
    assert rs[0][0] == 0 and rs[-1][1] == total
    for (a, b), (c, d) in zip(rs, rs[1:]):
        assert b == c and a <= b
    for lo, hi in rs[:-1]:
        assert (lo % 8 == 0 or lo == total) and (hi % 8 == 0 or hi == total)
    sizes = [hi - lo for lo, hi in rs]
    assert max(sizes) - min(sizes) <= 8


def test_vector_form_operator_schemas_and_cpu_stubs():
    assert str(torch.ops.rten.scale_bias_bwd.default._schema) == "rten::scale_bias_bwd(Tensor dout, SymInt seed) -> Tensor"
    assert str(torch.ops.rten.embed_fwd.default._schema) == \
        "rten::embed_fwd(Tensor idx, Tensor coefs, SymInt rowsize, SymInt seed) -> Tensor"
    assert str(torch.ops.rten.embed_bwd.default._schema) == \
        "rten::embed_bwd(Tensor idx, Tensor dout, SymInt dcoefs_size, SymInt rowsize, SymInt seed) -> Tensor"
    for call in (lambda: rb.ops.scale_bias_bwd(torch.ones(4), 0),
                 lambda: rb.ops.embed_fwd(torch.zeros(3, dtype=torch.int64), torch.ones(4), 5, 0),
                 lambda: rb.ops.rt_mm(torch.ones(2, 3), torch.ones(4), [3, 5], [5, 1], 0)):
        with pytest.raises(NotImplementedError, match="Unsupported CPU implementation"):
            call()
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        idx = torch.empty(2, 7, dtype=torch.int64, device="cuda")
        assert rb.ops.embed_fwd(idx, torch.empty(9, device="cuda"), 16, 1).shape == (2, 7, 16)
        assert rb.ops.scale_bias_bwd(torch.empty(50, device="cuda"), 1).shape == (1,)


def test_reference_convention_modules_on_cpu():
    """Parameters, buffers and the random-bias scales of the reference-style layers (construction only)."""
    m = rb.SillyLinear(12, 20, rb.listgen([6, 4]), rb.stepgen(3, 2), rt_bias=True)
    assert m.seed == [3, 5] and m.int_dim == [6, 4]
    assert {n for n, _ in m.named_parameters()} == {"weight_coef", "bias_coef", "weight_scale_bias", "bias_scale_bias"}
    assert m.weight.fused_bias and m.weight.scale_bias is m.weight_scale_bias and not m.weight.is_matrix_form
    assert abs(float(m.bias_scale_bias.detach()) - 1.0 / math.sqrt(12)) < 1e-6 and float(m.weight_coef.detach().abs().sum()) == 0.0
    assert list(m.state_dict()) == ["weight_coef", "bias_coef", "weight_scale_bias", "bias_scale_bias"]   # virtual tensors are not stored
    m.init_uniform_coef_zero_bias()                                     # the reference's other start
    assert float(m.weight_coef.detach().abs().sum()) > 0 and float(m.weight_scale_bias.detach()) == 0.0
    assert m.weight.scale_bias is m.weight_scale_bias
    mm = rb.SillyLinear(12, 20, [6, 4], [3, 5], rt_bias=True, coef_form="matrix")   # matrix-form weight: only the bias has a scale
    assert mm.weight.is_matrix_form and {n for n, _ in mm.named_parameters()} == {"weight_coef", "bias_coef", "bias_scale_bias"}
    with pytest.raises(ValueError):
        rb.SillyLinear(4, 4, [2, 2], [0, 1], coef_form="dense")
    e = rb.SillyEmbedding(100, 16, [8], rb.stepgen(9, 1), device="cpu")
    assert e.weight.shape == (100, 16) and e.weight_coef.shape == (8,) and e.seed == [9]
    with pytest.raises(AssertionError):
        rb.SillyEmbedding(10, 4, [2], [0], padding_idx=0, device="cpu")
    c = rb.SillyConv2d(3, 8, [16, 4], [5, 6], 3, padding=1)
    assert tuple(c.weight.shape) == (8, 3, 3, 3) and c.weight.noise_matrix_shape == (216, 16) and c.bias.shape == (8,)
    assert {n for n, _ in c.named_parameters()} == {"weight_coef", "bias_coef", "weight_scale_bias", "bias_scale_bias"}


def test_a_status_word_set_by_a_kernel_raises_and_is_cleared():
    """The host half of the bounded waits: a kernel whose wait expires writes a code into the per-device status words;
    ``kernels.check_status`` turns it into an exception and clears the words.  The code is injected here on the host (a CPU
    tensor stands in for the device words) -- no device wait is made to expire."""
    from randumb_b200 import kernels as K, _lib
    saved = dict(K._status_bufs)
    try:
        for code, text in ((2, "mma wait expired"), (4, "generator wait expired"), (5, "peer wait expired")):
            K._status_bufs.clear()
            K._status_bufs[0] = torch.tensor([code, 0, 0, 0], dtype=torch.int32)
            with pytest.raises(RuntimeError, match=text):
                K.check_status()
            assert K._status_bufs[0].tolist() == [0, 0, 0, 0]
            K.check_status()                          # clean again
        assert set(_lib.STATUS_NAMES) >= {0, 1, 2, 3, 4, 5}
    finally:
        K._status_bufs.clear()
        K._status_bufs.update(saved)
