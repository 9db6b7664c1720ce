"""Generate tests/golden/ref_vectors.npz by running the REFERENCE's own Triton kernels on CPU.

Usage (only where the reference checkout is available; the fixtures are committed):

    TRITON_INTERPRET=1 AUTOTUNE=0 python tests/golden/make_golden.py /path/to/reference

The reference package cannot be imported normally (its ``__init__`` loads an extension that
is not built), so ``RandumbTensor.py`` is loaded with importlib under a stub package.  The raw
``@triton.jit`` kernels are then launched on CPU tensors with explicit block sizes; the Triton
interpreter executes them with numpy.  No expected values are typed in by hand: everything in the
fixture file is an output of the reference code.

Kernels executed (paths inside the reference project, file ``src/rten_cpp/RandumbTensor.py``):
  squirrel5_kernel_2d :78-99   squirrel5_kernel_1d :108-114   materialize_fwd_kernel :235-290
  materialize_bwd_kernel :304-359   scale_bias_bwd_kernel :400-407   rt_mm_grouped_kernel :648-746
  embed_fwd_kernel :998-1056   embed_bwd_kernel :1060-1107
"""
import importlib.util
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("AUTOTUNE", "0")

import numpy as np
import torch


def load_reference(root: str):
    pkg_dir = os.path.join(root, "src", "rten_cpp")
    pkg = types.ModuleType("rten_ref")
    pkg.__path__ = [pkg_dir]
    sys.modules["rten_ref"] = pkg
    for name in ("utils", "RandumbTensor"):
        spec = importlib.util.spec_from_file_location(f"rten_ref.{name}", os.path.join(pkg_dir, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"rten_ref.{name}"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["rten_ref.RandumbTensor"]


def cdiv(a, b):
    return (a + b - 1) // b


def ref_noise_2d(rt, N, M, seed, row_lo=0):
    """Rows [row_lo, N) x M columns of the reference noise matrix (float32)."""
    out = torch.empty((N, M), dtype=torch.float32)
    BN, BM = 64, 16
    grid = (cdiv(N, BN), cdiv(M, BM))
    rt.squirrel5_kernel_2d[grid](out, N, M, seed, out.stride(0), out.stride(1), BLOCK_SIZE_N=BN, BLOCK_SIZE_M=BM)
    return out[row_lo:].numpy().copy()


def ref_noise_1d(rt, N, seed):
    out = torch.empty((N,), dtype=torch.float32)
    rt.squirrel5_kernel_1d[(cdiv(N, 64),)](out, N, seed, BLOCK_SIZE_N=64)
    return out.numpy().copy()


def ref_mat_fwd(rt, coef, P, Q, sP, sQ, seed):
    out = torch.empty((P, Q), dtype=torch.float32)
    N = P * Q
    dummy = torch.zeros(1, dtype=torch.float32)
    rt.materialize_fwd_kernel[(cdiv(N, 32),)](out, coef, N, coef.numel(), seed, P, Q, sP, sQ, dummy, 0,
                                              BLOCK_SIZE_N=32, BLOCK_SIZE_M=8)
    return out.numpy().copy()


def ref_mat_fwd_bias(rt, coef, P, Q, sP, sQ, seed, scale_bias):
    """materialise with the fused random bias: + scale_bias * sq5_1d(sq(n), seed)."""
    out = torch.empty((P, Q), dtype=torch.float32)
    N = P * Q
    sb = torch.tensor([scale_bias], dtype=torch.float32)
    rt.materialize_fwd_kernel[(cdiv(N, 32),)](out, coef, N, coef.numel(), seed, P, Q, sP, sQ, sb, 1,
                                              BLOCK_SIZE_N=32, BLOCK_SIZE_M=8)
    return out.numpy().copy()


def ref_scale_bias_bwd(rt, dout, seed):
    dbias = torch.zeros((1,), dtype=torch.float32)
    rt.scale_bias_bwd_kernel[(cdiv(dout.numel(), 64),)](dbias, dout, dout.numel(), seed, BLOCK_SIZE_N=64)
    return dbias.numpy().copy()


def ref_embed_fwd(rt, idx, coef, rowsize, seed):
    """Rows ``idx`` of the virtual (vocab, rowsize) embedding matrix."""
    out = torch.empty((idx.numel(), rowsize), dtype=torch.float32)
    BI, BR, BM = 16, 32, 8
    grid = (cdiv(idx.numel(), BI), cdiv(rowsize, BR))
    rt.embed_fwd_kernel[grid](out, coef, idx, rowsize, coef.numel(), idx.numel(), seed, out.stride(0),
                              BLOCK_SIZE_ROW=BR, BLOCK_SIZE_M=BM, BLOCK_SIZE_IDX=BI)
    return out.numpy().copy()


def ref_embed_bwd(rt, idx, dout, M, rowsize, seed):
    dcoef = torch.zeros((M,), dtype=torch.float32)
    SPLIT, BN, BM = 4, 32, 4
    rt.embed_bwd_kernel[(cdiv(M, BM), SPLIT)](dcoef, dout, idx, rowsize, M, idx.numel(), seed,
                                              BLOCK_SIZE_N=BN, BLOCK_SIZE_M=BM, SPLIT_N=SPLIT)
    return dcoef.numpy().copy()


def ref_mat_bwd(rt, dout, M, seed):
    dcoef = torch.zeros((M,), dtype=torch.float32)
    SPLIT, BN, BM = 4, 64, 4
    # launched through .fn to bypass the pre-run hook plumbing; the output starts at zero, as the hook would make it
    kern = rt.materialize_bwd_kernel
    kern[(cdiv(M, BM), SPLIT)](dcoef, dout, dout.numel(), M, seed, BLOCK_SIZE_N=BN, BLOCK_SIZE_M=BM, SPLIT_N=SPLIT)
    return dcoef.numpy().copy()


def ref_rt_mm(rt, mat1, coef, P, Q, sP, sQ, seed):
    L = mat1.shape[0]
    out = torch.zeros((L, Q), dtype=torch.float32)
    dummy = torch.zeros(1, dtype=torch.float32)
    BM, BP, BQ, BL, G = 32, 32, 32, 32, 2
    grid = (cdiv(L, BL), cdiv(Q, BQ), cdiv(P, BP))
    rt.rt_mm_grouped_kernel[grid](out, coef, mat1, dummy, coef.numel(), P, Q, L, sP, sQ,
                                  mat1.stride(0), mat1.stride(1), out.stride(0), out.stride(1), seed, dummy, 0,
                                  BLOCK_SIZE_M=BM, BLOCK_SIZE_P=BP, BLOCK_SIZE_Q=BQ, BLOCK_SIZE_L=BL, GROUP_SIZE=G)
    return out.numpy().copy()


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: TRITON_INTERPRET=1 AUTOTUNE=0 python tests/golden/make_golden.py /path/to/reference")
    root = sys.argv[1]
    rt = load_reference(root)
    out = {}

    # --- noise matrices (float32 bit patterns are the pin) ---------------------------------
    for seed in (0, 7, 42, 1337, -5):
        out[f"noise2d_48x20_seed{seed}"] = ref_noise_2d(rt, 48, 20, seed)
    out["noise2d_256x64_seed0"] = ref_noise_2d(rt, 256, 64, 0)
    # rows that cross the first uint32 wrap of PRIME*row (row 22) and far rows
    out["noise2d_rows65472to65536_x8_seed7"] = ref_noise_2d(rt, 65536, 8, 7, row_lo=65472)
    out["noise2d_300x130_seed42"] = ref_noise_2d(rt, 300, 130, 42)
    for seed in (0, 1337):
        out[f"noise1d_200_seed{seed}"] = ref_noise_1d(rt, 200, seed)

    # --- materialise fwd/bwd with a 1-D coefficient (the K=1 case of the matrix-coef layer) --
    g = torch.Generator().manual_seed(1234)
    coef = torch.randn(24, generator=g)
    out["matfwd_coef"] = coef.numpy().copy()
    out["matfwd_18x18_contig_seed1337"] = ref_mat_fwd(rt, coef, 18, 18, 18, 1, 1337)
    out["matfwd_18x10_transposed_seed5"] = ref_mat_fwd(rt, coef, 18, 10, 1, 18, 5)   # view of a (10,18) tensor
    out["matfwd_70x1_seed42"] = ref_mat_fwd(rt, coef, 70, 1, 1, 1, 42)
    dout = torch.randn(333, generator=g)
    out["matbwd_dout"] = dout.numpy().copy()
    out["matbwd_333_M24_seed1337"] = ref_mat_bwd(rt, dout, 24, 1337)

    # --- fused random bias (1-D hash of the element index) ------------------------------------
    out["matfwd_18x18_bias0p25_seed1337"] = ref_mat_fwd_bias(rt, coef, 18, 18, 18, 1, 1337, 0.25)
    out["matfwd_18x10_transposed_bias_m0p5_seed5"] = ref_mat_fwd_bias(rt, coef, 18, 10, 1, 18, 5, -0.5)
    out["scale_bias_bwd_333_seed1337"] = ref_scale_bias_bwd(rt, dout, 1337)

    # --- embedding rows of a virtual (vocab, rowsize) matrix -----------------------------------
    idx = torch.randint(0, 50, (13,), generator=g, dtype=torch.int64)
    idx[3] = idx[7]                      # a repeated token
    out["embed_idx"] = idx.numpy().copy()
    out["embed_fwd_13x20_seed77"] = ref_embed_fwd(rt, idx, coef, 20, 77)
    edout = torch.randn(13, 20, generator=g)
    out["embed_dout"] = edout.numpy().copy()
    out["embed_bwd_13x20_M24_seed77"] = ref_embed_bwd(rt, idx, edout, 24, 20, 77)

    # --- the reference's fused mat1 @ RT kernel --------------------------------------------
    P, Q, L = 40, 36, 33
    mat1 = torch.randn(L, P, generator=g)
    out["rtmm_mat1"] = mat1.numpy().copy()
    out["rtmm_33x40_40x36_seed9"] = ref_rt_mm(rt, mat1, coef, P, Q, Q, 1, 9)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})

    write_module_fixture(root)


# constructor cases of the reference's modules; "args" are passed positionally after the generators are built
MODULE_CASES = [
    ("SillyLinear", dict(args=[12, 20], int_dim=("listgen", [6, 4]), seed=("stepgen", 3, 2), kwargs={})),
    ("SillyLinear", dict(args=[12, 20], int_dim=("list", [6, 4]), seed=("list", [3, 5]), kwargs={"bias": False, "rt_bias": True})),
    ("SillyLinear", dict(args=[768, 3072], int_dim=("stepgen", 256, 0), seed=("stepgen", 13, 7), kwargs={"bias": False})),
    ("SillyConv2d", dict(args=[3, 8], int_dim=("list", [16, 4]), seed=("list", [5, 6]), kwargs={"kernel_size": 3, "padding": 1})),
    ("SillyConv2d", dict(args=[1, 32], int_dim=("stepgen", 128, 0), seed=("stepgen", 5, 4), kwargs={"kernel_size": 3, "stride": 1, "rt_bias": True})),
    ("SillyEmbedding", dict(args=[100, 16], int_dim=("list", [8]), seed=("stepgen", 9, 1), kwargs={"device": "cpu"})),
    ("SillyEmbedding", dict(args=[100, 16], int_dim=("list", [8]), seed=("stepgen", 9, 1), kwargs={"rt_bias": True, "device": "cpu"})),
]


def build_module(layers, cls_name, case):
    """Construct ``cls_name`` from a MODULE_CASES entry with the generators of ``layers`` (the reference's module
    file, or the library under test: both export stepgen / listgen and the three classes)."""
    def gen(spec):
        kind = spec[0]
        if kind == "list":
            return list(spec[1])
        if kind == "listgen":
            return layers.listgen(list(spec[1]))
        return layers.stepgen(spec[1], spec[2])
    return getattr(layers, cls_name)(*case["args"], gen(case["int_dim"]), gen(case["seed"]), **case["kwargs"])


def write_module_fixture(root):
    """Parameter names, shapes and initial values of the reference's modules for MODULE_CASES, constructed on CPU
    (src/rten_cpp/SillyLayers.py); virtual tensors are listed by buffer name."""
    import json
    pkg_dir = os.path.join(root, "src", "rten_cpp")
    spec = importlib.util.spec_from_file_location("rten_ref.SillyLayers", os.path.join(pkg_dir, "SillyLayers.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["rten_ref.SillyLayers"] = mod
    spec.loader.exec_module(mod)
    records = []
    for cls_name, case in MODULE_CASES:
        m = build_module(mod, cls_name, case)
        params = {n: {"shape": list(p.shape), "head": [float(v) for v in p.detach().flatten()[:8]],
                      "abs_sum": float(p.detach().abs().sum())} for n, p in m.named_parameters()}
        records.append({"cls": cls_name, "case": case, "params": params, "buffers": [n for n, _ in m.named_buffers()],
                        "seed": list(m.seed), "int_dim": list(m.int_dim)})
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_modules.json")
    with open(dst, "w") as f:
        json.dump(records, f, indent=1)
    print("wrote", dst, len(records), "module cases")


if __name__ == "__main__":
    main()
