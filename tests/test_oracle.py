"""The CPU oracle against the reference's own outputs (golden vectors) and against itself (numpy vs C)."""
import zlib

import numpy as np
import pytest
import torch

from oracle import oracle as O


def _bits_equal(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


@pytest.mark.parametrize("seed", [0, 7, 42, 1337, -5])
def test_noise_matches_reference_kernel(golden, seed):
    ref = golden[f"noise2d_48x20_seed{seed}"]
    assert _bits_equal(O.noise_f32(48, 20, seed), ref)
    assert _bits_equal(O.c_noise_f32(48, 20, seed), ref)


def test_noise_larger_and_far_rows(golden):
    assert _bits_equal(O.noise_f32(256, 64, 0), golden["noise2d_256x64_seed0"])
    assert _bits_equal(O.noise_f32(300, 130, 42), golden["noise2d_300x130_seed42"])
    # rows 65472..65535: PRIME*row has wrapped 2^32 many times by then
    assert _bits_equal(O.noise_f32(64, 8, 7, row0=65472), golden["noise2d_rows65472to65536_x8_seed7"])
    assert _bits_equal(O.c_noise_f32(64, 8, 7, row0=65472), golden["noise2d_rows65472to65536_x8_seed7"])


@pytest.mark.parametrize("seed", [0, 1337])
def test_noise_1d_matches_reference_kernel(golden, seed):
    assert _bits_equal(O.bits_to_f32(O.noise_bits_1d(200, seed)), golden[f"noise1d_200_seed{seed}"])


def test_known_answer_words():
    """Hash words cross-checked between the reference kernel (float view) and the integer restatement."""
    got = O.noise_bits(2, 4, 1337).ravel().tolist()
    assert got == [0x9F42372D, 0x77EA941E, 0xF520803C, 0xFDE87CE4, 0xB0083F71, 0xA8C867E0, 0x9D31EE7B, 0x746CEB95]
    assert O.noise_bits(1, 4, 0).ravel().tolist() == [0x16791E00, 0xC895CB1D, 0xB3601CD9, 0x8E59436E]
    assert O.noise_bits(1, 4, 7, row0=22).ravel().tolist() == [0x5FF3691A, 0x318B3C99, 0xA90FABBD, 0xD8C3EF42]
    f = O.noise_f32(1, 2, 1337).view(np.uint32).ravel().tolist()
    assert f == [0xBF417B92, 0x3F6FD528]


@pytest.mark.parametrize("rows,cols,seed,xor,crc", [(256, 64, 0, 0x4AB3E2E4, 0xD4C4AFCE), (4096, 256, 42, 0x33770230, 0x25E45BE9)])
def test_whole_matrix_checksums(rows, cols, seed, xor, crc):
    B = O.noise_bits(rows, cols, seed)
    assert int(np.bitwise_xor.reduce(B.ravel())) == xor
    assert zlib.crc32(B.tobytes()) == crc
    assert np.array_equal(B, O.c_noise_bits(rows, cols, seed))


def test_numpy_and_c_agree_with_offsets():
    for (r, c, s, r0, c0) in [(37, 19, 5, 1000, 3), (5, 300, -1, 2**31 - 3, 0), (64, 64, 2**31 - 1, 0, 2**20)]:
        assert np.array_equal(O.noise_bits(r, c, s, r0, c0), O.c_noise_bits(r, c, s, r0, c0))


def test_noise_shards_concatenate():
    full = O.noise_bits(64, 16, 7)
    parts = [O.noise_bits(16, 16, 7, row0=16 * r) for r in range(4)]
    assert np.array_equal(np.concatenate(parts), full)


def test_distribution_sanity():
    S = O.noise_f32(20000, 64, 7).astype(np.float64)
    assert abs(S.mean()) < 2e-3
    assert abs(S.var() - 1.0 / 3.0) < 2e-3
    assert S.min() >= -1.0 and S.max() <= 1.0


def test_materialize_fwd_bwd_match_reference_kernels(golden):
    coef = golden["matfwd_coef"]
    np.testing.assert_allclose(O.materialize_fwd(coef, 18, 18, 18, 1, 1337), golden["matfwd_18x18_contig_seed1337"], atol=2e-6)
    np.testing.assert_allclose(O.materialize_fwd(coef, 18, 10, 1, 18, 5), golden["matfwd_18x10_transposed_seed5"], atol=2e-6)
    np.testing.assert_allclose(O.materialize_fwd(coef, 70, 1, 1, 1, 42), golden["matfwd_70x1_seed42"], atol=2e-6)
    np.testing.assert_allclose(O.materialize_bwd(golden["matbwd_dout"], 24, 1337), golden["matbwd_333_M24_seed1337"], atol=1e-5)


def test_fused_random_bias_matches_reference_kernels(golden):
    coef = golden["matfwd_coef"]
    np.testing.assert_allclose(O.materialize_fwd(coef, 18, 18, 18, 1, 1337, 0.25), golden["matfwd_18x18_bias0p25_seed1337"], atol=2e-6)
    np.testing.assert_allclose(O.materialize_fwd(coef, 18, 10, 1, 18, 5, -0.5), golden["matfwd_18x10_transposed_bias_m0p5_seed5"],
                               atol=2e-6)
    # the bias term alone is scale * the reference's 1-D noise
    diff = golden["matfwd_18x18_bias0p25_seed1337"] - golden["matfwd_18x18_contig_seed1337"]
    np.testing.assert_allclose(diff.ravel()[:200], 0.25 * golden["noise1d_200_seed1337"], atol=2e-6)
    np.testing.assert_allclose(O.scale_bias_bwd(golden["matbwd_dout"], 1337), golden["scale_bias_bwd_333_seed1337"][0], atol=1e-5)


def test_embedding_rows_match_reference_kernels(golden):
    idx, coef = golden["embed_idx"], golden["matfwd_coef"]
    np.testing.assert_allclose(O.embed_fwd(idx, coef, 20, 77), golden["embed_fwd_13x20_seed77"], atol=2e-6)
    np.testing.assert_allclose(O.embed_bwd(idx, golden["embed_dout"], 24, 20, 77), golden["embed_bwd_13x20_M24_seed77"], atol=1e-5)
    # a looked-up row is the same row of the materialised (vocab, rowsize) matrix
    full = O.materialize_fwd(coef, 50, 20, 20, 1, 77)
    np.testing.assert_allclose(O.embed_fwd(idx, coef, 20, 77), full[idx], atol=1e-12)


def test_reference_fused_mm_kernel(golden):
    """mat1 @ RT from the reference's rt_mm_grouped_kernel equals mat1 @ materialize(RT)."""
    W = O.materialize_fwd(golden["matfwd_coef"], 40, 36, 36, 1, 9)
    np.testing.assert_allclose(golden["rtmm_mat1"].astype(np.float64) @ W, golden["rtmm_33x40_40x36_seed9"], atol=5e-5)


def test_matrix_coef_layer_reduces_to_reference_form_for_one_column(golden):
    """W = S @ C with C of shape [R, 1] is the reference's materialise of a contiguous [P*Q] tensor."""
    coef = torch.from_numpy(golden["matfwd_coef"]).reshape(24, 1)
    y, _, dc = O.linear_reference(torch.ones(1, 1), coef, 1337, 18 * 18, dy=torch.from_numpy(golden["matbwd_dout"][:324]).reshape(1, 324))
    np.testing.assert_allclose(y.numpy().ravel(), golden["matfwd_18x18_contig_seed1337"].ravel(), atol=2e-6)
    np.testing.assert_allclose(dc.numpy().ravel(), O.materialize_bwd(golden["matbwd_dout"][:324], 24, 1337), atol=1e-9)


def test_c_layer_matches_torch_autograd():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 7, generator=g)
    C = torch.randn(3, 7, generator=g)
    dy = torch.randn(5, 9, generator=g)
    y, dx, dc = O.linear_reference(x, C, 11, 9, row0=4, dy=dy)
    np.testing.assert_allclose(O.c_linear_fwd(x.numpy(), C.numpy(), 9, 11, 4), y.numpy(), atol=1e-12)
    dx2, dc2 = O.c_linear_bwd(dy.numpy(), x.numpy(), C.numpy(), 11, 4)
    np.testing.assert_allclose(dx2, dx.numpy(), atol=1e-12)
    np.testing.assert_allclose(dc2, dc.numpy(), atol=1e-12)


def test_empty_shapes():
    assert O.noise_bits(0, 5, 1).shape == (0, 5)
    assert O.c_noise_bits(3, 0, 1).shape == (3, 0)
    y, _, _ = O.linear_reference(torch.zeros(0, 4), torch.zeros(2, 4), 1, 3)
    assert y.shape == (0, 3)
