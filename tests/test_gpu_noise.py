"""Generator parity on the GPU, through the C ABI: hash words bit-exact against the oracle and against
the reference kernel's own outputs."""
import zlib

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from randumb_b200 import kernels
    assert torch.cuda.is_available()
    return kernels


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("rows,cols,seed,row0,col0", [
    (48, 20, 1337, 0, 0), (300, 130, 42, 0, 0), (64, 8, 7, 65472, 0), (1000, 257, -5, 123, 77),
    (1, 1, 0, 0, 0), (3, 5, 2**31 - 1, 2**31 - 2, 9), (17, 4099, 11, 5, 0)])
def test_bits_f32_bf16_bit_exact(K, rows, cols, seed, row0, col0):
    assert np.array_equal(_u32(K.noise_bits(rows, cols, seed, row0, col0)), O.noise_bits(rows, cols, seed, row0, col0))
    f = K.noise(rows, cols, seed, row0, col0).cpu().numpy()
    assert np.array_equal(f.view(np.uint32), O.noise_f32(rows, cols, seed, row0, col0).view(np.uint32))
    h = K.noise(rows, cols, seed, row0, col0, dtype=torch.bfloat16).cpu()
    assert torch.equal(h, O.noise_bf16(rows, cols, seed, row0, col0))


def test_against_reference_kernel_outputs(K, golden):
    for seed in (0, 7, 42, 1337, -5):
        got = K.noise(48, 20, seed).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), golden[f"noise2d_48x20_seed{seed}"].view(np.uint32))
    got = K.noise(64, 8, 7, row0=65472).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), golden["noise2d_rows65472to65536_x8_seed7"].view(np.uint32))
    got = K.noise_1d(200, 1337).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), golden["noise1d_200_seed1337"].view(np.uint32))


@pytest.mark.parametrize("rows,cols,seed,xor,crc", [
    (256, 64, 0, 0x4AB3E2E4, 0xD4C4AFCE), (4096, 256, 42, 0x33770230, 0x25E45BE9),
    (16384, 1024, 42, 0xC12CDCA8, 0xE19DAF48), (65536, 2048, 7, 0xE1BD012A, 0x4AACA585)])
def test_full_size_checksums(K, rows, cols, seed, xor, crc):
    """Whole noise matrices of the benchmark configurations: XOR of all words and CRC-32."""
    B = _u32(K.noise_bits(rows, cols, seed))
    assert int(np.bitwise_xor.reduce(B.ravel())) == xor
    assert zlib.crc32(B.tobytes()) == crc


def test_row_shards_concatenate_to_the_whole(K):
    full = K.noise_bits(4096, 64, 7)
    for world in (2, 4, 8):
        n = 4096 // world
        parts = [K.noise_bits(n, 64, 7, row0=r * n) for r in range(world)]
        assert torch.equal(torch.cat(parts), full)


def test_leading_dimension_and_empty(K):
    from randumb_b200 import _lib
    out = torch.full((5, 12), -1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().rdb_noise_bits(out.data_ptr(), 5, 7, 12, 3, 2, 9, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = out.cpu().numpy()
    assert np.array_equal(got[:, :7].view(np.uint32), O.noise_bits(5, 7, 9, 3, 2))
    assert (got[:, 7:] == -1).all()                       # padding columns untouched
    assert K.noise_bits(0, 16, 1).shape == (0, 16)
    assert K.noise(16, 0, 1).shape == (16, 0)
