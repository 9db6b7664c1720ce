// Squirrel5 noise generator, device side.
//
// Restates the hash of the reference (src/rten_cpp/csrc/cuda/rten.cu:13-48 and
// src/rten_cpp/RandumbTensor.py:130-164):
//   pos  = uint32(PRIME*row + col)
//   b    = pos*N1 + seed;  b ^= b>>9;  b += N2;  b ^= b>>11;  b *= N3;  b ^= b>>13;
//   b   += N4;  b ^= b>>15;  b *= N5;  b ^= b>>17
//   value = float(int32(b)) * 2^-31
//
// The first two steps are linear in (row, col) modulo 2^32, so a tile generator
// keeps   b0 = base + row*SN + col*SK   with  SN = PRIME*N1, SK = N1 (or swapped
// for the transposed walk) and only pays one add per element before the mixing tail.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace rdb {

constexpr uint32_t SQ5_N1 = 0xd2a80a3fu;
constexpr uint32_t SQ5_N2 = 0xa884f197u;
constexpr uint32_t SQ5_N3 = 0x6C736F4Bu;
constexpr uint32_t SQ5_N4 = 0xB79F3ABBu;
constexpr uint32_t SQ5_N5 = 0x1b56c4f5u;
constexpr uint32_t SQ5_PRIME = 198491317u;

// Linearised hash front end: b0(row, col) = lin.base + row*lin.sn + col*lin.sk  (mod 2^32)
// equals (PRIME*row + col)*N1 + seed for the natural orientation.
struct Sq5Lin {
    uint32_t base;  // seed (+ any constant offset already multiplied by N1)
    uint32_t sn;    // increment of b0 per step of the first tile index
    uint32_t sk;    // increment of b0 per step of the second tile index
};

// Natural orientation: first index walks noise rows (starting at row0), second walks noise columns.
__host__ __device__ inline Sq5Lin sq5_lin_rows(uint32_t seed, uint32_t row0, uint32_t col0) {
    Sq5Lin l;
    l.sn = SQ5_PRIME * SQ5_N1;
    l.sk = SQ5_N1;
    l.base = seed + row0 * l.sn + col0 * l.sk;
    return l;
}
// Transposed walk: first index walks noise columns, second walks noise rows (starting at row0).
__host__ __device__ inline Sq5Lin sq5_lin_cols(uint32_t seed, uint32_t row0, uint32_t col0) {
    Sq5Lin l;
    l.sn = SQ5_N1;
    l.sk = SQ5_PRIME * SQ5_N1;
    l.base = seed + row0 * l.sk + col0 * l.sn;
    return l;
}

// Mixing tail applied to b0 = pos*N1 + seed.
__host__ __device__ __forceinline__ uint32_t sq5_tail(uint32_t b) {
    b ^= b >> 9;
    b += SQ5_N2;
    b ^= b >> 11;
    b *= SQ5_N3;
    b ^= b >> 13;
    b += SQ5_N4;
    b ^= b >> 15;
    b *= SQ5_N5;
    b ^= b >> 17;
    return b;
}

__host__ __device__ __forceinline__ uint32_t sq5_bits(uint32_t row, uint32_t col, uint32_t seed) {
    return sq5_tail((SQ5_PRIME * row + col) * SQ5_N1 + seed);
}

// float(int32(bits)) * 2^-31.  (The reference multiplies by float(1/0x7FFFFFFF), which is exactly 2^-31.)
__host__ __device__ __forceinline__ float sq5_to_float(uint32_t bits) {
    return static_cast<float>(static_cast<int32_t>(bits)) * 4.6566128730773926e-10f;
}

// Two hash words -> two bf16 noise values in one 32-bit word (low half first).  bf16 noise is defined as the float32
// value float(int32(bits)) * 2^-31 rounded to nearest even; scaling by a power of two commutes with that rounding (no
// value here is subnormal or overflows in bf16), so the pair is rounded first and scaled with ONE packed multiply -- one
// instruction less per pair on the pipes the hash keeps busy.
__device__ __forceinline__ uint32_t sq5_pack_bf16x2(uint32_t bits0, uint32_t bits1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(static_cast<float>(static_cast<int32_t>(bits0)),
                                             static_cast<float>(static_cast<int32_t>(bits1)));
    h = __hmul2(h, __float2bfloat162_rn(4.6566128730773926e-10f));
    return *reinterpret_cast<uint32_t *>(&h);
}

}  // namespace rdb
