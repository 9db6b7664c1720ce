// CUDA-core (SIMT) products with float32 accumulation and arbitrary element strides.
//
// This is the float32 path of the layer (the reference's fused attempt computes in IEEE float32
// with tensor cores disabled: src/rten_cpp/RandumbTensor.py:539, 725) and the any-shape path for
// bf16 problems the tcgen05 kernels do not accept.  The B operand is either read from memory or
// regenerated from the hash, tile by tile, like rt_mm_grouped_kernel's RT operand
// (src/rten_cpp/RandumbTensor.py:648-746).
#include "common.cuh"

namespace rdb {

constexpr int ST_BM = 64, ST_BN = 64, ST_BK = 16, ST_THREADS = 256, ST_PAD = 4;

template <typename TA, typename TB, typename TD, bool GEN>
__global__ void __launch_bounds__(ST_THREADS)
simt_gemm_kernel(TD *__restrict__ d, int64_t d_rs, int64_t d_cs, const TA *__restrict__ a, int64_t a_rs, int64_t a_cs,
                 const TB *__restrict__ b, int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M, int64_t N, int64_t Kc) {
    __shared__ __align__(16) float As[ST_BK][ST_BM + ST_PAD];
    __shared__ __align__(16) float Bs[ST_BK][ST_BN + ST_PAD];
    const int t = threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.y * ST_BM;
    const int64_t n0 = (int64_t)blockIdx.x * ST_BN;
    const int ty = t >> 4, tx = t & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const bool a_kfast = (a_cs == 1);
    const bool b_kfast = GEN ? true : (b_cs == 1);

    for (int64_t k0 = 0; k0 < Kc; k0 += ST_BK) {
#pragma unroll
        for (int i = 0; i < (ST_BM * ST_BK) / ST_THREADS; ++i) {
            const int idx = t + i * ST_THREADS;
            const int kk = a_kfast ? (idx & (ST_BK - 1)) : (idx >> 6);
            const int mm = a_kfast ? (idx >> 4) : (idx & (ST_BM - 1));
            const int64_t gm = m0 + mm, gk = k0 + kk;
            float v = 0.0f;
            if (gm < M && gk < Kc) v = to_f32<TA>(a[gm * a_rs + gk * a_cs]);
            As[kk][mm] = v;
        }
#pragma unroll
        for (int i = 0; i < (ST_BN * ST_BK) / ST_THREADS; ++i) {
            const int idx = t + i * ST_THREADS;
            const int kk = b_kfast ? (idx & (ST_BK - 1)) : (idx >> 6);
            const int nn = b_kfast ? (idx >> 4) : (idx & (ST_BN - 1));
            const int64_t gn = n0 + nn, gk = k0 + kk;
            float v = 0.0f;
            if (gn < N && gk < Kc) {
                if (GEN) {
                    v = sq5_to_float(sq5_tail(lin.base + (uint32_t)gn * lin.sn + (uint32_t)gk * lin.sk));
                } else {
                    v = to_f32<TB>(b[gn * b_rs + gk * b_cs]);
                }
            }
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < ST_BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn < N) d[gm * d_rs + gn * d_cs] = from_f32<TD>(acc[i][j]);
        }
    }
}

template <typename TA, typename TB, typename TD, bool GEN>
static int launch_simt(void *d, int64_t d_rs, int64_t d_cs, const void *a, int64_t a_rs, int64_t a_cs, const void *b,
                       int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M, int64_t N, int64_t Kc, cudaStream_t st) {
    const int64_t gy = cdiv64(M, ST_BM), gx = cdiv64(N, ST_BN);
    if (gy > 65535 || gx > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    dim3 grid((unsigned)gx, (unsigned)gy);
    simt_gemm_kernel<TA, TB, TD, GEN><<<grid, ST_THREADS, 0, st>>>(
        reinterpret_cast<TD *>(d), d_rs, d_cs, reinterpret_cast<const TA *>(a), a_rs, a_cs,
        reinterpret_cast<const TB *>(b), b_rs, b_cs, lin, M, N, Kc);
    return launch_status();
}

template <typename TA, typename TD>
static int dispatch_b(void *d, int64_t d_rs, int64_t d_cs, const void *a, int64_t a_rs, int64_t a_cs, const void *b,
                      int b_dtype, int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M, int64_t N, int64_t Kc,
                      cudaStream_t st) {
    if (!b) return launch_simt<TA, float, TD, true>(d, d_rs, d_cs, a, a_rs, a_cs, nullptr, 0, 0, lin, M, N, Kc, st);
    if (b_dtype == RDB_F32)
        return launch_simt<TA, float, TD, false>(d, d_rs, d_cs, a, a_rs, a_cs, b, b_rs, b_cs, lin, M, N, Kc, st);
    if (b_dtype == RDB_BF16)
        return launch_simt<TA, __nv_bfloat16, TD, false>(d, d_rs, d_cs, a, a_rs, a_cs, b, b_rs, b_cs, lin, M, N, Kc, st);
    return RDB_ERR_DTYPE;
}

template <typename TA>
static int dispatch_d(void *d, int d_dtype, int64_t d_rs, int64_t d_cs, const void *a, int64_t a_rs, int64_t a_cs,
                      const void *b, int b_dtype, int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M, int64_t N,
                      int64_t Kc, cudaStream_t st) {
    if (d_dtype == RDB_F32)
        return dispatch_b<TA, float>(d, d_rs, d_cs, a, a_rs, a_cs, b, b_dtype, b_rs, b_cs, lin, M, N, Kc, st);
    if (d_dtype == RDB_BF16)
        return dispatch_b<TA, __nv_bfloat16>(d, d_rs, d_cs, a, a_rs, a_cs, b, b_dtype, b_rs, b_cs, lin, M, N, Kc, st);
    return RDB_ERR_DTYPE;
}

int simt_gemm(void *d, int d_dtype, int64_t d_rs, int64_t d_cs, const void *a, int a_dtype, int64_t a_rs, int64_t a_cs,
              const void *b, int b_dtype, int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M, int64_t N, int64_t Kc,
              cudaStream_t st) {
    if (M == 0 || N == 0) return RDB_OK;
    if (a_dtype == RDB_F32)
        return dispatch_d<float>(d, d_dtype, d_rs, d_cs, a, a_rs, a_cs, b, b_dtype, b_rs, b_cs, lin, M, N, Kc, st);
    if (a_dtype == RDB_BF16)
        return dispatch_d<__nv_bfloat16>(d, d_dtype, d_rs, d_cs, a, a_rs, a_cs, b, b_dtype, b_rs, b_cs, lin, M, N, Kc, st);
    return RDB_ERR_DTYPE;
}

}  // namespace rdb
