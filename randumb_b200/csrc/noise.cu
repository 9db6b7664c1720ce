// Explicit noise matrices and the reference's 1-D-coefficient materialise kernels (CUDA cores).
//
// Reference behaviour restated here (paths inside the reference project):
//   explicit noise matrix      src/rten_cpp/RandumbTensor.py:78-105, csrc/cuda/rten.cu:50-71
//   1-D noise                  src/rten_cpp/RandumbTensor.py:204-232
//   materialise forward        src/rten_cpp/RandumbTensor.py:235-290, csrc/cuda/rten.cu:74-110
//   materialise backward       src/rten_cpp/RandumbTensor.py:304-359 (atomics there; a fixed
//                              two-pass reduction order here so results repeat run to run)
#include "common.cuh"

namespace rdb {

// mode 0: uint32 words, 1: float32, 2: bf16
template <int MODE>
__global__ void noise_kernel(void *__restrict__ out, int64_t rows, int64_t cols, int64_t ld, Sq5Lin lin) {
    const int64_t cgroups = (cols + 3) >> 2;
    const int64_t total = rows * cgroups;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / cgroups;
        const int64_t c0 = (idx - r * cgroups) << 2;
        const uint32_t b0 = lin.base + (uint32_t)r * lin.sn + (uint32_t)c0 * lin.sk;
        uint32_t bits[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) bits[j] = sq5_tail(b0 + (uint32_t)j * lin.sk);
        const int64_t off = r * ld + c0;
        const int nvalid = (int)((cols - c0) < 4 ? (cols - c0) : 4);
        if (MODE == 0) {
            uint32_t *o = reinterpret_cast<uint32_t *>(out) + off;
            if (nvalid == 4 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
                *reinterpret_cast<uint4 *>(o) = make_uint4(bits[0], bits[1], bits[2], bits[3]);
            } else {
                for (int j = 0; j < nvalid; ++j) o[j] = bits[j];
            }
        } else if (MODE == 1) {
            float *o = reinterpret_cast<float *>(out) + off;
            float f[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = sq5_to_float(bits[j]);
            if (nvalid == 4 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
                *reinterpret_cast<float4 *>(o) = make_float4(f[0], f[1], f[2], f[3]);
            } else {
                for (int j = 0; j < nvalid; ++j) o[j] = f[j];
            }
        } else {
            __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(out) + off;
            __nv_bfloat16 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __float2bfloat16_rn(sq5_to_float(bits[j]));
            if (nvalid == 4 && ((reinterpret_cast<uintptr_t>(o) & 7) == 0)) {
                uint2 v;
                v.x = (uint32_t)__bfloat16_as_ushort(h[0]) | ((uint32_t)__bfloat16_as_ushort(h[1]) << 16);
                v.y = (uint32_t)__bfloat16_as_ushort(h[2]) | ((uint32_t)__bfloat16_as_ushort(h[3]) << 16);
                *reinterpret_cast<uint2 *>(o) = v;
            } else {
                for (int j = 0; j < nvalid; ++j) o[j] = h[j];
            }
        }
    }
}

// bf16 fast path (the staged noise operand of the tensor-core products): cols a multiple of 8, 16-byte aligned rows,
// fewer than 2^31 groups.  One thread hashes 8 consecutive elements of a row and writes them with one 16-byte store;
// all index arithmetic is 32-bit.
__global__ void __launch_bounds__(256) noise_bf16x8_kernel(uint4 *__restrict__ out, uint32_t total, uint32_t cgroups,
                                                           uint32_t ld_groups, Sq5Lin lin) {
    pdl_launch_dependents();
    pdl_wait();
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t r = idx / cgroups;
        const uint32_t cg = idx - r * cgroups;
        const uint32_t b0 = lin.base + r * lin.sn + (cg << 3) * lin.sk;
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            p[j] = sq5_pack_bf16x2(sq5_tail(b0 + (uint32_t)(2 * j) * lin.sk), sq5_tail(b0 + (uint32_t)(2 * j + 1) * lin.sk));
        }
        out[(size_t)r * ld_groups + cg] = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

// Same for rows whose length is a multiple of 1024: one warp hashes a 1024-element row segment, each lane four groups of
// 8 elements 256 apart (every store instruction of the warp writes 512 contiguous bytes), so the row/column split costs
// one division per 32 hashes.
__global__ void __launch_bounds__(256) noise_bf16_seg_kernel(uint4 *__restrict__ out, uint32_t total_segs, uint32_t segs_per_row,
                                                             uint32_t ld_groups, Sq5Lin lin) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
    pdl_launch_dependents();
    pdl_wait();
    for (uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total_segs; w += warps) {
        const uint32_t r = w / segs_per_row;
        const uint32_t sg = w - r * segs_per_row;
        const uint32_t b0 = lin.base + r * lin.sn + ((sg << 10) + (lane << 3)) * lin.sk;
        uint4 *dst = out + (size_t)r * ld_groups + (sg << 7) + lane;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t b = b0 + (uint32_t)(c * 256) * lin.sk;
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                p[j] = sq5_pack_bf16x2(sq5_tail(b + (uint32_t)(2 * j) * lin.sk), sq5_tail(b + (uint32_t)(2 * j + 1) * lin.sk));
            }
            dst[c * 32] = make_uint4(p[0], p[1], p[2], p[3]);
        }
    }
}

__global__ void noise_1d_kernel(float *__restrict__ out, int64_t n, uint32_t idx0, uint32_t seed) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = sq5_to_float(sq5_tail((idx0 + (uint32_t)i) * SQ5_N1 + seed));
}

static int grid_for(int64_t work_items, int block) {
    int64_t g = cdiv64(work_items, block);
    const int64_t cap = 148 * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

template <int MODE>
static int launch_noise(void *out, int64_t rows, int64_t cols, int64_t ld, int64_t row0, int64_t col0, uint32_t seed,
                        cudaStream_t st) {
    if (rows == 0 || cols == 0) return RDB_OK;
    Sq5Lin lin = sq5_lin_rows(seed, (uint32_t)row0, (uint32_t)col0);
    if (MODE == 2 && (cols & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
        rows * (cols >> 3) < (1LL << 31)) {
        if ((cols & 1023) == 0) {
            const uint32_t total_segs = (uint32_t)(rows * (cols >> 10));
            const int64_t want = cdiv64(total_segs, 8);        // eight warps per block, one segment per warp and pass
            const int grid = (int)(want < 148 * 8 ? (want < 1 ? 1 : want) : 148 * 8);
            return launch_pdl(noise_bf16_seg_kernel, dim3(grid), 256, 0, st, reinterpret_cast<uint4 *>(out), total_segs,
                              (uint32_t)(cols >> 10), (uint32_t)(ld >> 3), lin);
        }
        const uint32_t total = (uint32_t)(rows * (cols >> 3));
        const int64_t want = cdiv64(total, 256 * 4);           // about four groups (32 elements) per thread
        const int grid = (int)(want < 148 * 8 ? (want < 1 ? 1 : want) : 148 * 8);
        return launch_pdl(noise_bf16x8_kernel, dim3(grid), 256, 0, st, reinterpret_cast<uint4 *>(out), total, (uint32_t)(cols >> 3),
                          (uint32_t)(ld >> 3), lin);
    }
    const int64_t items = rows * ((cols + 3) >> 2);
    noise_kernel<MODE><<<grid_for(items, 256), 256, 0, st>>>(out, rows, cols, ld, lin);
    return launch_status();
}

// ---- materialise forward (1-D coefficient vector) ---------------------------------------------
// Element n of the output is a dot product of noise row rowsel(n) with the coefficient vector.  Two row
// selections share the kernels: a strided view of a virtual tensor (sq(n), the reference's Form R) and rows of
// a virtual (vocab, rowsize) embedding matrix picked by an index vector.
constexpr int MAT_CHUNK = 1024;

struct RowSel {
    const int64_t *idx;   // null: strided view; else embedding rows
    int64_t Q, stride_P, stride_Q;   // strided view
    int64_t rowsize, n_idx;          // embedding
};

__device__ __forceinline__ uint32_t noise_row_of(const RowSel &rs, int64_t n) {
    if (rs.idx) {
        const int64_t i = n / rs.rowsize;
        return (uint32_t)(rs.idx[i] * rs.rowsize + (n - i * rs.rowsize));
    }
    return (uint32_t)((n % rs.Q) * rs.stride_Q + (n / rs.Q) * rs.stride_P);
}

__global__ void materialize_fwd_kernel(float *__restrict__ out, const float *__restrict__ coef, int64_t M, int64_t Nel,
                                       RowSel rs, int64_t ld_out, const float *__restrict__ scale_bias, uint32_t seed) {
    __shared__ float coef_s[MAT_CHUNK];
    const int64_t n = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const bool live = n < Nel;
    uint32_t row = 0, rowpos = 0;
    if (live) {
        row = noise_row_of(rs, n);
        rowpos = (row * SQ5_PRIME) * SQ5_N1 + seed;
    }
    float acc = 0.0f;
    for (int64_t m0 = 0; m0 < M; m0 += MAT_CHUNK) {
        const int len = (int)((M - m0) < MAT_CHUNK ? (M - m0) : MAT_CHUNK);
        __syncthreads();
        for (int i = threadIdx.x; i < len; i += blockDim.x) coef_s[i] = coef[m0 + i];
        __syncthreads();
        if (live) {
            uint32_t b0 = rowpos + (uint32_t)m0 * SQ5_N1;
            for (int m = 0; m < len; ++m) {
                acc = fmaf(sq5_to_float(sq5_tail(b0)), coef_s[m], acc);
                b0 += SQ5_N1;
            }
        }
    }
    if (!live) return;
    // fused random bias: scale * 1-D noise of the same row index (no prime multiply)
    if (scale_bias) acc = fmaf(scale_bias[0], sq5_to_float(sq5_tail(row * SQ5_N1 + seed)), acc);
    if (rs.idx) {
        const int64_t i = n / rs.rowsize;
        out[i * ld_out + (n - i * rs.rowsize)] = acc;
    } else {
        out[n] = acc;
    }
}

// ---- materialise backward: partial[split][m] then ordered sum over splits ----------------------
constexpr int BWD_MB = 8;       // coefficient columns per block
constexpr int BWD_THREADS = 256;
constexpr int64_t BWD_SPAN = 8192;  // dout elements per split

__global__ void materialize_bwd_partial_kernel(float *__restrict__ partial, const float *__restrict__ dout, int64_t Nel,
                                               int64_t M, RowSel rs, uint32_t seed) {
    __shared__ float red[BWD_MB][BWD_THREADS];
    const int64_t m0 = (int64_t)blockIdx.x * BWD_MB;
    const int64_t split = blockIdx.y;
    const int64_t n_lo = split * BWD_SPAN;
    const int64_t n_hi = (n_lo + BWD_SPAN) < Nel ? (n_lo + BWD_SPAN) : Nel;
    float acc[BWD_MB];
#pragma unroll
    for (int j = 0; j < BWD_MB; ++j) acc[j] = 0.0f;
    for (int64_t n = n_lo + threadIdx.x; n < n_hi; n += BWD_THREADS) {
        const float d = dout[n];
        const uint32_t row = rs.idx ? noise_row_of(rs, n) : (uint32_t)n;   // the gradient arrives contiguous
        const uint32_t b0 = (row * SQ5_PRIME + (uint32_t)m0) * SQ5_N1 + seed;
#pragma unroll
        for (int j = 0; j < BWD_MB; ++j) acc[j] = fmaf(sq5_to_float(sq5_tail(b0 + (uint32_t)j * SQ5_N1)), d, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < BWD_MB; ++j) red[j][threadIdx.x] = acc[j];
    __syncthreads();
    for (int s = BWD_THREADS / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
#pragma unroll
            for (int j = 0; j < BWD_MB; ++j) red[j][threadIdx.x] += red[j][threadIdx.x + s];
        }
        __syncthreads();
    }
    if (threadIdx.x < BWD_MB && m0 + threadIdx.x < M) partial[split * M + m0 + threadIdx.x] = red[threadIdx.x][0];
}

__global__ void materialize_bwd_final_kernel(float *__restrict__ dcoef, const float *__restrict__ partial, int64_t M,
                                             int64_t nsplit) {
    const int64_t m = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (m >= M) return;
    float acc = 0.0f;
    for (int64_t s = 0; s < nsplit; ++s) acc += partial[s * M + m];
    dcoef[m] = acc;
}

// ---- gradient of the random-bias scale: sum_n dout[n] * noise1d(n) -----------------------------
__global__ void scale_bias_bwd_partial_kernel(float *__restrict__ partial, const float *__restrict__ dout, int64_t Nel,
                                              uint32_t seed) {
    __shared__ float red[BWD_THREADS];
    const int64_t n_lo = (int64_t)blockIdx.x * BWD_SPAN;
    const int64_t n_hi = (n_lo + BWD_SPAN) < Nel ? (n_lo + BWD_SPAN) : Nel;
    float acc = 0.0f;
    for (int64_t n = n_lo + threadIdx.x; n < n_hi; n += BWD_THREADS)
        acc = fmaf(sq5_to_float(sq5_tail((uint32_t)n * SQ5_N1 + seed)), dout[n], acc);
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int s = BWD_THREADS / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

__global__ void scale_bias_bwd_final_kernel(float *__restrict__ dbias, const float *__restrict__ partial, int64_t nsplit) {
    __shared__ float red[BWD_THREADS];
    float acc = 0.0f;
    for (int64_t s = threadIdx.x; s < nsplit; s += BWD_THREADS) acc += partial[s];
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int s = BWD_THREADS / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[0] = red[0];
}

static int launch_materialize_bwd(float *dcoef, const float *dout, float *workspace, int64_t Nel, int64_t M,
                                  const RowSel &rs, uint32_t seed, cudaStream_t st) {
    if (Nel == 0) {
        cudaError_t e = cudaMemsetAsync(dcoef, 0, (size_t)M * sizeof(float), st);
        return e == cudaSuccess ? RDB_OK : (int)e;
    }
    if (!dout || !workspace) return RDB_ERR_NULL;
    const int64_t nsplit = cdiv64(Nel, BWD_SPAN);
    if (nsplit > 65535) return RDB_ERR_TOO_LARGE;
    dim3 grid((unsigned)cdiv64(M, BWD_MB), (unsigned)nsplit);
    materialize_bwd_partial_kernel<<<grid, BWD_THREADS, 0, st>>>(workspace, dout, Nel, M, rs, seed);
    int rc = launch_status();
    if (rc) return rc;
    materialize_bwd_final_kernel<<<(unsigned)cdiv64(M, 128), 128, 0, st>>>(dcoef, workspace, M, nsplit);
    return launch_status();
}

}  // namespace rdb

using namespace rdb;

extern "C" int rdb_noise_bits(uint32_t *out, int64_t rows, int64_t cols, int64_t ld, int64_t row0, int64_t col0,
                              uint32_t seed, void *stream) {
    if (rows < 0 || cols < 0 || ld < cols) return RDB_ERR_SHAPE;
    if (rows > 0 && cols > 0 && !out) return RDB_ERR_NULL;
    return launch_noise<0>(out, rows, cols, ld, row0, col0, seed, (cudaStream_t)stream);
}

extern "C" int rdb_noise(void *out, int dtype, int64_t rows, int64_t cols, int64_t ld, int64_t row0, int64_t col0,
                         uint32_t seed, void *stream) {
    if (rows < 0 || cols < 0 || ld < cols) return RDB_ERR_SHAPE;
    if (rows > 0 && cols > 0 && !out) return RDB_ERR_NULL;
    if (dtype == RDB_F32) return launch_noise<1>(out, rows, cols, ld, row0, col0, seed, (cudaStream_t)stream);
    if (dtype == RDB_BF16) return launch_noise<2>(out, rows, cols, ld, row0, col0, seed, (cudaStream_t)stream);
    return RDB_ERR_DTYPE;
}

extern "C" int rdb_noise_1d(float *out, int64_t n, int64_t idx0, uint32_t seed, void *stream) {
    if (n < 0) return RDB_ERR_SHAPE;
    if (n == 0) return RDB_OK;
    if (!out) return RDB_ERR_NULL;
    noise_1d_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(out, n, (uint32_t)idx0, seed);
    return launch_status();
}

extern "C" int rdb_materialize_fwd(float *out, const float *coef, int64_t M, int64_t P, int64_t Q, int64_t stride_P,
                                   int64_t stride_Q, const float *scale_bias, uint32_t seed, void *stream) {
    if (M < 0 || P < 0 || Q < 0) return RDB_ERR_SHAPE;
    const int64_t Nel = P * Q;
    if (Nel == 0) return RDB_OK;
    if (!out || (M > 0 && !coef)) return RDB_ERR_NULL;
    if (cdiv64(Nel, 128) > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    RowSel rs{nullptr, Q, stride_P, stride_Q, 0, 0};
    materialize_fwd_kernel<<<(unsigned)cdiv64(Nel, 128), 128, 0, (cudaStream_t)stream>>>(out, coef, M, Nel, rs, 0,
                                                                                       scale_bias, seed);
    return launch_status();
}

extern "C" size_t rdb_materialize_bwd_workspace_bytes(int64_t Nel, int64_t M) {
    if (Nel <= 0 || M <= 0) return 0;
    return (size_t)cdiv64(Nel, BWD_SPAN) * (size_t)M * sizeof(float);
}

extern "C" int rdb_materialize_bwd(float *dcoef, const float *dout, float *workspace, int64_t Nel, int64_t M,
                                   uint32_t seed, void *stream) {
    if (Nel < 0 || M < 0) return RDB_ERR_SHAPE;
    if (M == 0) return RDB_OK;
    if (!dcoef) return RDB_ERR_NULL;
    RowSel rs{nullptr, 1, 1, 1, 0, 0};
    return launch_materialize_bwd(dcoef, dout, workspace, Nel, M, rs, seed, (cudaStream_t)stream);
}

extern "C" size_t rdb_scale_bias_bwd_workspace_bytes(int64_t Nel) {
    if (Nel <= 0) return 0;
    return (size_t)cdiv64(Nel, BWD_SPAN) * sizeof(float);
}

extern "C" int rdb_scale_bias_bwd(float *dbias, const float *dout, float *workspace, int64_t Nel, uint32_t seed,
                                  void *stream) {
    if (Nel < 0) return RDB_ERR_SHAPE;
    if (!dbias) return RDB_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (Nel == 0) {
        cudaError_t e = cudaMemsetAsync(dbias, 0, sizeof(float), st);
        return e == cudaSuccess ? RDB_OK : (int)e;
    }
    if (!dout || !workspace) return RDB_ERR_NULL;
    const int64_t nsplit = cdiv64(Nel, BWD_SPAN);
    if (nsplit > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    scale_bias_bwd_partial_kernel<<<(unsigned)nsplit, BWD_THREADS, 0, st>>>(workspace, dout, Nel, seed);
    int rc = launch_status();
    if (rc) return rc;
    scale_bias_bwd_final_kernel<<<1, BWD_THREADS, 0, st>>>(dbias, workspace, nsplit);
    return launch_status();
}

extern "C" int rdb_embed_fwd(float *out, const int64_t *idx, const float *coef, int64_t n_idx, int64_t rowsize, int64_t M,
                             int64_t ld_out, uint32_t seed, void *stream) {
    if (n_idx < 0 || rowsize < 0 || M < 0 || ld_out < rowsize) return RDB_ERR_SHAPE;
    const int64_t Nel = n_idx * rowsize;
    if (Nel == 0) return RDB_OK;
    if (!out || !idx || (M > 0 && !coef)) return RDB_ERR_NULL;
    if (cdiv64(Nel, 128) > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    RowSel rs{idx, 1, 1, 1, rowsize, n_idx};
    materialize_fwd_kernel<<<(unsigned)cdiv64(Nel, 128), 128, 0, (cudaStream_t)stream>>>(out, coef, M, Nel, rs, ld_out,
                                                                                       nullptr, seed);
    return launch_status();
}

extern "C" int rdb_embed_bwd(float *dcoef, const float *dout, const int64_t *idx, float *workspace, int64_t n_idx,
                             int64_t rowsize, int64_t M, uint32_t seed, void *stream) {
    if (n_idx < 0 || rowsize < 0 || M < 0) return RDB_ERR_SHAPE;
    if (M == 0) return RDB_OK;
    if (!dcoef) return RDB_ERR_NULL;
    const int64_t Nel = n_idx * rowsize;
    if (Nel > 0 && !idx) return RDB_ERR_NULL;
    RowSel rs{idx, 1, 1, 1, rowsize, n_idx};
    return launch_materialize_bwd(dcoef, dout, workspace, Nel, M, rs, seed, (cudaStream_t)stream);
}
