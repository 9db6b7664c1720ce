// Batch-1 float32 path:  y = S (C x)  and its backward, as matrix-vector kernels.
//
// One activation row makes every product a matrix-vector product, so the cost is reading C
// (and writing dC) once: 128-bit loads, warp-shuffle reductions, the noise regenerated in
// registers from (seed, row, k).  Same reference slot as the aten.mm override
// (src/rten_cpp/RandumbTensor.py:942-946, 771-791) for a single input row.
#include <atomic>
#include <cooperative_groups.h>
#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace rdb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// sum over the 8 warps of a 256-thread block; the total is returned to thread 0 (red: 8 floats of shared memory)
__device__ __forceinline__ float block_sum_to_thread0(float acc, float *red) {
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float s = 0.0f;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w];
    }
    __syncthreads();          // red may be reused by the caller's next row
    return s;
}

// ---- the four steps, as device functions shared by the stand-alone kernels and the single-launch kernels ----------------
// z[r] = sum_i C[r,i] * x[i], the whole block on one coefficient row
__device__ __forceinline__ void row_dot(float *__restrict__ z, const float *__restrict__ C, const float *__restrict__ x, int64_t K,
                                        int64_t r, float *red) {
    const float *row = C + r * K;
    float acc = 0.0f;
    const bool vec = ((K & 3) == 0) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec) {
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        // four 128-bit loads of the row in flight per thread before the first multiply-add needs one: a K = 4096 row is
        // a single round trip to memory instead of four dependent ones
        const int64_t K4 = K >> 2;
        for (int64_t i0 = threadIdx.x; i0 < K4; i0 += 4 * 256) {
            float4 c[4], v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int64_t i = i0 + u * 256;
                c[u] = i < K4 ? __ldg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[u] = i < K4 ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                acc = fmaf(c[u].x, v[u].x, acc);
                acc = fmaf(c[u].y, v[u].y, acc);
                acc = fmaf(c[u].z, v[u].z, acc);
                acc = fmaf(c[u].w, v[u].w, acc);
            }
        }
    } else {
        for (int64_t i = threadIdx.x; i < K; i += 256) acc = fmaf(row[i], x[i], acc);
    }
    const float s = block_sum_to_thread0(acc, red);
    if (threadIdx.x == 0) z[r] = s;
}

// y[o] = sum_k S[row0+o, k] * z[k], one warp per output row, lanes stride over k.  z may have been written earlier in the
// same launch: read through L2 (ld.global.cg), not through the read-only path.
__device__ __forceinline__ void noise_row_dot(float *__restrict__ y, const float *z, int64_t R, Sq5Lin lin, int64_t o) {
    const int lane = threadIdx.x & 31;
    const uint32_t rowb = lin.base + (uint32_t)o * lin.sn;
    float acc = 0.0f;
    for (int64_t k = lane; k < R; k += 32)
        acc = fmaf(sq5_to_float(sq5_tail(rowb + (uint32_t)k * lin.sk)), __ldcg(z + k), acc);
    acc = warp_sum(acc);
    if (lane == 0) y[o] = acc;
}

// g[k] = sum_o dy[o] * S[row0+o, k], the whole block on one noise column
__device__ __forceinline__ void noise_col_dot(float *__restrict__ g, const float *__restrict__ dy, int64_t N, Sq5Lin lin, int64_t k,
                                              float *red) {
    const uint32_t colb = lin.base + (uint32_t)k * lin.sk;
    float acc = 0.0f;
    for (int64_t o = threadIdx.x; o < N; o += 256)
        acc = fmaf(sq5_to_float(sq5_tail(colb + (uint32_t)o * lin.sn)), __ldg(dy + o), acc);
    const float s = block_sum_to_thread0(acc, red);
    if (threadIdx.x == 0) g[k] = s;
}

// One pass over C for 32 columns (8 lanes x float4 = one 128-byte line per row) and rows [r_lo, r_hi), walked with 32 row
// slots: dc[r,i] = g[r] * x[i] is written, the partial sums of dx[i] = sum_r g[r] * C[r,i] go to out_dx[c] (c = the 32 columns
// of the group).  g may have been written earlier in the same launch (read through L2).
__device__ __forceinline__ void dxdc_group(float *out_dx, float *__restrict__ dc, bool want_dx, const float *g,
                                           const float *__restrict__ x, const float *__restrict__ C, int64_t K, int64_t group,
                                           int64_t r_lo, int64_t r_hi, float (*sums)[33]) {
    const int slot = threadIdx.x >> 3;  // 0..31
    const int l8 = threadIdx.x & 7;     // 0..7
    const int64_t c0 = group * 32 + l8 * 4;
    float ax[4] = {0.f, 0.f, 0.f, 0.f};
    float xv[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = ((K & 3) == 0) && (c0 + 3 < K) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) &&
                     (dc == nullptr || (reinterpret_cast<uintptr_t>(dc) & 15) == 0);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (dc && c0 + j < K) xv[j] = x[c0 + j];
    for (int64_t r = r_lo + slot; r < r_hi; r += 32) {
        const float gr = __ldcg(g + r);
        if (vec) {
            if (want_dx) {
                const float4 c = __ldg(reinterpret_cast<const float4 *>(C + r * K + c0));
                ax[0] = fmaf(gr, c.x, ax[0]);
                ax[1] = fmaf(gr, c.y, ax[1]);
                ax[2] = fmaf(gr, c.z, ax[2]);
                ax[3] = fmaf(gr, c.w, ax[3]);
            }
            if (dc)
                *reinterpret_cast<float4 *>(dc + r * K + c0) = make_float4(gr * xv[0], gr * xv[1], gr * xv[2], gr * xv[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (c0 + j < K) {
                    if (want_dx) ax[j] = fmaf(gr, C[r * K + c0 + j], ax[j]);
                    if (dc) dc[r * K + c0 + j] = gr * xv[j];
                }
            }
        }
    }
    if (!want_dx) return;                 // uniform over the block
#pragma unroll
    for (int j = 0; j < 4; ++j) sums[slot][l8 * 4 + j] = ax[j];
    __syncthreads();
    if (threadIdx.x < 32) {
        float s = 0.0f;
#pragma unroll
        for (int sidx = 0; sidx < 32; ++sidx) s += sums[sidx][threadIdx.x];
        const int64_t c = group * 32 + threadIdx.x;
        if (c < K) out_dx[c] = s;
    }
    __syncthreads();                      // sums may be reused by the caller's next group
}

// ---- stand-alone kernels (one per step; chained with programmatic dependent launch) ------------------------------------
__global__ void __launch_bounds__(256) gemv_cx_kernel(float *__restrict__ z, const float *__restrict__ C,
                                                      const float *__restrict__ x, int64_t K) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    row_dot(z, C, x, K, blockIdx.x, red);
}

__global__ void __launch_bounds__(256) gemv_sz_kernel(float *__restrict__ y, const float *__restrict__ z, int64_t N,
                                                      int64_t R, Sq5Lin lin) {
    const int64_t o = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (o < N) noise_row_dot(y, z, R, lin, o);
}

// Also clears the arrival counters of the kernel that follows (one per 32-column group).
__global__ void __launch_bounds__(256) gemv_stdy_kernel(float *__restrict__ g, const float *__restrict__ dy, int64_t N,
                                                        Sq5Lin lin, unsigned int *__restrict__ counters, int64_t ncounters) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < ncounters; i += (int64_t)gridDim.x * 256) counters[i] = 0u;
    noise_col_dot(g, dy, N, lin, blockIdx.x, red);
}

// Grid (K/32 column groups, row slices): K/32 x slices blocks keep enough bytes in flight for HBM (C read once, dC written
// once).  dx: every block writes its slice's partial sums to `part[slice][K]`; the block of a column group that arrives
// last (one counter per group, cleared by the previous kernel) adds the slices in slice order, so the result does not
// depend on which block that was.
__global__ void __launch_bounds__(256) gemv_dxdc_kernel(float *__restrict__ dx, float *__restrict__ dc,
                                                        const float *__restrict__ g, const float *__restrict__ x,
                                                        const float *__restrict__ C, int64_t K, int64_t R,
                                                        float *__restrict__ part, unsigned int *__restrict__ counters) {
    __shared__ float sums[32][33];
    __shared__ unsigned int arrived;
    const int nsl = gridDim.y, sl = blockIdx.y;
    const int64_t rows_per = (R + nsl - 1) / nsl;
    const int64_t r_lo = sl * rows_per, r_hi = (r_lo + rows_per < R) ? r_lo + rows_per : R;
    pdl_launch_dependents();
    pdl_wait();
    dxdc_group(nsl == 1 ? dx : part + (int64_t)sl * K, dc, dx != nullptr, g, x, C, K, blockIdx.x, r_lo, r_hi, sums);
    if (!dx || nsl == 1) return;
    __threadfence();                       // this block's partial sums are visible before it is counted
    __syncthreads();
    if (threadIdx.x == 0) arrived = atomicAdd(&counters[blockIdx.x], 1u);
    __syncthreads();
    if (arrived != (unsigned)(nsl - 1)) return;
    __threadfence();                       // the last block of the group: the other slices' sums are visible to it
    const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
    if (threadIdx.x < 32 && c < K) {
        float s = 0.0f;
        for (int q = 0; q < nsl; ++q) s += __ldcg(part + (int64_t)q * K + c);
        dx[c] = s;
    }
}

// ---- single-launch kernels (cooperative launch: all blocks resident, grid-wide barriers between the steps) --------------
// A batch-1 step moves a few megabytes, so as four kernels it is mostly latency.  Launched cooperatively, the forward is
// ONE kernel (z = C x, barrier, y = S z) and the backward ONE kernel (g = S^T dy, barrier, the pass over C, barrier, the
// ordered sum of the dx slices).  Same device functions, same summation order: results are bit-identical to the stand-alone
// kernels.  Measured on the 4096 x 4096, d_c = 256 layer, replayed from a CUDA graph with L2 flushed: 28.6 us per
// forward + backward against 18.2 us for the four stand-alone kernels -- a cooperative launch and its grid-wide barriers
// cost more than the kernel boundaries they replace -- so this path is off by default (RDB_OPT_GEMV_FUSED).
__global__ void __launch_bounds__(256) gemv_fwd_coop_kernel(float *__restrict__ y, float *z, const float *__restrict__ C,
                                                            const float *__restrict__ x, int64_t K, int64_t N, int64_t R, Sq5Lin lin) {
    __shared__ float red[8];
    cg::grid_group grid = cg::this_grid();
    for (int64_t r = blockIdx.x; r < R; r += gridDim.x) row_dot(z, C, x, K, r, red);
    grid.sync();
    const int64_t warps = (int64_t)gridDim.x * 8;
    for (int64_t o = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); o < N; o += warps) noise_row_dot(y, z, R, lin, o);
}

__global__ void __launch_bounds__(256) gemv_bwd_coop_kernel(float *__restrict__ dx, float *__restrict__ dc, const float *__restrict__ dy,
                                                            const float *__restrict__ x, const float *__restrict__ C, float *g, float *part,
                                                            int64_t K, int64_t N, int64_t R, int nsl, Sq5Lin lin) {
    __shared__ float red[8];
    __shared__ float sums[32][33];
    cg::grid_group grid = cg::this_grid();
    for (int64_t k = blockIdx.x; k < R; k += gridDim.x) noise_col_dot(g, dy, N, lin, k, red);
    grid.sync();
    const int64_t groups = (K + 31) / 32, rows_per = (R + nsl - 1) / nsl;
    for (int64_t w = blockIdx.x; w < groups * nsl; w += gridDim.x) {
        const int64_t group = w % groups, sl = w / groups;
        const int64_t r_lo = sl * rows_per, r_hi = (r_lo + rows_per < R) ? r_lo + rows_per : R;
        dxdc_group(nsl == 1 ? dx : part + sl * K, dc, dx != nullptr, g, x, C, K, group, r_lo, r_hi, sums);
    }
    if (!dx || nsl == 1) return;          // uniform over the grid
    grid.sync();
    for (int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x; c < K; c += (int64_t)gridDim.x * 256) {
        float s = 0.0f;
        for (int q = 0; q < nsl; ++q) s += __ldcg(part + (int64_t)q * K + c);
        dx[c] = s;
    }
}

// Scratch of rdb_gemv_fwd_static: the R intermediate values z = C x.  It lives in the library image, so
// every GPU that loads the library holds these 64 KB until the process exits.  In host code this name is
// only a stand-in for the symbol; the device address is looked up once per device below.
static __device__ __align__(256) float g_gemv_static_scratch[RDB_GEMV_STATIC_MAX_R];

// Device address of the scratch array on the current device (looked up on first use, then cached).
static int gemv_static_scratch(float **out) {
    static std::mutex mu;
    static float *per_device[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RDB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (!per_device[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_gemv_static_scratch);
        if (e != cudaSuccess) return (int)e;
        per_device[dev] = reinterpret_cast<float *>(p);
    }
    *out = per_device[dev];
    return RDB_OK;
}

// RDB_OPT_GEMV_FUSED (process default; no per-call form: the batch-1 entry points take no options)
static std::atomic<int> g_gemv_fused{0};
void set_gemv_fused(int v) { g_gemv_fused.store(v); }
int get_gemv_fused() { return g_gemv_fused.load(); }

// Largest cooperative grid of a 256-thread kernel on the current device (0: cooperative launch not available); two blocks
// per SM are asked for at most -- enough loads in flight for a few megabytes, and a cheap grid-wide barrier.
template <typename Kern>
static int coop_grid(Kern kern) {
    int dev = 0, coop = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, 0) != cudaSuccess || per_sm <= 0) {
        (void)cudaGetLastError();
        return 0;
    }
    return sms * (per_sm < 2 ? per_sm : 2);
}

template <typename... KArgs, typename... Args>
static int launch_coop(void (*kern)(KArgs...), int grid, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// row slices of the dX / dC kernel: enough blocks to keep HBM busy (about four per SM), at least 32 rows per slice
static int dxdc_slices(int64_t K, int64_t R) {
    const int64_t groups = cdiv64(K, 32);
    int64_t want = cdiv64(148 * 4, groups);
    if (want > R / 32) want = R / 32;
    if (want > 16) want = 16;
    int s = 1;
    while (2 * s <= want) s *= 2;          // a power of two: every slice is a whole number of 32-row passes when R is one too
    return s;
}

}  // namespace rdb

using namespace rdb;

extern "C" size_t rdb_gemv_bwd_workspace_bytes(int64_t K, int64_t N, int64_t R) {
    (void)N;
    if (K <= 0 || R <= 0) return 0;
    // g[R], then per-slice partial sums of dx [slices, K], then one arrival counter per 32-column group
    return (size_t)(align_up((size_t)R * 4, 256) + align_up((size_t)dxdc_slices(K, R) * K * 4, 256) + align_up((size_t)cdiv64(K, 32) * 4, 256));
}

extern "C" int rdb_gemv_fwd(float *y, const float *x, const float *coef, float *workspace, int64_t K, int64_t N,
                            int64_t R, int64_t row0, uint32_t seed, void *stream) {
    if (K < 0 || N < 0 || R < 0) return RDB_ERR_SHAPE;
    if (N == 0) return RDB_OK;
    if (!y || (R > 0 && (!workspace || (K > 0 && (!x || !coef))))) return RDB_ERR_NULL;
    if (R > 0x7fffffffLL || cdiv64(N, 8) > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (R > 0 && K > 0 && g_gemv_fused.load()) {
        static thread_local int grid_dev = -1, grid = 0;
        int dev = 0;
        (void)cudaGetDevice(&dev);
        if (dev != grid_dev) {
            grid = coop_grid(gemv_fwd_coop_kernel);
            grid_dev = dev;
        }
        if (grid > 0)
            return launch_coop(gemv_fwd_coop_kernel, grid, st, y, workspace, coef, x, K, N, R, sq5_lin_rows(seed, (uint32_t)row0, 0));
    }
    if (R > 0) {
        int rc = launch_pdl(gemv_cx_kernel, dim3((unsigned)R), 256, 0, st, workspace, coef, x, K);
        if (rc) return rc;
    }
    return launch_pdl(gemv_sz_kernel, dim3((unsigned)cdiv64(N, 8)), 256, 0, st, y, (const float *)workspace, N, R,
                      sq5_lin_rows(seed, (uint32_t)row0, 0));
}

extern "C" int rdb_gemv_fwd_static(float *y, const float *x, const float *coef, int64_t K, int64_t N, int64_t R, int64_t row0,
                                   uint32_t seed, void *stream) {
    if (K < 0 || N < 0 || R < 0) return RDB_ERR_SHAPE;
    if (R > RDB_GEMV_STATIC_MAX_R) return RDB_ERR_TOO_LARGE;   // the built-in scratch holds at most this many values
    float *scratch = nullptr;
    const int rc = gemv_static_scratch(&scratch);
    if (rc) return rc;
    // Same two kernels as rdb_gemv_fwd.  The first writes scratch[0..R) in full before the second reads
    // it, so nothing left over from an earlier call is ever read and nothing needs clearing.
    return rdb_gemv_fwd(y, x, coef, scratch, K, N, R, row0, seed, stream);
}

extern "C" int rdb_gemv_bwd(float *dx, float *dc, const float *dy, const float *x, const float *coef, float *workspace,
                            int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, void *stream) {
    if (K < 0 || N < 0 || R < 0) return RDB_ERR_SHAPE;
    if (!dx && !dc) return RDB_OK;
    if (K == 0) return RDB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (R == 0) {
        if (dx) {
            cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)K * sizeof(float), st);
            if (e != cudaSuccess) return (int)e;
        }
        return RDB_OK;
    }
    if (!workspace || (N > 0 && !dy) || (dx && !coef) || (dc && !x)) return RDB_ERR_NULL;
    if (R > 0x7fffffffLL || cdiv64(K, 32) > 0x7fffffffLL) return RDB_ERR_TOO_LARGE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return RDB_ERR_WORKSPACE;
    const int slices = dxdc_slices(K, R);
    uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
    float *g = workspace;
    float *part = reinterpret_cast<float *>(ws + align_up((size_t)R * 4, 256));
    unsigned int *counters = reinterpret_cast<unsigned int *>(ws + align_up((size_t)R * 4, 256) + align_up((size_t)slices * K * 4, 256));
    const int64_t groups = cdiv64(K, 32);
    if (g_gemv_fused.load()) {
        static thread_local int grid_dev = -1, grid = 0;
        int dev = 0;
        (void)cudaGetDevice(&dev);
        if (dev != grid_dev) {
            grid = coop_grid(gemv_bwd_coop_kernel);
            grid_dev = dev;
        }
        if (grid > 0)
            return launch_coop(gemv_bwd_coop_kernel, grid, st, dx, dc, dy, x, coef, g, part, K, N, R, slices,
                               sq5_lin_rows(seed, (uint32_t)row0, 0));
    }
    int rc = launch_pdl(gemv_stdy_kernel, dim3((unsigned)R), 256, 0, st, g, dy, N, sq5_lin_rows(seed, (uint32_t)row0, 0), counters,
                        slices > 1 ? groups : (int64_t)0);
    if (rc) return rc;
    return launch_pdl(gemv_dxdc_kernel, dim3((unsigned)groups, (unsigned)slices), 256, 0, st, dx, dc, (const float *)g, x, coef, K, R,
                      part, counters);
}
