// Shared host/device helpers for the randumb_b200 kernels.
#pragma once
#include <cstdint>
#include <cstddef>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include "../../include/randumb_b200.h"
#include "sq5.cuh"

namespace rdb {

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? RDB_OK : static_cast<int>(e);
}

inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline size_t dtype_size(int dtype) { return dtype == RDB_BF16 ? 2 : 4; }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- programmatic dependent launch -------------------------------------------------------------------
// The products of one layer call are a chain of kernels, each a few to a few hundred microseconds long; the gap between one
// kernel's last block and the next kernel's first block (a few microseconds) is paid once per link.  The kernels of this
// library are launched with the programmatic-serialization attribute: their blocks may become resident -- and run their
// prologue: barrier initialisation, TMEM allocation, tensor-map prefetch -- while the previous kernel of the stream is
// still running, wait in pdl_wait() until that kernel has completed and its writes are visible, and let the launch of the
// kernel after them proceed with pdl_launch_dependents().  Nothing a predecessor may have written is touched before
// pdl_wait().  (Both are no-ops for a launch without the attribute; the attribute is captured into CUDA graphs.)
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// <<<grid, block, smem, stream>>> with programmatic stream serialization allowed
template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kern)(KArgs...), dim3 grid, int block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}
#endif

// ---- implemented in simt.cu ------------------------------------------------------------------
// D(m,n) = sum_k A(m,k) * B(n,k); element (i,j) of an operand lives at base[i*rs + j*cs].
// When b == nullptr the B operand is generated: B(n,k) = value(lin.base + n*lin.sn + k*lin.sk).
int simt_gemm(void *d, int d_dtype, int64_t d_rs, int64_t d_cs, const void *a, int a_dtype, int64_t a_rs,
              int64_t a_cs, const void *b, int b_dtype, int64_t b_rs, int64_t b_cs, Sq5Lin lin, int64_t M,
              int64_t N, int64_t Kc, cudaStream_t stream);

// Tuning switches of one call, resolved from the caller's rdb_call_options (fields < 0 take the process default
// that rdb_set_option holds).  Passed by value down to the launch: no launch reads process state.
struct CallOpts {
    int noise_tile;    // RDB_OPT_NOISE_TILE
    int dense_pair;    // RDB_OPT_DENSE_PAIR
    int stage_noise;   // RDB_OPT_STAGE_NOISE
    int reserve_sms;   // RDB_OPT_RESERVE_SMS
    int fill_overlap;  // RDB_OPT_FILL_OVERLAP
    int grads_beside;  // RDB_OPT_GRADS_BESIDE
};

// ---- implemented in gemv.cu ---------------------------------------------------------------------
void set_gemv_fused(int v);
int get_gemv_fused();

// ---- implemented in umma_gemm.cu -------------------------------------------------------------
void set_profile_buffer(void *p, size_t bytes);
bool umma_shape_ok_noise(int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, const void *a, const void *d);
int umma_gemm_noise(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, Sq5Lin lin,
                    int32_t *status, cudaStream_t stream, const CallOpts &o);
bool umma_shape_ok_dense(int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int d_dtype,
                         int a_kmajor, int b_kmajor, const void *a, const void *b, const void *d);
int dense_split_k_slices(int64_t M, int64_t N, int64_t Kc);
int umma_gemm_dense_split_k(void *d, const void *a, const void *b, float *partials, int split, int64_t M, int64_t N,
                            int64_t Kc, int64_t lda, int64_t ldb, int d_dtype, int a_kmajor, int b_kmajor, int32_t *status,
                            cudaStream_t stream, const CallOpts &o);
int umma_gemm_dense(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda,
                    int64_t ldb, int64_t ldd, int d_dtype, int a_kmajor, int b_kmajor, int32_t *status,
                    cudaStream_t stream, const CallOpts &o);

bool dense_beside_plan(int64_t M1, int64_t N1, int64_t Kc1, int64_t M2, int64_t N2, int64_t Kc2, int reserve_sms, bool always,
                       int *pairs1, int *pairs2);
int umma_gemm_dense_on_pairs(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb,
                             int64_t ldd, int a_kmajor, int b_kmajor, int pairs, int32_t *status, cudaStream_t stream);

int umma_gemm_dense_scatter(void *const *dsts, int ndst, int64_t rows_per_dst, const void *a, const void *b, int64_t M, int64_t N,
                            int64_t Kc, int64_t lda, int64_t ldb, int b_kmajor, int32_t *status, cudaStream_t stream,
                            const CallOpts &o);

}  // namespace rdb
