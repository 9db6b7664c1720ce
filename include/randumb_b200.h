/*
 * randumb_b200 -- C ABI of the B200 (sm_100a) pseudorandom-weight linear layer.
 *
 * The layer's weight is never stored:  W[o,i] = sum_k S[o,k] * C[k,i]  where
 *   S[o,k] = squirrel5(uint32(198491317*o + k), seed)  in [-1,1]   (N x R, regenerated on the fly)
 *   C      = trainable coefficient matrix                          (R x K, row-major)
 * and   y = x W^T,   dX = dY W,   dC = S^T (dY^T X).
 * W is never formed on the factored path (every BASELINE layer but a 256 -> 10 head); the W path, chosen when it costs
 * fewer FLOPs, keeps W in the caller's workspace for the length of one call.  S is regenerated from the seed in every call: tile by tile in shared
 * memory, or (every backward; forwards of more than 1024 tokens) once per call as a transient bf16 copy in the caller's workspace -- see
 * RDB_OPT_STAGE_NOISE.  Nothing of it survives the call.
 *
 * Conventions for every entry point
 *   - all pointers are DEVICE pointers owned by the caller (row-major, densely packed unless a
 *     leading dimension is passed); the library allocates nothing and frees nothing;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream);
 *     no entry point synchronises the device;
 *   - return value: 0 = ok, <0 = argument error found on the host before any launch
 *     (rdb_strerror names it), >0 = a cudaError_t raised by a launch or by tensor-map encoding;
 *   - `status` (optional, may be NULL) points to 4 device int32 words, zeroed by the caller.  A
 *     kernel whose bounded internal wait expires writes a non-zero code there and returns early
 *     instead of hanging; the caller reads it after synchronising when it wants to check;
 *   - row0 is the global index of the first noise row this call owns: a rank that holds output
 *     rows [row0, row0+N) of a larger virtual layer passes its own row0 and regenerates exactly
 *     its rows, so sharding a layer moves no weight bytes;
 *   - seed is used modulo 2^32 (two's complement for negative Python ints).
 *
 * Each declaration cites the reference interface it stands in for (paths inside the reference
 * project Clyde013/randumb).
 */
#ifndef RANDUMB_B200_H
#define RANDUMB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RDB_VERSION 100

/* element types */
#define RDB_F32 0
#define RDB_BF16 1

/* association of W = S*C with the activation (rdb_linear_*): */
#define RDB_PATH_AUTO 0     /* pick by FLOP count */
#define RDB_PATH_FACTORED 1 /* y = (x C^T) S^T ;  g = dY S, dX = g C, dC = g^T X  */
#define RDB_PATH_WPATH 2    /* W = S C in workspace (bf16 on the tensor-core kernels, float32 on CUDA cores), then dense products */

/* which kernels may run (rdb_linear_*): */
#define RDB_IMPL_AUTO 0   /* tcgen05 tensor-core kernels when dtype/shape allow, else SIMT */
#define RDB_IMPL_SIMT 1   /* CUDA-core kernels only (any shape, any dtype) */
#define RDB_IMPL_UMMA 2   /* tcgen05 kernels only; error if the shape does not qualify */

/* error codes (negative) */
#define RDB_OK 0
#define RDB_ERR_NULL -1
#define RDB_ERR_SHAPE -2
#define RDB_ERR_DTYPE -3
#define RDB_ERR_ALIGN -4
#define RDB_ERR_WORKSPACE -5
#define RDB_ERR_UNSUPPORTED -6
#define RDB_ERR_DRIVER -7
#define RDB_ERR_TOO_LARGE -8
#define RDB_ERR_PEER -9
/* tensor-map encoding rejected by the driver: the code is RDB_ERR_DRIVER_BASE - CUresult */
#define RDB_ERR_DRIVER_BASE -1000

/* device-side give-up codes written to status[0] */
#define RDB_STATUS_TIMEOUT_PRODUCER 1
#define RDB_STATUS_TIMEOUT_MMA 2
#define RDB_STATUS_TIMEOUT_EPILOGUE 3
#define RDB_STATUS_TIMEOUT_GENERATOR 4
#define RDB_STATUS_TIMEOUT_PEER 5      /* a rank of a peer exchange did not arrive in time */

int rdb_version(void);
const char *rdb_strerror(int code);

/*
 * Tuning switches (not part of the reference surface; defaults are the tuned ones).  rdb_set_option sets the PROCESS
 * DEFAULT of one switch; the *_ex entry points take a `const rdb_call_options *` whose fields override the defaults for
 * that one call (a field < 0, or a NULL pointer, keeps the default), so concurrent callers -- autograd worker threads,
 * several streams -- never have to change process state around a launch.
 *   RDB_OPT_NOISE_TILE   kernel variant / work unit of the generated-operand product:
 *                        0: automatic (8 for more than 512 tokens; for one token tile 1 with a contraction of at most 4096, else 9)
 *                        single-CTA MMAs (cta_group::1), (cluster size, token sub-tiles, generated rows):
 *                          1: (1, 4, 128)   2: (1, 2, 256)   3: (2, 4, 128)   4: (4, 4, 128)   5: (4, 2, 256)   6: (1, 4, 128) with a deeper ring
 *                          CTAs of a cluster share each generated stage through distributed shared memory
 *                        CTA-pair MMAs (cta_group::2), 512 tokens x 256 generated rows per pair:
 *                          7: one pair per cluster   8: two pairs   9: four pairs sharing the generated rows
 *   RDB_OPT_DENSE_PAIR   plain bf16 products with more than 128 rows and columns:
 *                        1 (default): CTA pairs (cta_group::2, 512 x 256 tiles) when the tiles fill the resident
 *                           pairs evenly, else the single-CTA 128 x 256 kernel
 *                        0: always the single-CTA kernel   2: always CTA pairs
 *   RDB_OPT_STAGE_NOISE  how rdb_linear_fwd / rdb_linear_bwd (bf16, factored) obtain the noise operand:
 *                        0 (default): automatic -- S (bf16, N x R, never W) is written once per call into the workspace
 *                           and consumed by the plain tensor-core product, which hashes every noise element once instead
 *                           of once per 512-token tile: by the backward at every token count (g = dY S has too few work
 *                           units to hash S in otherwise), by the forward for more than 1024 tokens; a forward of at most 1024,
 *                           and every call whose S would exceed 1 GiB, regenerates S tile by tile in shared memory
 *                        1: always regenerate tile by tile (no S in memory)   2: always stage when it fits
 *   RDB_OPT_RESERVE_SMS  0 (default) .. RDB_MAX_RESERVE_SMS: SMs the persistent plain-product kernels leave without a
 *                        CTA.  Their CTAs take a whole SM each for the length of the launch, so a collective enqueued
 *                        beside them (an NCCL all-reduce of the previous product's result) only runs at the same time
 *                        if some SMs are left free.  Meant to be given per call, for the launch that should overlap.
 *   RDB_OPT_FILL_OVERLAP 1 (default): automatic -- when S has 64 Mi elements or more, or 1 Mi or fewer, rdb_linear_fwd hashes
 *                        the staged S on a stream of the library's own, forked from and joined back into the caller's stream
 *                        with events, so the integer-ALU fill runs beside the tensor-core product z = x C^T it does not depend
 *                        on (a fill in between stays on the caller's stream: it is more than launch latency, and beside a
 *                        short product its resident threads cost the product's MMA-issuing thread as much as it takes).  The
 *                        stream and its two events are created once per device by the first such call (make it before any
 *                        stream capture; a call that finds its stream capturing before they exist keeps the fill on the
 *                        caller's stream).
 *                        0: always on the caller's stream.   2: always beside the z product.
 *   RDB_OPT_GEMV_FUSED   0 (default): the batch-1 entry points (rdb_gemv_fwd, rdb_gemv_bwd, and rdb_linear_* for one float32 row)
 *                        launch one kernel per step (two forward, two backward), chained with programmatic dependent launch.
 *                        1: ONE cooperative launch each, the steps separated by grid-wide barriers (when the device supports
 *                        cooperative launch).  Same results bit for bit; measured slower (28.6 against 18.2 us per forward +
 *                        backward of the 4096 x 4096, d_c = 256 layer), kept as a switch.  Process default only.
 *   RDB_OPT_GRADS_BESIDE 1 (default): automatic -- rdb_linear_bwd (bf16, factored, both gradients asked for) runs dX = g C and
 *                        dC = g^T x at the same time, dX on the library's own stream (the one RDB_OPT_FILL_OVERLAP describes,
 *                        same fork and join by events, same rule about stream capture) on some of the CTA pairs and dC on the
 *                        caller's stream on the others, when both can run on CTA pairs and their tile lists pack at least 7 %
 *                        better side by side than one after the other (the headline layer: 256 tiles of 16 k-blocks and 32
 *                        tiles of 128 k-blocks for 74 pairs).  Same results bit for bit as RDB_OPT_DENSE_PAIR = 2 gives.
 *                        0: one after the other on the caller's stream.   2: side by side whenever both can run on CTA pairs.
 * rdb_set_option returns the previous default, or RDB_ERR_UNSUPPORTED for an unknown key or a value outside the
 * range above (nothing changes then); a call whose rdb_call_options holds such a value returns the same error.
 */
#define RDB_OPT_NOISE_TILE 1
#define RDB_OPT_DENSE_PAIR 2
#define RDB_OPT_STAGE_NOISE 3
#define RDB_OPT_RESERVE_SMS 4
#define RDB_OPT_FILL_OVERLAP 5
#define RDB_OPT_GEMV_FUSED 6
#define RDB_OPT_GRADS_BESIDE 7
#define RDB_MAX_RESERVE_SMS 64
int rdb_set_option(int key, int value);

typedef struct rdb_call_options {
    int32_t noise_tile;   /* RDB_OPT_NOISE_TILE, or < 0 for the process default */
    int32_t dense_pair;   /* RDB_OPT_DENSE_PAIR   ... */
    int32_t stage_noise;  /* RDB_OPT_STAGE_NOISE  ... */
    int32_t reserve_sms;  /* RDB_OPT_RESERVE_SMS  ... */
    int32_t fill_overlap; /* RDB_OPT_FILL_OVERLAP ... */
    int32_t grads_beside; /* RDB_OPT_GRADS_BESIDE ... */
} rdb_call_options;

/*
 * Cycle counters of the tensor-core kernels (diagnostics; no reference counterpart).  While a device buffer of at
 * least 128 bytes per CTA (148 * 128 covers any launch) is registered, every launch of the generated-operand kernels
 * writes sixteen int64 SM-cycle counters per CTA into it: [0] MMA thread waiting for the streamed operand, [1] waiting
 * for the generated operand, [2] waiting for the epilogue to drain TMEM, [3] MMA thread total, [4] TMA thread waiting
 * for a free stage, [5] generator waiting for a free stage, [6] generator hashing and storing, [7] epilogue busy,
 * [8] MMA thread in fences, [9] issuing MMAs, [10] issuing commits; the rest unused.  The CTA-pair plain-product kernel
 * writes [0] (operands), [2], [3] and [4] the same way, and from the first epilogue warp of each CTA, summed over its tiles,
 * [5] accumulator 0 seen complete -> handed back, [6] -> accumulator 1 handed back, [7] the store phase (the buffer must be
 * zeroed before such a launch: these three are added to); the benchmark divides [3] by the launch's event time to report
 * the SM clock the kernel really ran at.  Pass NULL to switch it off (the default; the counters then cost nothing).
 */
int rdb_set_profile_buffer(void *device_buffer, size_t bytes);

/*
 * Raw hash words of the noise matrix: out[r*ld + c] = bits(row0 + r, col0 + c, seed), uint32.
 * The reference never exposes the integers; this is the bit-exactness surface for
 * squirrel5_gen_2d (src/rten_cpp/RandumbTensor.py:130-164) and sq5_2d (csrc/cuda/rten.cu:28-48).
 */
int rdb_noise_bits(uint32_t *out, int64_t rows, int64_t cols, int64_t ld, int64_t row0, int64_t col0,
                   uint32_t seed, void *stream);

/*
 * Explicit noise matrix as float32 or bfloat16 (bf16 = round-to-nearest-even of the float32 value).
 * Stands in for squirrel5_generate_2d (src/rten_cpp/RandumbTensor.py:78-105),
 * RandumbTensor.get_noise_matrix (:870-873) and rten_cpp::sq5_gen_2d (csrc/cuda/rten.cu:50-71,
 * without its row-stride defect at :55).
 */
int rdb_noise(void *out, int dtype, int64_t rows, int64_t cols, int64_t ld, int64_t row0, int64_t col0,
              uint32_t seed, void *stream);

/*
 * 1-D noise out[i] = value(idx0 + i, seed) with no row mixing: squirrel5_gen_1d
 * (src/rten_cpp/RandumbTensor.py:204-232), the generator of the reference's fused random bias.
 */
int rdb_noise_1d(float *out, int64_t n, int64_t idx0, uint32_t seed, void *stream);

/*
 * Bytes of scratch the linear entry points need for the given problem (op: 0 = forward,
 * 1 = backward).  The workspace must be 256-byte aligned.  bf16 tensor-core path: T*R*2 bytes for z or g, plus
 * N*R*2 bytes when the noise operand is staged (rdb_linear_stages_noise); the size depends on the option values
 * in force, so query it after setting them (or pass the call's options to the _ex form).  The query assumes 16-byte
 * aligned operands; a call with RDB_IMPL_AUTO whose x, coef, y, dy, dx or dc is not 16-byte aligned runs on the CUDA-core
 * kernels instead (RDB_IMPL_UMMA returns RDB_ERR_ALIGN) and needs the size this query returns for RDB_IMPL_SIMT.
 */
size_t rdb_linear_workspace_bytes(int op, int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path,
                                  int impl);
size_t rdb_linear_workspace_bytes_ex(int op, int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path,
                                     int impl, const rdb_call_options *options);

/*
 * Whether the linear entry points would, for this problem, write S (bf16, N x R) into the workspace once per call and run
 * the plain tensor-core product on it: bit 0 (value 1) for rdb_linear_fwd, bit 1 (value 2) for rdb_linear_bwd; a clear bit
 * means that call regenerates S tile by tile inside the kernel (or uses the float32 kernels); negative: error.  See
 * RDB_OPT_STAGE_NOISE.  No reference counterpart (a planning query).
 */
int rdb_linear_stages_noise(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl);
int rdb_linear_stages_noise_ex(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl,
                               const rdb_call_options *options);

/*
 * Planning query: which association and which kernels the linear entry points would use for this problem (operands
 * assumed 16-byte aligned): returns RDB_PATH_* | (RDB_IMPL_* << 8) with both resolved (never AUTO), or a negative error.
 * RDB_PATH_AUTO picks by FLOP count -- factored 2TR(K+N) per result against 2NRK + 2TNK through W; RDB_IMPL_AUTO picks
 * the tcgen05 kernels for bf16 problems whose extents are multiples of 8 (both associations run on them), else the
 * CUDA-core kernels.  No reference counterpart.
 */
int rdb_linear_path(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl);

/*
 * Planning query: 1 when rdb_linear_bwd, asked for both gradients of this problem with these options, would run dX beside
 * dC (RDB_OPT_GRADS_BESIDE), with the CTA pairs each of the two gets in *pairs_dx / *pairs_dc (either may be NULL); 0 when
 * it runs them one after the other (both set to 0); a negative error for a bad dtype or option.  No reference counterpart.
 */
int rdb_linear_bwd_plan(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl,
                        const rdb_call_options *options, int *pairs_dx, int *pairs_dc);

/*
 * Forward  y[T,N] = x[T,K] * W^T  with W regenerated from (seed, row0) and coef[R,K].
 * This is the fused product the reference left as a placeholder: the aten.mm override
 * (src/rten_cpp/RandumbTensor.py:942-946) -> fakeMM (:771-791), and the abandoned Triton
 * attempts rt_mm / rt_mm_grouped (:457-769).
 */
int rdb_linear_fwd(void *y, const void *x, const void *coef, void *workspace, size_t workspace_bytes,
                   int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, int dtype,
                   int path, int impl, int32_t *status, void *stream);
int rdb_linear_fwd_ex(void *y, const void *x, const void *coef, void *workspace, size_t workspace_bytes,
                      int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, int dtype,
                      int path, int impl, const rdb_call_options *options, int32_t *status, void *stream);

/*
 * Backward: dx[T,K] = dy W (skipped when dx == NULL) and dc[R,K] = S^T (dy^T x) (skipped when
 * dc == NULL).  dc is written in `dtype`.  Replaces fakeMMFunction.backward
 * (src/rten_cpp/RandumbTensor.py:783-788) followed by RandumbTensorConstructor.backward
 * (:979-990) / materialize_bwd (:304-359, :383-390): no dense dW is formed on the factored path.
 */
int rdb_linear_bwd(void *dx, void *dc, const void *dy, const void *x, const void *coef, void *workspace,
                   size_t workspace_bytes, int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0,
                   uint32_t seed, int dtype, int path, int impl, int32_t *status, void *stream);
int rdb_linear_bwd_ex(void *dx, void *dc, const void *dy, const void *x, const void *coef, void *workspace,
                      size_t workspace_bytes, int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0,
                      uint32_t seed, int dtype, int path, int impl, const rdb_call_options *options,
                      int32_t *status, void *stream);

/*
 * Dense weight w[N,K] = S[row0:row0+N, 0:R] * coef[R,K] written out in `dtype` (debugging and ops
 * that have no fused kernel).  Stands in for RandumbTensor.materialize / get_materialized
 * (src/rten_cpp/RandumbTensor.py:862-868, 887-892) for a matrix-shaped coefficient.
 */
int rdb_linear_weight(void *w, const void *coef, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed,
                      int dtype, void *stream);

/*
 * Batch-1 float32 forward: y[N] = S (C x).  workspace: R floats.  Same reference slot as
 * rdb_linear_fwd, specialised for a single activation row (matrix-vector; bandwidth bound).
 */
int rdb_gemv_fwd(float *y, const float *x, const float *coef, float *workspace, int64_t K, int64_t N,
                 int64_t R, int64_t row0, uint32_t seed, void *stream);

/*
 * rdb_gemv_fwd for callers that have no device memory to hand over as workspace and may not allocate
 * any: for example a serving loop whose memory was divided up completely at start-up, or a host runtime
 * that forbids allocation calls on its request path.  (No counterpart in the reference, which allocates
 * a fresh tensor for every intermediate.)  The R intermediate values live in a fixed array inside the
 * library instead, so
 *   - R may be at most RDB_GEMV_STATIC_MAX_R; a larger R returns RDB_ERR_TOO_LARGE and launches nothing;
 *   - the library keeps RDB_GEMV_STATIC_MAX_R * 4 bytes on every GPU it is loaded on until exit;
 *   - the call itself performs no cudaMalloc/cudaFree and calls no allocating library routine;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, cached
 *     per device afterwards); make that first call with the device current and before any stream
 *     capture is started;
 *   - all calls on a device share the one array: two calls that overlap on the GPU (different streams)
 *     race on it and may return wrong results; calls on one stream are safe.  The array keeps the last
 *     call's values, which is harmless: every call overwrites the R entries it later reads.
 * Results are bitwise those of rdb_gemv_fwd.
 */
#define RDB_GEMV_STATIC_MAX_R 16384
int rdb_gemv_fwd_static(float *y, const float *x, const float *coef, int64_t K, int64_t N, int64_t R,
                        int64_t row0, uint32_t seed, void *stream);

/*
 * Batch-1 float32 backward: g = S^T dy, dx[K] = g C, dc[R,K] = g x^T.  dx or dc may be NULL.
 * workspace: rdb_gemv_bwd_workspace_bytes(K, N, R) bytes, 256-byte aligned (g, the per-slice partial sums of dx -- the pass
 * over C is cut into row slices so that enough blocks keep HBM busy, and the slices are added in a fixed order -- and one
 * arrival counter per 32 columns; contents on entry do not matter).
 * The four kernels of a forward + backward step are launched with programmatic stream serialization: each one's blocks
 * become resident while the previous kernel of the stream is still running and wait for its completion on the device,
 * which takes the launch gap out of a step that is only a few microseconds of memory traffic.
 */
size_t rdb_gemv_bwd_workspace_bytes(int64_t K, int64_t N, int64_t R);
int rdb_gemv_bwd(float *dx, float *dc, const float *dy, const float *x, const float *coef, float *workspace,
                 int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, void *stream);

/*
 * Building block: D[M,N] = A[M,Kc] * G^T where G is generated, never read from memory.
 *   transposed == 0:  G[n,k] = S[row0+n, col0+k]      (y = z S^T : contraction over noise columns)
 *   transposed == 1:  G[n,k] = S[row0+k, col0+n]      (g = dY S  : contraction over noise rows)
 * A is row-major with leading dimension lda; D row-major with ldd.
 * a_dtype / d_dtype: RDB_F32 or RDB_BF16 (the tcgen05 kernel needs both bf16).
 * Same reference slot as rt_mm_grouped_kernel (src/rten_cpp/RandumbTensor.py:648-746), whose RT
 * operand is regenerated tile by tile inside the kernel.
 */
int rdb_gemm_noise(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd,
                   int a_dtype, int d_dtype, int transposed, int64_t row0, int64_t col0, uint32_t seed,
                   int impl, int32_t *status, void *stream);

/*
 * Building block: dense D[M,N] = op(A) * op(B)^T, float32 accumulation.
 *   a_kmajor != 0: A is [M,Kc] row-major (lda);  == 0: A is stored [Kc,M] row-major (lda).
 *   b_kmajor != 0: B is [N,Kc] row-major (ldb);  == 0: B is stored [Kc,N] row-major (ldb).
 * The plain products of the factored layer (x C^T, g C, g^T x); the reference calls cuBLAS here
 * (src/rten_cpp/RandumbTensor.py:780, 786-787).
 */
int rdb_gemm_dense(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda,
                   int64_t ldb, int64_t ldd, int a_dtype, int b_dtype, int d_dtype, int a_kmajor,
                   int b_kmajor, int impl, int32_t *status, void *stream);

/*
 * The same product with scratch for split-K: when the output has few tiles and the contraction is long
 * (rdb_gemm_dense_workspace_bytes > 0), the contraction is cut into slices that run as independent work items writing
 * float32 partial products into `workspace`, summed afterwards in a fixed order.  Needs a densely packed output
 * (ldd == N) and a 256-byte aligned workspace; falls back to rdb_gemm_dense otherwise.  No reference counterpart.
 */
size_t rdb_gemm_dense_workspace_bytes(int64_t M, int64_t N, int64_t Kc);
int rdb_gemm_dense_ws(void *d, const void *a, const void *b, void *workspace, size_t workspace_bytes, int64_t M, int64_t N,
                      int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int a_dtype, int b_dtype, int d_dtype,
                      int a_kmajor, int b_kmajor, int impl, int32_t *status, void *stream);
/* ... and with per-call options (workspace may be NULL: no split-K then) */
int rdb_gemm_dense_ex(void *d, const void *a, const void *b, void *workspace, size_t workspace_bytes, int64_t M, int64_t N,
                      int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int a_dtype, int b_dtype, int d_dtype,
                      int a_kmajor, int b_kmajor, int impl, const rdb_call_options *options, int32_t *status,
                      void *stream);

/*
 * Reference 1-D-coefficient form (every existing randumb model):
 *   out[n] = sum_m S[sq(n), m] * coef[m],  sq(n) = (n % Q)*stride_Q + (n / Q)*stride_P,  float32 [P,Q].
 * Stands in for rten::materialize_fwd (src/rten_cpp/RandumbTensor.py:235-290, 371-381) and
 * rten_cpp::materialize_fwd (csrc/cuda/rten.cu:74-152).
 * scale_bias: null, or a device pointer to one float; when given, the fused random bias of the reference
 * (RAND_BIAS branch, src/rten_cpp/RandumbTensor.py:283-286) is added:
 *   out[n] += scale_bias[0] * noise1d(sq(n))     (the 1-D hash of the same index, no prime multiply).
 */
int rdb_materialize_fwd(float *out, const float *coef, int64_t M, int64_t P, int64_t Q, int64_t stride_P,
                        int64_t stride_Q, const float *scale_bias, uint32_t seed, void *stream);

/*
 * dcoef[m] = sum_n S[n,m] * dout[n] over the flattened contiguous dout (float32), deterministic
 * reduction order.  Stands in for rten::materialize_bwd (src/rten_cpp/RandumbTensor.py:304-359,
 * 383-390).  workspace: rdb_materialize_bwd_workspace_bytes(Nel, M) bytes.
 */
size_t rdb_materialize_bwd_workspace_bytes(int64_t Nel, int64_t M);
int rdb_materialize_bwd(float *dcoef, const float *dout, float *workspace, int64_t Nel, int64_t M,
                        uint32_t seed, void *stream);

/*
 * Gradient of the random-bias scale: dbias[0] = sum_n dout[n] * noise1d(n) over the flattened contiguous
 * dout (float32), deterministic reduction order.  Stands in for rten::scale_bias_bwd
 * (src/rten_cpp/RandumbTensor.py:400-420).  workspace: rdb_scale_bias_bwd_workspace_bytes(Nel) bytes.
 */
size_t rdb_scale_bias_bwd_workspace_bytes(int64_t Nel);
int rdb_scale_bias_bwd(float *dbias, const float *dout, float *workspace, int64_t Nel, uint32_t seed,
                       void *stream);

/*
 * Rows of a virtual (vocab, rowsize) embedding matrix in the 1-D-coefficient form:
 *   out[i, j] = sum_m S[idx[i]*rowsize + j, m] * coef[m]     out float32 [n_idx, rowsize], row pitch ld_out
 *   dcoef[m]  = sum_{i,j} S[idx[i]*rowsize + j, m] * dout[i, j]   (dout contiguous; repeated indices add)
 * idx: n_idx int64 row numbers on the device.  Stand in for rten::embed_fwd / rten::embed_bwd
 * (src/rten_cpp/RandumbTensor.py:999-1056, 1060-1107, 1121-1134).  The backward pass is deterministic;
 * workspace: rdb_materialize_bwd_workspace_bytes(n_idx*rowsize, M) bytes.
 */
int rdb_embed_fwd(float *out, const int64_t *idx, const float *coef, int64_t n_idx, int64_t rowsize, int64_t M,
                  int64_t ld_out, uint32_t seed, void *stream);
int rdb_embed_bwd(float *dcoef, const float *dout, const int64_t *idx, float *workspace, int64_t n_idx,
                  int64_t rowsize, int64_t M, uint32_t seed, void *stream);

/*
 * Exchange steps of a layer whose output rows are split over the GPUs of one node (each rank regenerates its own noise
 * rows, so only activations move: z = x C^T is gathered, g = dY S is summed).  The reference has no counterpart -- its
 * only collectives are DDP's (modded-nanogpt/train_gpt2.py:346, 441); these are this library's own kernels over peer
 * memory, plain stores through NVLink / NVSwitch (no TMA multicast, no multimem), as an alternative to NCCL calls
 * between the products.  The caller owns all memory: every rank allocates one exchange buffer that the other ranks of
 * the node have mapped (symmetric memory or CUDA IPC) and passes the resulting pointer lists -- `ptrs[r]` is rank r's
 * buffer as addressable from the calling process, 16-byte aligned, at most RDB_MAX_PEERS of them.
 *
 * rdb_peer_barrier   every rank has enqueued the barrier with this `epoch` and everything it stored before has landed.
 *                    flag_ptrs[r]: RDB_MAX_PEERS uint64 words in rank r's buffer, zero before the first barrier; epochs
 *                    must grow (1, 2, 3, ...) and be the same on all ranks for the same barrier.  A rank that waits longer
 *                    than RDB_PEER_WAIT_LIMIT_NS writes RDB_STATUS_TIMEOUT_PEER to status[0] and returns.  Never enqueue
 *                    the barriers of several ranks on ONE GPU: they wait for each other and nothing makes two launches
 *                    run at the same time.
 * rdb_peer_copy      src[0, nbytes) -> dst_ptrs[d] + dst_offset_bytes for every d < ndst (an all-gather step: every
 *                    rank sends its block to the same place in all buffers).  max_blocks <= 0: library default.
 * rdb_peer_scatter   block j of src (block_bytes each) -> dst_ptrs[j] + dst_offset_bytes (the scatter half of a
 *                    reduce-scatter: rank j collects everybody's contribution to its block).
 * rdb_reduce_slots_bf16   out[i] = sum over s < nslots of slots[s * slot_stride_bytes + i] (bf16, float32 accumulation,
 *                    fixed order s = 0, 1, ...: the result does not depend on arrival order).
 * rdb_gemm_dense_scatter  D = A op(B)^T (bf16, CTA-pair tcgen05 kernel) with the scatter fused into the product: row block
 *                    j of D (rows_per_dst rows, a multiple of 32) is stored by the kernel's epilogue straight into
 *                    dst_ptrs[j] + dst_offset_bytes as a dense [rows_per_dst x N] matrix, tile by tile while later tiles are
 *                    still being computed.  A is [M, Kc] row-major; B is [N, Kc] (b_kmajor) or [Kc, N].  Needs M and N
 *                    above 128 and extents in multiples of 8 (else RDB_ERR_UNSUPPORTED: use rdb_gemm_dense +
 *                    rdb_peer_scatter).
 */
#define RDB_MAX_PEERS 8
#define RDB_PEER_WAIT_LIMIT_NS 4000000000ull
int rdb_peer_barrier(void *const *flag_ptrs, int rank, int world, uint64_t epoch, int32_t *status, void *stream);
int rdb_peer_copy(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, const void *src, size_t nbytes, int max_blocks,
                  void *stream);
int rdb_peer_scatter(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, const void *src, size_t block_bytes,
                     int max_blocks, void *stream);
int rdb_reduce_slots_bf16(void *out, const void *slots, size_t slot_stride_bytes, int nslots, size_t nbytes, void *stream);
int rdb_gemm_dense_scatter(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, int64_t rows_per_dst, const void *a,
                           const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int b_kmajor,
                           const rdb_call_options *options, int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RANDUMB_B200_H */
