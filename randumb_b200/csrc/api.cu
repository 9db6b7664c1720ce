// C-ABI entry points of the layer: argument checks, association/kernel choice, workspace carving.
#include <atomic>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace rdb {

// process defaults of the tuning switches (rdb_set_option); a call may override each of them (rdb_call_options)
static std::atomic<int> g_noise_tile{0};     // RDB_OPT_NOISE_TILE
static std::atomic<int> g_dense_pair{1};     // RDB_OPT_DENSE_PAIR
static std::atomic<int> g_stage_noise{0};    // RDB_OPT_STAGE_NOISE
static std::atomic<int> g_reserve_sms{0};    // RDB_OPT_RESERVE_SMS
static std::atomic<int> g_fill_overlap{1};   // RDB_OPT_FILL_OVERLAP
static std::atomic<int> g_grads_beside{1};   // RDB_OPT_GRADS_BESIDE

static bool opt_in_range(int key, int v) {
    switch (key) {
        case RDB_OPT_NOISE_TILE: return v >= 0 && v <= 9;
        case RDB_OPT_DENSE_PAIR: return v >= 0 && v <= 2;
        case RDB_OPT_STAGE_NOISE: return v >= 0 && v <= 2;
        case RDB_OPT_RESERVE_SMS: return v >= 0 && v <= RDB_MAX_RESERVE_SMS;
        case RDB_OPT_FILL_OVERLAP: return v >= 0 && v <= 2;
        case RDB_OPT_GRADS_BESIDE: return v >= 0 && v <= 2;
        case RDB_OPT_GEMV_FUSED: return v == 0 || v == 1;
        default: return false;
    }
}

// Options of one call: the caller's values where given (>= 0), the process defaults elsewhere.
static int resolve_opts(const rdb_call_options *o, CallOpts *out) {
    CallOpts c{g_noise_tile.load(), g_dense_pair.load(), g_stage_noise.load(), g_reserve_sms.load(), g_fill_overlap.load(),
               g_grads_beside.load()};
    if (o) {
        const int keys[6] = {RDB_OPT_NOISE_TILE,  RDB_OPT_DENSE_PAIR,   RDB_OPT_STAGE_NOISE,
                             RDB_OPT_RESERVE_SMS, RDB_OPT_FILL_OVERLAP, RDB_OPT_GRADS_BESIDE};
        const int vals[6] = {o->noise_tile, o->dense_pair, o->stage_noise, o->reserve_sms, o->fill_overlap, o->grads_beside};
        int *dst[6] = {&c.noise_tile, &c.dense_pair, &c.stage_noise, &c.reserve_sms, &c.fill_overlap, &c.grads_beside};
        for (int i = 0; i < 6; ++i) {
            if (vals[i] < 0) continue;
            if (!opt_in_range(keys[i], vals[i])) return RDB_ERR_UNSUPPORTED;
            *dst[i] = vals[i];
        }
    }
    *out = c;
    return RDB_OK;
}

static bool umma_dims_ok(int64_t T, int64_t K, int64_t N, int64_t R, int dtype) {
    return dtype == RDB_BF16 && T >= 1 && (K % 8) == 0 && (N % 8) == 0 && (R % 8) == 0 && K >= 8 && N >= 8 && R >= 8 &&
           T < (1LL << 31) && K < (1LL << 31) && N < (1LL << 31) && R < (1LL << 31);
}

// The W path on tensor cores keeps S (bf16, N x R) and W (bf16, N x K) in the workspace for the length of the call.
static bool wpath_umma_fits(int64_t K, int64_t N, int64_t R) {
    return (double)N * (double)R * 2.0 <= 1073741824.0 && (double)N * (double)K * 2.0 <= 4294967296.0;
}

// FLOP-count rule: factored costs 2TR(K+N) per result, the W path 2NRK + 2TNK.
static int choose_path(int path, int64_t T, int64_t K, int64_t N, int64_t R) {
    if (path == RDB_PATH_FACTORED || path == RDB_PATH_WPATH) return path;
    const double fact = 2.0 * (double)T * (double)R * ((double)K + (double)N);
    const double wp = 2.0 * (double)N * (double)R * (double)K + 2.0 * (double)T * (double)N * (double)K;
    return fact <= wp ? RDB_PATH_FACTORED : RDB_PATH_WPATH;
}

static bool umma_eligible(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path) {
    if (!umma_dims_ok(T, K, N, R, dtype)) return false;
    return path == RDB_PATH_FACTORED || wpath_umma_fits(K, N, R);
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// returns RDB_IMPL_SIMT or RDB_IMPL_UMMA, or a negative error.  `aligned`: every operand the tensor-core kernels would
// touch starts on a 16-byte boundary (TMA needs that); the planning queries, which see no pointers, pass true.
static int choose_impl(int impl, int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, bool aligned) {
    const bool ok = umma_eligible(T, K, N, R, dtype, path);
    if (impl == RDB_IMPL_UMMA) {
        if (!ok) return RDB_ERR_UNSUPPORTED;
        return aligned ? RDB_IMPL_UMMA : RDB_ERR_ALIGN;
    }
    if (impl == RDB_IMPL_SIMT) return RDB_IMPL_SIMT;
    if (impl != RDB_IMPL_AUTO) return RDB_ERR_UNSUPPORTED;
    return (ok && aligned) ? RDB_IMPL_UMMA : RDB_IMPL_SIMT;
}

// Whether the bf16 factored products take S from a staged copy in the workspace (hashing every element once per
// call) or regenerate it tile by tile inside the kernel (once per 512-token tile, nothing in memory).
static bool stage_noise(int op, int64_t T, int64_t N, int64_t R, const CallOpts &o) {
    const bool fits = (double)N * (double)R * 2.0 <= 1073741824.0;
    if (o.stage_noise == 1 || !fits) return false;
    if (o.stage_noise == 2) return true;
    // Forward (op 0): y = z S^T has N / 256 work units whatever the token count, and up to 1024 tokens the regenerating
    // kernel hashes every element once too (one 512-token tile, or two that share each generated stage), under its MMAs and
    // without the round trip of S through memory: 53 against 64 us for 1024 tokens of the headline layer, 251 against 290
    // for a 65536 x 2048 noise block; from 1536 tokens on the fill wins.
    // Backward (op 1): g = dY S has only R / 256 work units per 512 tokens to hash all of S in, so hashing it once on every SM
    // wins at every token count (512 tokens, 16384 x 1024: 206 against 60 us for the whole backward).
    return op == 1 || T > 1024;
}

struct WsLayout {
    size_t off[4];
    size_t total;
};

// Workspace segments (each 1024-byte aligned):
//   UMMA factored  fwd: z bf16[T,R], then S bf16[N,R] when the noise operand is staged
//                  bwd: g bf16[T,R], then S bf16[N,R] when staged, then float32 [split,R,K] when dC is computed split-K
//   UMMA W path    fwd: S bf16[N,R], W bf16[N,K]      bwd: S bf16[N,R], W bf16[N,K], dW bf16[N,K]
//   SIMT factored  fwd: z f32[T,R]           bwd: g f32[T,R]
//   SIMT W path    fwd: W f32[N,K]           bwd: W f32[N,K], dW f32[N,K]
static WsLayout ws_layout(int op, int64_t T, int64_t K, int64_t N, int64_t R, int path, int impl, const CallOpts &o, int dtype) {
    WsLayout w{};
    size_t seg[4] = {0, 0, 0, 0};
    if (path == RDB_PATH_FACTORED) {
        if (impl == RDB_IMPL_UMMA) {
            seg[0] = (size_t)T * R * 2;
            if (stage_noise(op, T, N, R, o)) seg[1] = (size_t)N * R * 2;
            // float32 partial products of the products with few output tiles and a long contraction, computed split-K:
            // forward z = x C^T (contraction K); backward g = dY S (contraction N, staged S only) and dC = g^T x (contraction T)
            if (op == 0) {
                const int split = dense_split_k_slices(T, R, K);
                if (split > 1) seg[2] = (size_t)split * T * R * 4;
            } else {
                const int sg = stage_noise(1, T, N, R, o) ? dense_split_k_slices(T, R, N) : 1;
                const int sc = dense_split_k_slices(R, K, T);
                const size_t a = sg > 1 ? (size_t)sg * T * R * 4 : 0, b = sc > 1 ? (size_t)sc * R * K * 4 : 0;
                seg[2] = a > b ? a : b;        // used one after the other
            }
        } else {
            seg[0] = (size_t)T * R * 4;
            // a single float32 row goes to the matrix-vector kernels, whose backward keeps per-slice sums and counters too
            if (T == 1 && dtype == RDB_F32 && op == 1) seg[0] = rdb_gemv_bwd_workspace_bytes(K, N, R);
        }
    } else if (impl == RDB_IMPL_UMMA) {
        seg[0] = (size_t)N * R * 2;
        seg[1] = (size_t)N * K * 2;
        if (op == 1) seg[2] = (size_t)N * K * 2;
    } else {
        seg[0] = (size_t)N * K * 4;
        if (op == 1) seg[1] = (size_t)N * K * 4;
    }
    size_t o_ = 0;
    for (int i = 0; i < 4; ++i) {
        w.off[i] = o_;
        o_ += align_up(seg[i], 1024);
    }
    w.total = o_;
    return w;
}

// One extra stream and two events per device, created on first use: the forward's noise fill (integer ALU) runs on it
// beside the z product (tensor pipe) and joins the caller's stream before the y product; the backward's dX runs on it
// beside dC.  Nothing is created per call.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex mu;           // one fork/join sequence at a time per device (the events are shared)
    bool tried = false, ok = false;
};

// `st`: the caller's stream.  While it is being captured nothing is created (the first call on a device should come before
// any capture); without the extra stream the fill simply stays on the caller's stream.
static SideStream *side_stream(cudaStream_t st) {
    static SideStream per_device[64];
    static std::mutex create_mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SideStream *s = &per_device[dev];
    std::lock_guard<std::mutex> lock(create_mu);
    if (!s->tried) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        if (cap != cudaStreamCaptureStatusNone) return nullptr;
        s->tried = true;
        if (cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&s->join, cudaEventDisableTiming) == cudaSuccess)
            s->ok = true;
        else
            (void)cudaGetLastError();
    }
    return s->ok ? s : nullptr;
}

}  // namespace rdb

using namespace rdb;

extern "C" int rdb_version(void) { return RDB_VERSION; }

extern "C" const char *rdb_strerror(int code) {
    switch (code) {
        case RDB_OK: return "ok";
        case RDB_ERR_NULL: return "null pointer argument";
        case RDB_ERR_SHAPE: return "invalid shape or leading dimension";
        case RDB_ERR_DTYPE: return "unsupported element type";
        case RDB_ERR_ALIGN: return "pointer or leading dimension not aligned as required (the tensor-core kernels need 16-byte aligned operands)";
        case RDB_ERR_WORKSPACE: return "workspace too small or misaligned";
        case RDB_ERR_UNSUPPORTED: return "combination or value of options not supported for this problem";
        case RDB_ERR_DRIVER: return "tensor-map encoding failed (driver entry point unavailable or rejected arguments)";
        case RDB_ERR_TOO_LARGE: return "problem exceeds a launch limit or a built-in maximum size";
        case RDB_ERR_PEER: return "peer exchange arguments invalid (rank, world size or a peer pointer)";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    if (code <= RDB_ERR_DRIVER_BASE && code > RDB_ERR_DRIVER_BASE - 1000) {
        static thread_local char buf[96];
        snprintf(buf, sizeof(buf), "tensor-map encoding rejected by the driver (CUresult %d)", RDB_ERR_DRIVER_BASE - code);
        return buf;
    }
    return "unknown error";
}

extern "C" int rdb_set_option(int key, int value) {
    std::atomic<int> *slot = nullptr;
    switch (key) {
        case RDB_OPT_NOISE_TILE: slot = &g_noise_tile; break;
        case RDB_OPT_DENSE_PAIR: slot = &g_dense_pair; break;
        case RDB_OPT_STAGE_NOISE: slot = &g_stage_noise; break;
        case RDB_OPT_RESERVE_SMS: slot = &g_reserve_sms; break;
        case RDB_OPT_FILL_OVERLAP: slot = &g_fill_overlap; break;
        case RDB_OPT_GRADS_BESIDE: slot = &g_grads_beside; break;
        case RDB_OPT_GEMV_FUSED: {
            if (!opt_in_range(key, value)) return RDB_ERR_UNSUPPORTED;
            const int prev = get_gemv_fused();
            set_gemv_fused(value);
            return prev;
        }
        default: return RDB_ERR_UNSUPPORTED;
    }
    if (!opt_in_range(key, value)) return RDB_ERR_UNSUPPORTED;   // nothing changes
    return slot->exchange(value);
}

extern "C" int rdb_set_profile_buffer(void *device_buffer, size_t bytes) {
    set_profile_buffer(device_buffer, bytes);
    return RDB_OK;
}

extern "C" int rdb_gemm_noise(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, int a_dtype,
                              int d_dtype, int transposed, int64_t row0, int64_t col0, uint32_t seed, int impl,
                              int32_t *status, void *stream) {
    if (M < 0 || N < 0 || Kc < 0 || lda < Kc || ldd < N) return RDB_ERR_SHAPE;
    if (M == 0 || N == 0) return RDB_OK;
    if (!d || (Kc > 0 && !a)) return RDB_ERR_NULL;
    if ((a_dtype != RDB_F32 && a_dtype != RDB_BF16) || (d_dtype != RDB_F32 && d_dtype != RDB_BF16)) return RDB_ERR_DTYPE;
    CallOpts o;
    int rc = resolve_opts(nullptr, &o);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const Sq5Lin lin = transposed ? sq5_lin_cols(seed, (uint32_t)row0, (uint32_t)col0)
                                  : sq5_lin_rows(seed, (uint32_t)row0, (uint32_t)col0);
    const bool can = a_dtype == RDB_BF16 && d_dtype == RDB_BF16 && umma_shape_ok_noise(M, N, Kc, lda, ldd, a, d);
    if (impl == RDB_IMPL_UMMA && !can) return RDB_ERR_UNSUPPORTED;
    if (impl != RDB_IMPL_SIMT && can) return umma_gemm_noise(d, a, M, N, Kc, lda, ldd, lin, status, st, o);
    return simt_gemm(d, d_dtype, ldd, 1, a, a_dtype, lda, 1, nullptr, RDB_F32, 0, 0, lin, M, N, Kc, st);
}

extern "C" size_t rdb_gemm_dense_workspace_bytes(int64_t M, int64_t N, int64_t Kc) {
    if (M <= 0 || N <= 0 || Kc <= 0) return 0;
    const int split = dense_split_k_slices(M, N, Kc);
    return split > 1 ? (size_t)split * (size_t)M * (size_t)N * sizeof(float) : 0;
}

extern "C" int rdb_gemm_dense_ex(void *d, const void *a, const void *b, void *workspace, size_t workspace_bytes, int64_t M,
                                 int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int a_dtype, int b_dtype,
                                 int d_dtype, int a_kmajor, int b_kmajor, int impl, const rdb_call_options *options,
                                 int32_t *status, void *stream) {
    if (M < 0 || N < 0 || Kc < 0 || ldd < N) return RDB_ERR_SHAPE;
    if (lda < (a_kmajor ? Kc : M) || ldb < (b_kmajor ? Kc : N)) return RDB_ERR_SHAPE;
    CallOpts o;
    int rc = resolve_opts(options, &o);
    if (rc) return rc;
    if (M == 0 || N == 0) return RDB_OK;
    if (!d || (Kc > 0 && (!a || !b))) return RDB_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    const bool can = a_dtype == RDB_BF16 && b_dtype == RDB_BF16 &&
                     umma_shape_ok_dense(M, N, Kc, lda, ldb, ldd, d_dtype, a_kmajor, b_kmajor, a, b, d);
    if (impl == RDB_IMPL_UMMA && !can) return RDB_ERR_UNSUPPORTED;
    if (impl != RDB_IMPL_SIMT && can) {
        const size_t need = rdb_gemm_dense_workspace_bytes(M, N, Kc);
        const bool split_ok = need > 0 && o.dense_pair != 2 && workspace && workspace_bytes >= need &&
                              (reinterpret_cast<uintptr_t>(workspace) & 255) == 0 && ldd == N;
        if (split_ok)
            return umma_gemm_dense_split_k(d, a, b, reinterpret_cast<float *>(workspace), dense_split_k_slices(M, N, Kc), M, N, Kc,
                                           lda, ldb, d_dtype, a_kmajor, b_kmajor, status, st, o);
        return umma_gemm_dense(d, a, b, M, N, Kc, lda, ldb, ldd, d_dtype, a_kmajor, b_kmajor, status, st, o);
    }
    Sq5Lin none{0, 0, 0};
    // SIMT needs a real B pointer; b == nullptr would select the generated operand.
    return simt_gemm(d, d_dtype, ldd, 1, a, a_dtype, a_kmajor ? lda : 1, a_kmajor ? 1 : lda, b, b_dtype,
                     b_kmajor ? ldb : 1, b_kmajor ? 1 : ldb, none, M, N, Kc, st);
}

extern "C" int rdb_gemm_dense_scatter(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, int64_t rows_per_dst, const void *a,
                                      const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int b_kmajor,
                                      const rdb_call_options *options, int32_t *status, void *stream) {
    if (M < 0 || N < 0 || Kc < 0 || lda < Kc || ldb < (b_kmajor ? Kc : N)) return RDB_ERR_SHAPE;
    CallOpts o;
    int rc = resolve_opts(options, &o);
    if (rc) return rc;
    if (!dst_ptrs || ndst < 1 || ndst > RDB_MAX_PEERS || rows_per_dst <= 0 || (rows_per_dst % 32) != 0 ||
        (M + rows_per_dst - 1) / rows_per_dst > ndst || (dst_offset_bytes & 15))
        return RDB_ERR_PEER;
    if (M == 0 || N == 0) return RDB_OK;
    if (!a || !b) return RDB_ERR_NULL;
    void *dsts[RDB_MAX_PEERS];
    for (int i = 0; i < ndst; ++i) {
        if (!dst_ptrs[i] || (reinterpret_cast<uintptr_t>(dst_ptrs[i]) & 15)) return RDB_ERR_PEER;
        dsts[i] = reinterpret_cast<uint8_t *>(dst_ptrs[i]) + dst_offset_bytes;
    }
    if (M <= 128 || N <= 128 || !umma_shape_ok_dense(M, N, Kc, lda, ldb, N, RDB_BF16, 1, b_kmajor, a, b, dsts[0]))
        return RDB_ERR_UNSUPPORTED;
    return umma_gemm_dense_scatter(dsts, ndst, rows_per_dst, a, b, M, N, Kc, lda, ldb, b_kmajor, status, (cudaStream_t)stream, o);
}

extern "C" int rdb_gemm_dense(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda,
                              int64_t ldb, int64_t ldd, int a_dtype, int b_dtype, int d_dtype, int a_kmajor, int b_kmajor,
                              int impl, int32_t *status, void *stream) {
    return rdb_gemm_dense_ex(d, a, b, nullptr, 0, M, N, Kc, lda, ldb, ldd, a_dtype, b_dtype, d_dtype, a_kmajor, b_kmajor, impl,
                             nullptr, status, stream);
}

extern "C" int rdb_gemm_dense_ws(void *d, const void *a, const void *b, void *workspace, size_t workspace_bytes, int64_t M,
                                 int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int a_dtype, int b_dtype,
                                 int d_dtype, int a_kmajor, int b_kmajor, int impl, int32_t *status, void *stream) {
    return rdb_gemm_dense_ex(d, a, b, workspace, workspace_bytes, M, N, Kc, lda, ldb, ldd, a_dtype, b_dtype, d_dtype, a_kmajor,
                             b_kmajor, impl, nullptr, status, stream);
}

extern "C" size_t rdb_linear_workspace_bytes_ex(int op, int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path,
                                                int impl, const rdb_call_options *options) {
    if (T <= 0 || K <= 0 || N <= 0 || R <= 0) return 0;
    CallOpts o;
    if (resolve_opts(options, &o)) return 0;
    const int p = choose_path(path, T, K, N, R);
    const int im = choose_impl(impl, T, K, N, R, dtype, p, true);
    if (im < 0) return 0;
    return ws_layout(op, T, K, N, R, p, im, o, dtype).total;
}

extern "C" size_t rdb_linear_workspace_bytes(int op, int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path,
                                             int impl) {
    return rdb_linear_workspace_bytes_ex(op, T, K, N, R, dtype, path, impl, nullptr);
}

extern "C" int rdb_linear_stages_noise_ex(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl,
                                          const rdb_call_options *options) {
    if (T <= 0 || K <= 0 || N <= 0 || R <= 0) return 0;
    CallOpts o;
    int rc = resolve_opts(options, &o);
    if (rc) return rc;
    const int p = choose_path(path, T, K, N, R);
    const int im = choose_impl(impl, T, K, N, R, dtype, p, true);
    if (im < 0) return im;
    if (im != RDB_IMPL_UMMA) return 0;
    if (p == RDB_PATH_WPATH) return 3;
    return (stage_noise(0, T, N, R, o) ? 1 : 0) | (stage_noise(1, T, N, R, o) ? 2 : 0);
}

extern "C" int rdb_linear_stages_noise(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl) {
    return rdb_linear_stages_noise_ex(T, K, N, R, dtype, path, impl, nullptr);
}

extern "C" int rdb_linear_path(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl) {
    if (T <= 0 || K <= 0 || N <= 0 || R <= 0) return RDB_PATH_FACTORED;
    if (dtype != RDB_F32 && dtype != RDB_BF16) return RDB_ERR_DTYPE;
    const int p = choose_path(path, T, K, N, R);
    const int im = choose_impl(impl, T, K, N, R, dtype, p, true);
    if (im < 0) return im;
    return p | (im << 8);
}

// whether rdb_linear_bwd would run dX beside dC for this problem, and on how many CTA pairs each
static bool grads_beside(int64_t T, int64_t K, int64_t R, const CallOpts &o, int *pairs_dx, int *pairs_dc) {
    return o.grads_beside && o.dense_pair && dense_split_k_slices(R, K, T) == 1 &&
           dense_beside_plan(T, K, R, R, K, T, o.reserve_sms, o.grads_beside == 2, pairs_dx, pairs_dc);
}

extern "C" int rdb_linear_bwd_plan(int64_t T, int64_t K, int64_t N, int64_t R, int dtype, int path, int impl,
                                   const rdb_call_options *options, int *pairs_dx, int *pairs_dc) {
    if (pairs_dx) *pairs_dx = 0;
    if (pairs_dc) *pairs_dc = 0;
    if (T <= 0 || K <= 0 || N <= 0 || R <= 0) return 0;
    if (dtype != RDB_F32 && dtype != RDB_BF16) return RDB_ERR_DTYPE;
    CallOpts o;
    int rc = resolve_opts(options, &o);
    if (rc) return rc;
    const int p = choose_path(path, T, K, N, R);
    const int im = choose_impl(impl, T, K, N, R, dtype, p, true);
    if (im < 0) return im;
    int a = 0, b = 0;
    if (p != RDB_PATH_FACTORED || im != RDB_IMPL_UMMA || !grads_beside(T, K, R, o, &a, &b)) return 0;
    if (pairs_dx) *pairs_dx = a;
    if (pairs_dc) *pairs_dc = b;
    return 1;
}

extern "C" int rdb_linear_weight(void *w, const void *coef, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed,
                                 int dtype, void *stream) {
    if (K < 0 || N < 0 || R < 0) return RDB_ERR_SHAPE;
    if (dtype != RDB_F32 && dtype != RDB_BF16) return RDB_ERR_DTYPE;
    if (K == 0 || N == 0) return RDB_OK;
    if (!w || (R > 0 && !coef)) return RDB_ERR_NULL;
    // W[o,i] = sum_r C[r,i] S[row0+o, r], written as D(m=i, n=o) at o*K + i
    return simt_gemm(w, dtype, 1, K, coef, dtype, 1, K, nullptr, RDB_F32, 0, 0, sq5_lin_rows(seed, (uint32_t)row0, 0), K, N,
                     R, (cudaStream_t)stream);
}

static int check_common(int64_t T, int64_t K, int64_t N, int64_t R, int dtype) {
    if (T < 0 || K < 0 || N < 0 || R < 0) return RDB_ERR_SHAPE;
    if (dtype != RDB_F32 && dtype != RDB_BF16) return RDB_ERR_DTYPE;
    return RDB_OK;
}

// S (bf16, N x R) into the workspace.  With `side` the fill runs on the library's extra stream, forked from the caller's
// stream here; join_side() makes the caller's stream wait for it.
static int fill_noise(void *S, int64_t N, int64_t R, int64_t row0, uint32_t seed, cudaStream_t st, SideStream *side) {
    if (!side) return rdb_noise(S, RDB_BF16, N, R, R, row0, 0, seed, st);
    cudaError_t e = cudaEventRecord(side->fork, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
    if (e != cudaSuccess) return (int)e;
    int rc = rdb_noise(S, RDB_BF16, N, R, R, row0, 0, seed, side->stream);
    // the join is recorded even after a failed launch, so a captured fork always rejoins its origin
    e = cudaEventRecord(side->join, side->stream);
    if (rc) return rc;
    return e == cudaSuccess ? RDB_OK : (int)e;
}

static int join_side(cudaStream_t st, SideStream *side) {
    if (!side) return RDB_OK;
    cudaError_t e = cudaStreamWaitEvent(st, side->join, 0);
    return e == cudaSuccess ? RDB_OK : (int)e;
}

extern "C" int rdb_linear_fwd_ex(void *y, const void *x, const void *coef, void *workspace, size_t workspace_bytes, int64_t T,
                                 int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, int dtype, int path, int impl,
                                 const rdb_call_options *options, int32_t *status, void *stream) {
    int rc = check_common(T, K, N, R, dtype);
    if (rc) return rc;
    CallOpts o;
    rc = resolve_opts(options, &o);
    if (rc) return rc;
    if (T == 0 || N == 0) return RDB_OK;
    if (!y) return RDB_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (K == 0 || R == 0) {
        cudaError_t e = cudaMemsetAsync(y, 0, (size_t)T * N * dtype_size(dtype), st);
        return e == cudaSuccess ? RDB_OK : (int)e;
    }
    if (!x || !coef) return RDB_ERR_NULL;
    const int p = choose_path(path, T, K, N, R);
    const int im = choose_impl(impl, T, K, N, R, dtype, p, aligned16(x) && aligned16(coef) && aligned16(y));
    if (im < 0) return im;
    const WsLayout w = ws_layout(0, T, K, N, R, p, im, o, dtype);
    if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return RDB_ERR_WORKSPACE;
    uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
    const Sq5Lin rows = sq5_lin_rows(seed, (uint32_t)row0, 0);
    const Sq5Lin none{0, 0, 0};

    if (p == RDB_PATH_FACTORED) {
        if (im == RDB_IMPL_UMMA) {
            void *z = ws + w.off[0];
            const bool staged = stage_noise(0, T, N, R, o);
            void *S = ws + w.off[1];
            // the hash of S (integer ALU) does not depend on z = x C^T (tensor pipe), so a long fill runs beside that product,
            // and so does one so short that it is all launch latency (at most 1 Mi elements: the 24 layers of the
            // GPT-2-shaped workload 0.620 -> 0.600 ms forward).  In between it does not: the fill's two thousand resident
            // threads per SM slow the product's single MMA-issuing thread down by about as much as the fill takes (measured:
            // 16.8 M elements beside a 40-50 us product lose, 67 M and more beside a 100-180 us product win 20 us)
            const double s_elems = (double)N * (double)R;
            const bool beside = o.fill_overlap == 2 || (o.fill_overlap == 1 && (s_elems >= 64.0 * 1024 * 1024 || s_elems <= 1024.0 * 1024));
            SideStream *side = (staged && beside) ? side_stream(st) : nullptr;
            std::unique_lock<std::mutex> side_lock;
            if (side) side_lock = std::unique_lock<std::mutex>(side->mu);
            if (staged && side) {
                rc = fill_noise(S, N, R, row0, seed, st, side);
                if (rc) {
                    (void)join_side(st, side);
                    return rc;
                }
            }
            const int sz = dense_split_k_slices(T, R, K);
            if (sz > 1)
                rc = umma_gemm_dense_split_k(z, x, coef, reinterpret_cast<float *>(ws + w.off[2]), sz, T, R, K, K, K, RDB_BF16, 1, 1,
                                             status, st, o);
            else
                rc = umma_gemm_dense(z, x, coef, T, R, K, K, K, R, RDB_BF16, 1, 1, status, st, o);
            if (staged) {
                const int rj = side ? join_side(st, side) : fill_noise(S, N, R, row0, seed, st, nullptr);
                if (rc == RDB_OK) rc = rj;
            }
            if (side) side_lock.unlock();
            if (rc) return rc;
            if (staged) return umma_gemm_dense(y, z, S, T, N, R, R, R, N, RDB_BF16, 1, 1, status, st, o);   // y = z S^T
            return umma_gemm_noise(y, z, T, N, R, R, N, rows, status, st, o);
        }
        if (dtype == RDB_F32 && T == 1)
            return rdb_gemv_fwd((float *)y, (const float *)x, (const float *)coef, (float *)(ws + w.off[0]), K, N, R, row0,
                                seed, stream);
        float *z = reinterpret_cast<float *>(ws + w.off[0]);
        rc = simt_gemm(z, RDB_F32, R, 1, x, dtype, K, 1, coef, dtype, K, 1, none, T, R, K, st);
        if (rc) return rc;
        return simt_gemm(y, dtype, N, 1, z, RDB_F32, R, 1, nullptr, RDB_F32, 0, 0, rows, T, N, R, st);
    }
    if (im == RDB_IMPL_UMMA) {
        // W path on the tensor cores: S hashed once into the workspace, W = S C (bf16, the dtype the reference casts its
        // materialised weight to: src/rten_cpp/RandumbTensor.py:892), y = x W^T.  W lives in the workspace for this call only.
        void *S = ws + w.off[0], *W = ws + w.off[1];
        rc = fill_noise(S, N, R, row0, seed, st, nullptr);
        if (rc) return rc;
        rc = umma_gemm_dense(W, S, coef, N, K, R, R, K, K, RDB_BF16, 1, 0, status, st, o);     // C read in place as an MN-major operand
        if (rc) return rc;
        return umma_gemm_dense(y, x, W, T, N, K, K, K, N, RDB_BF16, 1, 1, status, st, o);
    }
    // W path: W[o,i] = sum_r S[row0+o, r] C[r,i], written as D(m=i, n=o) at o*K + i
    float *W = reinterpret_cast<float *>(ws + w.off[0]);
    rc = simt_gemm(W, RDB_F32, 1, K, coef, dtype, 1, K, nullptr, RDB_F32, 0, 0, rows, K, N, R, st);
    if (rc) return rc;
    return simt_gemm(y, dtype, N, 1, x, dtype, K, 1, W, RDB_F32, K, 1, none, T, N, K, st);
}

extern "C" int rdb_linear_fwd(void *y, const void *x, const void *coef, void *workspace, size_t workspace_bytes, int64_t T,
                              int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed, int dtype, int path, int impl,
                              int32_t *status, void *stream) {
    return rdb_linear_fwd_ex(y, x, coef, workspace, workspace_bytes, T, K, N, R, row0, seed, dtype, path, impl, nullptr, status,
                             stream);
}

extern "C" int rdb_linear_bwd_ex(void *dx, void *dc, const void *dy, const void *x, const void *coef, void *workspace,
                                 size_t workspace_bytes, int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed,
                                 int dtype, int path, int impl, const rdb_call_options *options, int32_t *status, void *stream) {
    int rc = check_common(T, K, N, R, dtype);
    if (rc) return rc;
    CallOpts o;
    rc = resolve_opts(options, &o);
    if (rc) return rc;
    if (!dx && !dc) return RDB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = dtype_size(dtype);
    if (T == 0 || N == 0 || R == 0 || K == 0) {
        cudaError_t e = cudaSuccess;
        if (dx && T > 0 && K > 0) e = cudaMemsetAsync(dx, 0, (size_t)T * K * es, st);
        if (e == cudaSuccess && dc && R > 0 && K > 0) e = cudaMemsetAsync(dc, 0, (size_t)R * K * es, st);
        return e == cudaSuccess ? RDB_OK : (int)e;
    }
    if (!dy || (dx && !coef) || (dc && !x)) return RDB_ERR_NULL;
    const int p = choose_path(path, T, K, N, R);
    const bool al = aligned16(dy) && aligned16(dx) && aligned16(dc) && (!dx || aligned16(coef)) && (!dc || aligned16(x));
    const int im = choose_impl(impl, T, K, N, R, dtype, p, al);
    if (im < 0) return im;
    const WsLayout w = ws_layout(1, T, K, N, R, p, im, o, dtype);
    if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return RDB_ERR_WORKSPACE;
    uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
    const Sq5Lin rows = sq5_lin_rows(seed, (uint32_t)row0, 0);
    const Sq5Lin cols = sq5_lin_cols(seed, (uint32_t)row0, 0);
    const Sq5Lin none{0, 0, 0};

    if (p == RDB_PATH_FACTORED) {
        if (im == RDB_IMPL_UMMA) {
            void *g = ws + w.off[0];
            // g = dY S ; dX = g C (C read in place as an MN-major B operand) ; dC = g^T x (both operands MN-major)
            if (stage_noise(1, T, N, R, o)) {
                void *S = ws + w.off[1];
                rc = fill_noise(S, N, R, row0, seed, st, nullptr);
                if (rc) return rc;
                const int sg = dense_split_k_slices(T, R, N);
                if (sg > 1)
                    rc = umma_gemm_dense_split_k(g, dy, S, reinterpret_cast<float *>(ws + w.off[2]), sg, T, R, N, N, R, RDB_BF16, 1, 0,
                                                 status, st, o);
                else
                    rc = umma_gemm_dense(g, dy, S, T, R, N, N, R, R, RDB_BF16, 1, 0, status, st, o);    // S read as an MN-major operand
            } else {
                rc = umma_gemm_noise(g, dy, T, R, N, N, R, cols, status, st, o);
            }
            if (rc) return rc;
            // dX and dC both read g and nothing of one another: when their tile lists pack better side by side than one after
            // the other, dX goes to the library's own stream on some of the CTA pairs and dC stays here on the rest
            int pairs_dx = 0, pairs_dc = 0;
            if (dx && dc && grads_beside(T, K, R, o, &pairs_dx, &pairs_dc)) {
                if (SideStream *side = side_stream(st)) {
                    std::lock_guard<std::mutex> side_lock(side->mu);
                    cudaError_t e = cudaEventRecord(side->fork, st);
                    if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
                    if (e != cudaSuccess) return (int)e;
                    rc = umma_gemm_dense_on_pairs(dx, g, coef, T, K, R, R, K, K, 1, 0, pairs_dx, status, side->stream);
                    // the join is recorded and waited for even after a failed launch, so a captured fork always rejoins
                    e = cudaEventRecord(side->join, side->stream);
                    const int rc2 = rc ? rc : umma_gemm_dense_on_pairs(dc, g, x, R, K, T, R, K, K, 0, 0, pairs_dc, status, st);
                    const cudaError_t ej = (e == cudaSuccess) ? cudaStreamWaitEvent(st, side->join, 0) : e;
                    if (rc2) return rc2;
                    return ej == cudaSuccess ? RDB_OK : (int)ej;
                }
            }
            if (dx) {
                rc = umma_gemm_dense(dx, g, coef, T, K, R, R, K, K, RDB_BF16, 1, 0, status, st, o);
                if (rc) return rc;
            }
            if (dc) {
                const int split = dense_split_k_slices(R, K, T);
                if (split > 1)
                    rc = umma_gemm_dense_split_k(dc, g, x, reinterpret_cast<float *>(ws + w.off[2]), split, R, K, T, R, K, RDB_BF16, 0,
                                                 0, status, st, o);
                else
                    rc = umma_gemm_dense(dc, g, x, R, K, T, R, K, K, RDB_BF16, 0, 0, status, st, o);
                if (rc) return rc;
            }
            return RDB_OK;
        }
        if (dtype == RDB_F32 && T == 1)
            return rdb_gemv_bwd((float *)dx, (float *)dc, (const float *)dy, (const float *)x, (const float *)coef,
                                (float *)(ws + w.off[0]), K, N, R, row0, seed, stream);
        float *g = reinterpret_cast<float *>(ws + w.off[0]);
        rc = simt_gemm(g, RDB_F32, R, 1, dy, dtype, N, 1, nullptr, RDB_F32, 0, 0, cols, T, R, N, st);
        if (rc) return rc;
        if (dx) {
            rc = simt_gemm(dx, dtype, K, 1, g, RDB_F32, R, 1, coef, dtype, 1, K, none, T, K, R, st);
            if (rc) return rc;
        }
        if (dc) {
            rc = simt_gemm(dc, dtype, K, 1, g, RDB_F32, 1, R, x, dtype, 1, K, none, R, K, T, st);
            if (rc) return rc;
        }
        return RDB_OK;
    }
    if (im == RDB_IMPL_UMMA) {
        // W path on the tensor cores: dX = dY W with W = S C rebuilt in the workspace; dC = S^T dW with dW = dY^T x (bf16)
        void *S = ws + w.off[0], *W = ws + w.off[1], *dW = ws + w.off[2];
        rc = fill_noise(S, N, R, row0, seed, st, nullptr);
        if (rc) return rc;
        if (dx) {
            rc = umma_gemm_dense(W, S, coef, N, K, R, R, K, K, RDB_BF16, 1, 0, status, st, o);
            if (rc) return rc;
            rc = umma_gemm_dense(dx, dy, W, T, K, N, N, K, K, RDB_BF16, 1, 0, status, st, o);      // W [N,K] read as an MN-major operand
            if (rc) return rc;
        }
        if (dc) {
            rc = umma_gemm_dense(dW, dy, x, N, K, T, N, K, K, RDB_BF16, 0, 0, status, st, o);      // dW[o,i] = sum_t dY[t,o] x[t,i]
            if (rc) return rc;
            rc = umma_gemm_dense(dc, S, dW, R, K, N, R, K, K, RDB_BF16, 0, 0, status, st, o);      // dC[r,i] = sum_o S[o,r] dW[o,i]
            if (rc) return rc;
        }
        return RDB_OK;
    }
    // W path
    float *W = reinterpret_cast<float *>(ws + w.off[0]);
    float *dW = reinterpret_cast<float *>(ws + w.off[1]);
    if (dx) {
        rc = simt_gemm(W, RDB_F32, 1, K, coef, dtype, 1, K, nullptr, RDB_F32, 0, 0, rows, K, N, R, st);
        if (rc) return rc;
        rc = simt_gemm(dx, dtype, K, 1, dy, dtype, N, 1, W, RDB_F32, 1, K, none, T, K, N, st);
        if (rc) return rc;
    }
    if (dc) {
        // dW[o,i] = sum_t dY[t,o] x[t,i] ; dC[r,i] = sum_o S[row0+o, r] dW[o,i], written as D(m=i, n=r) at r*K + i
        rc = simt_gemm(dW, RDB_F32, K, 1, dy, dtype, 1, N, x, dtype, 1, K, none, N, K, T, st);
        if (rc) return rc;
        rc = simt_gemm(dc, dtype, 1, K, dW, RDB_F32, 1, K, nullptr, RDB_F32, 0, 0, cols, K, R, N, st);
        if (rc) return rc;
    }
    return RDB_OK;
}

extern "C" int rdb_linear_bwd(void *dx, void *dc, const void *dy, const void *x, const void *coef, void *workspace,
                              size_t workspace_bytes, int64_t T, int64_t K, int64_t N, int64_t R, int64_t row0, uint32_t seed,
                              int dtype, int path, int impl, int32_t *status, void *stream) {
    return rdb_linear_bwd_ex(dx, dc, dy, x, coef, workspace, workspace_bytes, T, K, N, R, row0, seed, dtype, path, impl, nullptr,
                             status, stream);
}
