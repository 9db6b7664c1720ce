// bf16 tensor-core (tcgen05 / TMEM / TMA) kernels of the pseudorandom-weight layer.
//
// Persistent, warp-specialised kernels, one CTA per SM:
//
//  noise_gemm_kernel   D[M,N] = A[M,Kc] * G^T  where the B operand G is never read from memory:
//                      generator warps hash (seed, row, k) with 32-bit integer ALU ops in
//                      registers, convert to bf16 and write the tile straight into shared
//                      memory in the 128-byte-swizzled K-major layout the MMA descriptor
//                      expects, while a TMA warp stages the A tiles beside it.  One generated
//                      [BN x 64] stage is consumed by MT token sub-tiles (MT*128 rows of A), so
//                      every hash is amortised over MT*128 tokens.
//  noise_pair_kernel   the same product on CTA pairs (cta_group::2 MMAs, 512 tokens x 256 generated rows).
//                      Both serve y = z S^T and g = dY S (transposed walk) when S is regenerated per tile.
//
//  dense_pair_kernel   D[M,N] = op(A) op(B)^T with both operands staged by TMA (K-major or MN-major) on CTA
//                      pairs: 512 x 256 tiles, each CTA stages its own rows of A and its own half of B.
//  dense_gemm_kernel   the same on single CTAs: 128 x 256 tiles, double-buffered TMEM accumulators so the
//                      epilogue of one tile overlaps the main loop of the next.
//                      They serve z = x C^T, dX = g C, dC = g^T x, and y / g on a staged copy of S.
//
// The reference has no tensor-core path for any of this: its fused attempt runs tl.dot in IEEE
// float32 (src/rten_cpp/RandumbTensor.py:539, 725) and the production path materialises W and
// calls cuBLAS (:780, :786-787).
//
// Every barrier wait is bounded (ptx::mbar_wait); a role that gives up raises the CTA's abort
// flag, writes a code to status[0] and all roles fall through to the common teardown, which
// releases TMEM.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "umma.cuh"

namespace rdb {

using namespace ptx;

constexpr int BM = 128;            // rows of one MMA (TMEM lanes)
constexpr int BK = 64;             // bf16 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;         // K extent of one tcgen05.mma for 16-bit inputs
constexpr int SUB_BYTES = BM * BK * 2;  // one [128 x 64] bf16 sub-tile
constexpr int TMEM_COLS = 512;

// ------------------------------------------------------------------------------------------------
// epilogue helpers: one thread owns one accumulator row, 32 consecutive columns in registers
// ------------------------------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT *dst, const uint32_t (&r)[32], int ncols);

template <>
__device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16 *dst, const uint32_t (&r)[32], int ncols) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        if (v * 8 < ncols) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t *>(&h);
            }
            *reinterpret_cast<uint4 *>(dst + v * 8) = make_uint4(p[0], p[1], p[2], p[3]);
        }
    }
}

template <>
__device__ __forceinline__ void store_row32<float>(float *dst, const uint32_t (&r)[32], int ncols) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
        if (v * 4 < ncols)
            *reinterpret_cast<uint4 *>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
    }
}

// One 32-column slice of an accumulator row -> 32 bf16 = 64 contiguous bytes of the output row.
__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16 *dst, const uint32_t (&r)[32], int ncols, bool wide) {
    uint32_t p[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        p[j] = *reinterpret_cast<uint32_t *>(&h);
    }
    if (wide && ncols == 32) {   // two 256-bit stores: whole 32-byte sectors per instruction
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(p[0]), "r"(p[1]), "r"(p[2]),
                     "r"(p[3]), "r"(p[4]), "r"(p[5]), "r"(p[6]), "r"(p[7]) : "memory");
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16), "r"(p[8]), "r"(p[9]), "r"(p[10]),
                     "r"(p[11]), "r"(p[12]), "r"(p[13]), "r"(p[14]), "r"(p[15]) : "memory");
    } else {
#pragma unroll
        for (int v = 0; v < 4; ++v)
            if (v * 8 < ncols) *reinterpret_cast<uint4 *>(dst + v * 8) = make_uint4(p[4 * v], p[4 * v + 1], p[4 * v + 2], p[4 * v + 3]);
    }
}

struct PipeState {
    uint32_t idx = 0, phase = 0;
    template <int STAGES> __device__ __forceinline__ void advance() {
        if (++idx == STAGES) { idx = 0; phase ^= 1; }
    }
};

__device__ __forceinline__ void raise_abort(volatile int *abort_flag, int32_t *status, int code) {
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, code);
}

// ================================================================================================
// noise_gemm_kernel
// ================================================================================================
template <int CS, int MT, int BN, int SA, int SB>
struct NoiseCfg {
    static constexpr int A_STAGE = MT * SUB_BYTES;
    static constexpr int B_STAGE = BN * BK * 2;
    static constexpr int GEN_WARPS = 8;
    static constexpr int GEN_THREADS = GEN_WARPS * 32;
    static constexpr int THREADS = (2 + 4 + GEN_WARPS) * 32;
    static constexpr int FIRST_EPI_WARP = 2;
    static constexpr int FIRST_GEN_WARP = 6;
    static constexpr int SMEM_DYN = SA * A_STAGE + SB * B_STAGE + 1024;
    static constexpr int ROWS_PER_CTA = BN / CS;                       // noise rows of a stage this CTA generates
    static constexpr int CHUNKS = (ROWS_PER_CTA * 8) / GEN_THREADS;    // 16-byte chunks per generator thread per stage
    static_assert(MT * BN <= TMEM_COLS, "accumulators exceed TMEM");
    static_assert(BN % 64 == 0 && BN <= 256, "BN");
    static_assert(CS == 1 || CS == 2 || CS == 4 || CS == 8, "cluster size");
    static_assert(BN % CS == 0 && (ROWS_PER_CTA * 8) % GEN_THREADS == 0 && CHUNKS >= 1, "generator chunking");
};

// CS CTAs of a thread-block cluster work on CS token tiles against the SAME generated operand: each CTA
// hashes 1/CS of every [BN x 64] stage and stores its part into the shared memory of all CS CTAs
// (distributed shared memory), so one hash is amortised over CS * MT * 128 tokens.
template <int CS, int MT, int BN, int SA, int SB>
__global__ void __launch_bounds__(NoiseCfg<CS, MT, BN, SA, SB>::THREADS, 1)
noise_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, __nv_bfloat16 *__restrict__ d, int64_t ldd, int64_t M,
                  int64_t N, int64_t Kc, Sq5Lin lin, int32_t *status, long long *prof) {
    using Cfg = NoiseCfg<CS, MT, BN, SA, SB>;
    // prof (optional): 8 cycle counters per CTA -- where each role waits; see rdb_set_profile_buffer
    long long pc0 = 0, pc1 = 0, pc2 = 0, pc3 = 0, pc4 = 0, pc5 = 0;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full_a[SA], bar_empty_a[SA], bar_full_b[SB], bar_empty_b[SB], bar_tmem_full, bar_tmem_empty;
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;

    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    const uint32_t smem_a = raw_addr + pad;
    const uint32_t smem_b = smem_a + SA * Cfg::A_STAGE;
    uint8_t *smem_gen = smem_raw + pad;   // generic pointer to the same place as smem_a

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CS > 1) ? cluster_ctarank() : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) { mbar_init(smem_u32(&bar_full_a[s]), 1); mbar_init(smem_u32(&bar_empty_a[s]), 1); }
        for (int s = 0; s < SB; ++s) {
            // single CTA: every generator thread arrives.  cluster: one local arrive.expect_tx per phase and the
            // stage's bytes land as asynchronous stores from all CTAs, each completing its transaction bytes.
            mbar_init(smem_u32(&bar_full_b[s]), CS > 1 ? 1 : Cfg::GEN_THREADS);
            mbar_init(smem_u32(&bar_empty_b[s]), CS);                   // one MMA commit from every CTA
        }
        mbar_init(smem_u32(&bar_tmem_full), 1);
        mbar_init(smem_u32(&bar_tmem_empty), 128);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_holder), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CS > 1) cluster_sync_all();   // peers must see initialised barriers before any remote arrive
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    volatile int *abortp = &abort_flag;
    pdl_launch_dependents();   // the next kernel of the stream may start its own prologue
    pdl_wait();                // ... and this one touches global memory only after its predecessor has completed

    const int64_t tiles_n = (N + BN - 1) / BN;
    const int64_t tiles_m = (M + (int64_t)MT * BM - 1) / ((int64_t)MT * BM);
    const int64_t ctiles_m = (tiles_m + CS - 1) / CS;          // cluster tiles along tokens
    const int64_t total_ctiles = ctiles_m * tiles_n;
    const int64_t cluster_id = blockIdx.x / CS;
    const int64_t num_clusters = gridDim.x / CS;
    const int num_kb = (int)((Kc + BK - 1) / BK);
    // token tile of this CTA inside cluster tile `ct` (may lie past the end: loads zero-fill, stores are masked)
    auto m_base = [&](int64_t ct) { return ((ct / tiles_n) * CS + cta_rank) * (int64_t)MT * BM; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (A tiles)
        if (lane == 0) {
            prefetch_tmap(&tmap_a);
            PipeState st;
            bool ok = true;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                const int64_t m0 = m_base(ct);
                for (int kb = 0; kb < num_kb; ++kb) {
                    const long long tw = prof ? clock64() : 0;
                    if (!mbar_wait(smem_u32(&bar_empty_a[st.idx]), st.phase ^ 1, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (prof) pc0 += clock64() - tw;
                    const uint32_t fb = smem_u32(&bar_full_a[st.idx]);
                    mbar_arrive_expect_tx(fb, Cfg::A_STAGE);
#pragma unroll
                    for (int s = 0; s < MT; ++s)
                        tma_load_2d(smem_a + st.idx * Cfg::A_STAGE + s * SUB_BYTES, &tmap_a, fb, kb * BK,
                                    (int32_t)(m0 + s * BM));
                    st.advance<SA>();
                }
            }
            if (prof) prof[blockIdx.x * 16 + 4] = pc0;
            // Loads still in flight complete on their own barriers; wait for them (bounded) so the
            // CTA does not retire with copies targeting its shared memory.
            if (!ok) {
                for (int s = 0; s < SA; ++s) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&bar_full_a[s]), 0) && !mbar_try_wait(smem_u32(&bar_full_a[s]), 1)) {
                        if (clock64() - t0 > 20000000LL) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN, 0, 0);
            PipeState sa, sb;
            uint32_t tphase = 0;
            bool ok = true;
            const long long t_start = prof ? clock64() : 0;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                long long tw = prof ? clock64() : 0;
                if (!mbar_wait(smem_u32(&bar_tmem_empty), tphase ^ 1, abortp)) {
                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                    break;
                }
                if (prof) pc2 += clock64() - tw;
                tc_fence_after_sync();
                for (int kb = 0; kb < num_kb; ++kb) {
                    tw = prof ? clock64() : 0;
                    const bool got_a = mbar_wait(smem_u32(&bar_full_a[sa.idx]), sa.phase, abortp);
                    const long long tw2 = prof ? clock64() : 0;
                    const bool got_b = got_a && (CS > 1 ? mbar_wait_cluster(smem_u32(&bar_full_b[sb.idx]), sb.phase, abortp)
                                                        : mbar_wait(smem_u32(&bar_full_b[sb.idx]), sb.phase, abortp));
                    if (prof) { pc0 += tw2 - tw; pc1 += clock64() - tw2; }
                    if (!got_b) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    const long long tf0 = prof ? clock64() : 0;
                    if (CS > 1) fence_proxy_async_smem();  // the stage arrived as stores from other threads/CTAs
                    tc_fence_after_sync();
                    const long long tf1 = prof ? clock64() : 0;
                    // descriptors: constant high word, low word = stage address field + a compile-time step
                    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
                    const uint32_t a_lo = smem_desc_lo(smem_a + sa.idx * Cfg::A_STAGE, 0);
                    const uint32_t b_lo = smem_desc_lo(smem_b + sb.idx * Cfg::B_STAGE, 0);
#pragma unroll
                    for (int s = 0; s < MT; ++s) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t adesc = pack_desc(a_lo + ((s * SUB_BYTES + k * UMMA_K * 2) >> 4), desc_hi);
                            const uint64_t bdesc = pack_desc(b_lo + ((k * UMMA_K * 2) >> 4), desc_hi);
                            umma_bf16(tmem_base + s * BN, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    const long long tf2 = prof ? clock64() : 0;
                    umma_commit(smem_u32(&bar_empty_a[sa.idx]));
                    // the stage is rewritten by every CTA's generators: tell all of them it is free here
                    if (CS > 1) {
#pragma unroll
                        for (int c = 0; c < CS; ++c) umma_commit(mapa(smem_u32(&bar_empty_b[sb.idx]), (uint32_t)c));
                    } else {
                        umma_commit(smem_u32(&bar_empty_b[sb.idx]));
                    }
                    if (prof) { pc3 += tf1 - tf0; pc4 += tf2 - tf1; pc5 += clock64() - tf2; }
                    sa.advance<SA>();
                    sb.advance<SB>();
                }
                if (ok) umma_commit(smem_u32(&bar_tmem_full));
                tphase ^= 1;
            }
            if (prof) {
                prof[blockIdx.x * 16 + 0] = pc0;
                prof[blockIdx.x * 16 + 1] = pc1;
                prof[blockIdx.x * 16 + 2] = pc2;
                prof[blockIdx.x * 16 + 3] = clock64() - t_start;
                prof[blockIdx.x * 16 + 8] = pc3;
                prof[blockIdx.x * 16 + 9] = pc4;
                prof[blockIdx.x * 16 + 10] = pc5;
            }
        }
    } else if (warp < Cfg::FIRST_GEN_WARP) {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        uint32_t tphase = 0;
        for (int64_t ct = cluster_id; ct < total_ctiles; ct += num_clusters) {
            const int64_t m0 = m_base(ct);
            const int64_t n0 = (ct % tiles_n) * BN;
            if (!mbar_wait_warp<false>(smem_u32(&bar_tmem_full), tphase, abortp)) {
                raise_abort(abortp, status, RDB_STATUS_TIMEOUT_EPILOGUE);
                break;
            }
            const long long te = prof ? clock64() : 0;
            tc_fence_after_sync();
#pragma unroll 1
            for (int s = 0; s < MT; ++s) {
                const int64_t row = m0 + s * BM + q * 32 + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    // two 32-column loads in flight per wait
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * BN + c0);
                    tmem_ld_32x32(taddr, r0);
                    tmem_ld_32x32(taddr + 32, r1);
                    tmem_ld_wait();
                    const int64_t col = n0 + c0;
                    const int nc0 = (int)((N - col) < 32 ? (N - col) : 32);
                    const int nc1 = (int)((N - col - 32) < 32 ? (N - col - 32) : 32);
                    if (row < M) {
                        if (nc0 > 0) store_row32<__nv_bfloat16>(d + row * ldd + col, r0, nc0);
                        if (nc1 > 0) store_row32<__nv_bfloat16>(d + row * ldd + col + 32, r1, nc1);
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bar_tmem_empty));
            tphase ^= 1;
            if (prof) pc0 += clock64() - te;
        }
        if (prof && warp == Cfg::FIRST_EPI_WARP && lane == 0) prof[blockIdx.x * 16 + 7] = pc0;
    } else {
        // ------------------------------------------------------------------ generators (8 warps)
        const int tg = threadIdx.x - Cfg::FIRST_GEN_WARP * 32;
        constexpr int CHUNKS = Cfg::CHUNKS;
        PipeState sb;
        bool ok = true;
        for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
            const int64_t n0 = (ct % tiles_n) * BN;
            // hash front end b0 of this thread's chunks at k-block 0, and their swizzled offsets in a stage
            uint32_t bstart[CHUNKS];
            uint32_t soff[CHUNKS];
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int id = tg + c * Cfg::GEN_THREADS;
                const int rowi = (int)cta_rank * Cfg::ROWS_PER_CTA + (id >> 3), ch = id & 7;
                bstart[c] = lin.base + (uint32_t)(n0 + rowi) * lin.sn + (uint32_t)(ch * 8) * lin.sk;
                soff[c] = (uint32_t)(rowi * 128 + ((ch ^ (rowi & 7)) << 4));
            }
            const uint32_t kb_step = (uint32_t)BK * lin.sk;
            for (int kb = 0; kb < num_kb; ++kb) {
                const uint32_t eb = smem_u32(&bar_empty_b[sb.idx]);
                const long long tw = prof ? clock64() : 0;
                if (!(CS > 1 ? mbar_wait_cluster(eb, sb.phase ^ 1, abortp) : mbar_wait(eb, sb.phase ^ 1, abortp))) {
                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_GENERATOR);
                    ok = false;
                    break;
                }
                const long long tc = prof ? clock64() : 0;
                const uint32_t stage = smem_b + sb.idx * Cfg::B_STAGE;
                const uint32_t fb = smem_u32(&bar_full_b[sb.idx]);
                if (CS > 1 && tg == 0) mbar_arrive_expect_tx(fb, Cfg::B_STAGE);   // this phase's local arrival + byte count
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    uint32_t p[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        p[j] = sq5_pack_bf16x2(sq5_tail(bstart[c] + (uint32_t)(2 * j) * lin.sk), sq5_tail(bstart[c] + (uint32_t)(2 * j + 1) * lin.sk));
                    }
                    if (CS > 1) {
#pragma unroll
                        for (int dst = 0; dst < CS; ++dst)
                            st_async_v4(mapa(stage + soff[c], (uint32_t)dst), p[0], p[1], p[2], p[3], mapa(fb, (uint32_t)dst));
                    } else {
                        *reinterpret_cast<uint4 *>(smem_gen + (stage - smem_a) + soff[c]) = make_uint4(p[0], p[1], p[2], p[3]);
                    }
                    bstart[c] += kb_step;
                }
                if (CS == 1) {
                    fence_proxy_async_smem();
                    mbar_arrive(fb);
                }
                if (prof) { pc0 += tc - tw; pc1 += clock64() - tc; }
                sb.advance<SB>();
            }
        }
        if (prof && tg == 0) {
            prof[blockIdx.x * 16 + 5] = pc0;
            prof[blockIdx.x * 16 + 6] = pc1;
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (CS > 1) cluster_sync_all();   // no CTA retires while a peer may still write into it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ================================================================================================
// noise_pair_kernel: the generated-operand product on CTA pairs (tcgen05 cta_group::2)
// ================================================================================================
// A pair of CTAs computes 512 tokens x 256 generated rows per work unit.  Every MMA has M = 256 (rows
// 0-127 from the even CTA's shared memory and TMEM, rows 128-255 from the odd CTA's), N = 256 with each CTA
// holding one half (128 rows) of the generated operand, so a CTA reads only 8 KB of shared memory per MMA
// instead of 12 KB and the tensor pipe is no longer limited by shared-memory bandwidth.
// NP pairs form one thread-block cluster (2*NP CTAs) and work on NP token tiles against the SAME generated
// rows: the NP CTAs that need the same half hash 128/NP rows each and send their 16-byte chunks to each
// other with asynchronous distributed-shared-memory stores (transaction bytes complete the receiver's
// `full` barrier).  Only plain TMA loads, st.async, mapa, remote mbarrier arrives and cluster barriers cross
// CTAs.
//
// Per-CTA barriers of ring stage s:
//   full[s]      A sub-tiles (TMA) and this CTA's half of the generated stage (st.async) have landed;
//                on the even CTA it also counts one arrival from the odd CTA ("my part is in place too")
//   free_[s]     the pair's MMAs have finished reading the stage (commit from the even CTA's MMA thread)
//   free_all[s]  ... in all NP CTAs that receive the same generated half (NP > 1)
template <int NP, int D>
struct PairCfg {
    static constexpr int MT = 2;                                       // accumulators per CTA (256 columns each)
    static constexpr int BN = 256;                                     // generated rows per work unit
    static constexpr int HALF = BN / 2;                                // ... of which this CTA holds 128
    static constexpr int A_PART = MT * SUB_BYTES;
    static constexpr int B_PART = HALF * BK * 2;
    static constexpr int STAGE = A_PART + B_PART;
    static constexpr int GEN_WARPS = 8;
    static constexpr int GEN_THREADS = GEN_WARPS * 32;
    static constexpr int FIRST_EPI_WARP = 2;
    static constexpr int FIRST_GEN_WARP = 6;
    static constexpr int FULL_RELAY_WARP = FIRST_GEN_WARP + GEN_WARPS;  // odd CTA -> even CTA: "stage is full here"
    static constexpr int FREE_RELAY_WARP = FULL_RELAY_WARP + 1;         // "stage is free here" -> the CTAs that write into it
    static constexpr int THREADS = (FREE_RELAY_WARP + 1) * 32;
    static constexpr int OUT_STAGING = 4 * 2 * 32 * 128;               // per epilogue warp: two [32 rows x 64 columns] bf16 boxes
    static constexpr int SMEM_DYN = D * STAGE + OUT_STAGING + 1024;
    static constexpr int GEN_ROWS = HALF / NP;                          // rows of the half this CTA hashes
    static constexpr int CHUNKS = (GEN_ROWS * 8) / GEN_THREADS;
    static_assert(NP == 1 || NP == 2 || NP == 4, "pairs per cluster");
    static_assert((GEN_ROWS * 8) % GEN_THREADS == 0 && CHUNKS >= 1, "generator chunking");
    static_assert(SMEM_DYN <= 232448 - 512, "shared memory");
};

template <int NP, int D>
__global__ void __launch_bounds__(PairCfg<NP, D>::THREADS, 1)
noise_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_d, int64_t M,
                  int64_t N, int64_t Kc, Sq5Lin lin, int32_t *status, long long *prof) {
    using Cfg = PairCfg<NP, D>;
    long long pc0 = 0, pc1 = 0, pc2 = 0;
    constexpr int MT = Cfg::MT, BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[D], bar_free[D], bar_free_all[D], bar_tmem_full, bar_tmem_empty[MT];
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;

    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;   // stage s: A sub-tiles, then this CTA's half of the generated tile
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t half = rank & 1;          // which 128 generated rows / which 128 token rows of every MMA live here
    const uint32_t pair = rank >> 1;
    const bool leader = (half == 0);         // the even CTA of the pair issues the MMAs

    if (threadIdx.x == 0) {
        for (int s = 0; s < D; ++s) {
            // TMA thread's arrive.expect_tx (+ the odd CTA's "complete" on the even CTA); the generated bytes
            // arrive as transaction bytes of asynchronous stores
            // TMA thread's arrive.expect_tx (+ the odd CTA's "complete" on the even CTA) + every local generator thread
            mbar_init(smem_u32(&bar_full[s]), (leader ? 2 : 1) + Cfg::GEN_THREADS);
            mbar_init(smem_u32(&bar_free[s]), 1);
            mbar_init(smem_u32(&bar_free_all[s]), NP);
        }
        mbar_init(smem_u32(&bar_tmem_full), 1);
        for (int s = 0; s < MT; ++s) mbar_init(smem_u32(&bar_tmem_empty[s]), 8);   // 4 epilogue warps of each CTA of the pair
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_holder), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    volatile int *abortp = &abort_flag;
    pdl_launch_dependents();   // the next kernel of the stream may start its own prologue
    pdl_wait();                // ... and this one touches global memory only after its predecessor has completed

    const int64_t tiles_n = (N + BN - 1) / BN;
    const int64_t tiles_m = (M + (int64_t)MT * 2 * BM - 1) / ((int64_t)MT * 2 * BM);   // 512-token pair tiles
    const int64_t ctiles_m = (tiles_m + NP - 1) / NP;
    const int64_t total_ctiles = ctiles_m * tiles_n;
    const int64_t cluster_id = blockIdx.x / (2 * NP);
    const int64_t num_clusters = gridDim.x / (2 * NP);
    const int num_kb = (int)((Kc + BK - 1) / BK);
    // first token row of this pair's tile; accumulator s of this CTA covers rows m0 + s*256 + half*128 + [0,128)
    auto m_base = [&](int64_t ct) { return ((ct / tiles_n) * NP + pair) * (int64_t)MT * 2 * BM; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (this CTA's A rows)
        if (lane == 0) {
            prefetch_tmap(&tmap_a);
            PipeState st;
            bool ok = true;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                const int64_t m0 = m_base(ct) + half * BM;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const long long tw = prof ? clock64() : 0;
                    if (!mbar_wait_cluster(smem_u32(&bar_free[st.idx]), st.phase ^ 1, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (prof) pc0 += clock64() - tw;
                    const uint32_t fb = smem_u32(&bar_full[st.idx]);
                    // A bytes by TMA + the rows of the generated half that other pairs' CTAs send here
                    mbar_arrive_expect_tx(fb, Cfg::A_PART + (NP - 1) * Cfg::GEN_ROWS * BK * 2);
#pragma unroll
                    for (int s = 0; s < MT; ++s)
                        tma_load_2d(smem_base + st.idx * Cfg::STAGE + s * SUB_BYTES, &tmap_a, fb, kb * BK,
                                    (int32_t)(m0 + s * 2 * BM));
                    st.advance<D>();
                }
            }
            if (prof) prof[blockIdx.x * 16 + 4] = pc0;
            if (!ok) {
                for (int s = 0; s < D; ++s) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&bar_full[s]), 0) && !mbar_try_wait(smem_u32(&bar_full[s]), 1)) {
                        if (clock64() - t0 > 20000000LL) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA of the pair only)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN, 0, 0);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t peer = rank ^ 1u;
            PipeState st;
            uint32_t tphase = 0;
            bool ok = true;
            const long long t_start = prof ? clock64() : 0;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    const long long tw = prof ? clock64() : 0;
                    if (!mbar_wait_cluster(smem_u32(&bar_full[st.idx]), st.phase, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    if (prof) pc0 += clock64() - tw;
                    fence_proxy_async_smem();
                    tc_fence_after_sync();
                    const uint32_t a_lo = smem_desc_lo(smem_base + st.idx * Cfg::STAGE, 0);
                    const uint32_t b_lo = smem_desc_lo(smem_base + st.idx * Cfg::STAGE + Cfg::A_PART, 0);
#pragma unroll
                    for (int s = 0; s < MT; ++s) {
                        if (kb == 0) {
                            // accumulator s is reusable once both CTAs' epilogues have drained it
                            const long long te = prof ? clock64() : 0;
                            if (!mbar_wait_cluster(smem_u32(&bar_tmem_empty[s]), tphase ^ 1, abortp)) {
                                raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            if (prof) pc2 += clock64() - te;
                        }
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t adesc = pack_desc(a_lo + ((s * SUB_BYTES + k * UMMA_K * 2) >> 4), desc_hi);
                            const uint64_t bdesc = pack_desc(b_lo + ((k * UMMA_K * 2) >> 4), desc_hi);
                            umma_bf16_pair(tmem_base + s * BN, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    // the stage is free in both CTAs of the pair once these MMAs have completed
                    umma_commit_pair(smem_u32(&bar_free[st.idx]));
                    umma_commit_pair(mapa(smem_u32(&bar_free[st.idx]), peer));
                    st.advance<D>();
                }
                if (ok) {
                    umma_commit_pair(smem_u32(&bar_tmem_full));
                    umma_commit_pair(mapa(smem_u32(&bar_tmem_full), peer));
                }
                tphase ^= 1;
            }
            if (prof) {
                prof[blockIdx.x * 16 + 0] = pc0;
                prof[blockIdx.x * 16 + 2] = pc2;
                prof[blockIdx.x * 16 + 3] = clock64() - t_start;
            }
        }
    } else if (warp < Cfg::FIRST_GEN_WARP) {
        // ------------------------------------------------------------------ epilogue (4 warps, this CTA's 128 rows)
        // TMEM -> registers -> bf16 -> swizzled staging in shared memory -> TMA tile stores: the global writes
        // are whole 128-byte rows issued by one lane, asynchronous, and clipped at the tensor edges by the TMA.
        const int q = warp & 3;
        const uint32_t leader_rank = rank & ~1u;
        const uint32_t stag = smem_base + D * Cfg::STAGE + (uint32_t)(warp - Cfg::FIRST_EPI_WARP) * 8192u;   // two 4 KB boxes
        uint32_t tphase = 0;
        for (int64_t ct = cluster_id; ct < total_ctiles; ct += num_clusters) {
            const int64_t m0 = m_base(ct) + half * BM;
            const int64_t n0 = (ct % tiles_n) * BN;
            if (!mbar_wait_warp<true>(smem_u32(&bar_tmem_full), tphase, abortp)) {
                raise_abort(abortp, status, RDB_STATUS_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int s = 0; s < MT; ++s) {
                const int64_t row_w = m0 + s * 2 * BM + q * 32;    // first row of this warp's 32-row slab
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 128) {
                    // the previous stores of this warp must have finished reading the staging boxes
                    if (lane == 0) bulk_wait_group_read0();
                    __syncwarp();
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        uint32_t r0[32], r1[32];
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * BN + c0 + hb * 64);
                        tmem_ld_32x32(taddr, r0);
                        tmem_ld_32x32(taddr + 32, r1);
                        tmem_ld_wait();
                        const uint32_t rowaddr = stag + hb * 4096u + (uint32_t)lane * 128u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t pk[4], pl[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r0[j * 8 + 2 * e]), __uint_as_float(r0[j * 8 + 2 * e + 1]));
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r1[j * 8 + 2 * e]), __uint_as_float(r1[j * 8 + 2 * e + 1]));
                                pk[e] = *reinterpret_cast<uint32_t *>(&h0);
                                pl[e] = *reinterpret_cast<uint32_t *>(&h1);
                            }
                            // 16-byte chunk j (columns 8j..8j+7) and chunk 4+j (columns 32+8j..) of this lane's 128-byte row
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)((j ^ (lane & 7)) << 4)),
                                         "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)(((4 + j) ^ (lane & 7)) << 4)),
                                         "r"(pl[0]), "r"(pl[1]), "r"(pl[2]), "r"(pl[3]) : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row_w < M) {
                        const int64_t col = n0 + c0;
                        if (col < N) tma_store_2d(&tmap_d, stag, (int32_t)col, (int32_t)row_w);
                        if (col + 64 < N) tma_store_2d(&tmap_d, stag + 4096u, (int32_t)(col + 64), (int32_t)row_w);
                        bulk_commit_group();
                    }
                }
                // accumulator s of this CTA has been read out: tell the MMA thread of the pair
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(mapa(smem_u32(&bar_tmem_empty[s]), leader_rank));
            }
            tphase ^= 1;
        }
        if (lane == 0) bulk_wait_group0();   // all output tiles written before the CTA retires
    } else if (warp < Cfg::FULL_RELAY_WARP) {
        // ------------------------------------------------------------------ generators (8 warps)
        const int tg = threadIdx.x - Cfg::FIRST_GEN_WARP * 32;
        constexpr int CHUNKS = Cfg::CHUNKS;
        PipeState st;
        bool ok = true;
        for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
            const int64_t n0 = (ct % tiles_n) * BN + half * Cfg::HALF;   // first generated row of this CTA's half
            uint32_t bstart[CHUNKS];
            uint32_t soff[CHUNKS];
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int id = tg + c * Cfg::GEN_THREADS;
                const int rowi = (int)pair * Cfg::GEN_ROWS + (id >> 3), ch = id & 7;   // row inside the half
                bstart[c] = lin.base + (uint32_t)(n0 + rowi) * lin.sn + (uint32_t)(ch * 8) * lin.sk;
                soff[c] = (uint32_t)(Cfg::A_PART + rowi * 128 + ((ch ^ (rowi & 7)) << 4));
            }
            const uint32_t kb_step = (uint32_t)BK * lin.sk;
            for (int kb = 0; kb < num_kb; ++kb) {
                const uint32_t wb = NP > 1 ? smem_u32(&bar_free_all[st.idx]) : smem_u32(&bar_free[st.idx]);
                const long long tw = prof ? clock64() : 0;
                if (!mbar_wait_cluster(wb, st.phase ^ 1, abortp)) {
                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_GENERATOR);
                    ok = false;
                    break;
                }
                const long long tc = prof ? clock64() : 0;
                const uint32_t stage = smem_base + st.idx * Cfg::STAGE;
                const uint32_t fb = smem_u32(&bar_full[st.idx]);
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    uint32_t p[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        p[j] = sq5_pack_bf16x2(sq5_tail(bstart[c] + (uint32_t)(2 * j) * lin.sk), sq5_tail(bstart[c] + (uint32_t)(2 * j + 1) * lin.sk));
                    }
                    // own copy: plain store; the other CTAs that hold this half get asynchronous 16-byte stores that
                    // complete their bytes on the receiver's `full` barrier
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + soff[c]), "r"(p[0]), "r"(p[1]), "r"(p[2]),
                                 "r"(p[3]) : "memory");
#pragma unroll
                    for (int qd = 0; qd < NP; ++qd) {
                        const uint32_t dst = 2u * qd + half;
                        if (dst != rank) st_async_v4(mapa(stage + soff[c], dst), p[0], p[1], p[2], p[3], mapa(fb, dst));
                    }
                    bstart[c] += kb_step;
                }
                fence_proxy_async_smem();
                mbar_arrive(fb);
                if (prof) { pc0 += tc - tw; pc1 += clock64() - tc; }
                st.advance<D>();
            }
        }
        if (prof && tg == 0) {
            prof[blockIdx.x * 16 + 5] = pc0;
            prof[blockIdx.x * 16 + 6] = pc1;
        }
    } else if (warp == Cfg::FULL_RELAY_WARP) {
        // ------------------------------------------------------------------ odd CTA: tell the even CTA a stage is complete here
        if (lane == 0 && !leader) {
            const uint32_t leader_rank = rank & ~1u;
            PipeState st;
            bool ok = true;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_cluster(smem_u32(&bar_full[st.idx]), st.phase, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    fence_proxy_async_smem();
                    mbar_arrive_remote(mapa(smem_u32(&bar_full[st.idx]), leader_rank));
                    st.advance<D>();
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ tell the CTAs that write this half that the stage is free
        if (lane == 0 && NP > 1) {
            PipeState st;
            bool ok = true;
            for (int64_t ct = cluster_id; ct < total_ctiles && ok; ct += num_clusters) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_cluster(smem_u32(&bar_free[st.idx]), st.phase, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_GENERATOR);
                        ok = false;
                        break;
                    }
                    const uint32_t fa = smem_u32(&bar_free_all[st.idx]);
#pragma unroll
                    for (int qd = 0; qd < NP; ++qd) mbar_arrive_remote(mapa(fa, 2u * qd + half));
                    st.advance<D>();
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // no CTA retires (or frees TMEM) while a peer may still use it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ================================================================================================
// dense_gemm_kernel
// ================================================================================================
template <int BN, int STAGES>
struct DenseCfg {
    static constexpr int A_STAGE = SUB_BYTES;
    static constexpr int B_STAGE = BN * BK * 2;
    static constexpr int STAGE = A_STAGE + B_STAGE;
    static constexpr int EPI_WARPS = 8;                               // two per TMEM lane quarter, half of the columns each
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    // per epilogue warp: [32 rows x 64 columns] bf16 boxes for the TMA tile stores.  With a ring of three stages (the
    // variant for contractions of at most three k-blocks, whose tiles are all epilogue) there is room for two per warp, so
    // a warp fills one while the store engine still reads the other
    static constexpr int STG = STAGES <= 3 ? 2 : 1;
    static constexpr int OUT_STAGING = EPI_WARPS * 4096 * STG;
    static constexpr int SMEM_DYN = STAGES * STAGE + OUT_STAGING + 1024;
    static_assert(SMEM_DYN <= 232448 - 512, "shared memory");
    static_assert(2 * BN <= TMEM_COLS, "two accumulator stages must fit TMEM");
    static_assert(BN % 64 == 0 && BN <= 256, "BN");
};

template <int BN, int STAGES, int A_MN, int B_MN, typename OutT>
__global__ void __launch_bounds__(DenseCfg<BN, STAGES>::THREADS, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, OutT *__restrict__ d, int64_t ldd, int64_t M, int64_t N, int64_t Kc, int m_fast, int split, int64_t slice_stride,
                  int f32_tma, int32_t *status) {
    // split > 1: the contraction is cut into `split` slices of whole k-blocks; work item = (slice, tile) and slice s
    // writes its partial product at d + s * slice_stride (the caller sums the slices in order)
    using Cfg = DenseCfg<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tmem_full[2], bar_tmem_empty[2];
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;

    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_tmem_full[s]), 1); mbar_init(smem_u32(&bar_tmem_empty[s]), Cfg::EPI_WARPS); }
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_holder), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    volatile int *abortp = &abort_flag;
    pdl_launch_dependents();   // the next kernel of the stream may start its own prologue
    pdl_wait();                // ... and this one touches global memory only after its predecessor has completed

    const int64_t tiles_n = (N + BN - 1) / BN;
    const int64_t tiles_m = (M + BM - 1) / BM;
    const int64_t tiles_mn = tiles_m * tiles_n;
    const int64_t total_tiles = tiles_mn * split;
    const int all_kb = (int)((Kc + BK - 1) / BK);
    const int kb_per = (all_kb + split - 1) / split;
    // k-block range of a work item
    auto kb_lo = [&](int64_t w) { return (int)(w / tiles_mn) * kb_per; };
    auto kb_hi = [&](int64_t w) { const int hi = ((int)(w / tiles_mn) + 1) * kb_per; return hi < all_kb ? hi : all_kb; };

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tmap(&tmap_a);
            prefetch_tmap(&tmap_b);
            PipeState st;
            bool ok = true;
            for (int64_t w = blockIdx.x; w < total_tiles && ok; w += gridDim.x) {
                const int64_t tile = w % tiles_mn;
                const int32_t m0 = (int32_t)((m_fast ? tile % tiles_m : tile / tiles_n) * BM);
                const int32_t n0 = (int32_t)((m_fast ? tile / tiles_m : tile % tiles_n) * BN);
                for (int kb = kb_lo(w); kb < kb_hi(w); ++kb) {
                    if (!mbar_wait(smem_u32(&bar_empty[st.idx]), st.phase ^ 1, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t fb = smem_u32(&bar_full[st.idx]);
                    mbar_arrive_expect_tx(fb, Cfg::STAGE);
                    const uint32_t sa = smem_base + st.idx * Cfg::STAGE;
                    const uint32_t sbm = sa + Cfg::A_STAGE;
                    if (A_MN) {
                        // operand stored [Kc, M]: two boxes of 64 (M, contiguous) x 64 (K rows)
#pragma unroll
                        for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * (64 * BK * 2), &tmap_a, fb, m0 + i * 64, kb * BK);
                    } else {
                        tma_load_2d(sa, &tmap_a, fb, kb * BK, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int i = 0; i < BN / 64; ++i) tma_load_2d(sbm + i * (64 * BK * 2), &tmap_b, fb, n0 + i * 64, kb * BK);
                    } else {
                        tma_load_2d(sbm, &tmap_b, fb, kb * BK, n0);
                    }
                    st.advance<STAGES>();
                }
            }
            if (!ok) {
                for (int s = 0; s < STAGES; ++s) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&bar_full[s]), 0) && !mbar_try_wait(smem_u32(&bar_full[s]), 1)) {
                        if (clock64() - t0 > 20000000LL) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN, A_MN, B_MN);
            // K-major: 8-row groups 1024 B apart, k-step = 32 B inside the swizzle row.
            // MN-major: 64-element column blocks 8192 B apart (LBO), 8-k groups 1024 B apart (SBO),
            //           k-step of 16 = two groups = 2048 B.
            constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 0, A_KSTEP = A_MN ? 2048 : UMMA_K * 2;
            constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 0, B_KSTEP = B_MN ? 2048 : UMMA_K * 2;
            PipeState st;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t w = blockIdx.x; w < total_tiles && ok; w += gridDim.x) {
                const int kb0 = kb_lo(w), kb1 = kb_hi(w);
                if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1, abortp)) {
                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tacc = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_full[st.idx]), st.phase, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + st.idx * Cfg::STAGE;
                    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
                    const uint32_t a_lo = smem_desc_lo(sa, A_LBO);
                    const uint32_t b_lo = smem_desc_lo(sa + Cfg::A_STAGE, B_LBO);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adesc = pack_desc(a_lo + ((k * A_KSTEP) >> 4), desc_hi);
                        const uint64_t bdesc = pack_desc(b_lo + ((k * B_KSTEP) >> 4), desc_hi);
                        umma_bf16(tacc, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[st.idx]));
                    st.advance<STAGES>();
                }
                if (ok) umma_commit(smem_u32(&bar_tmem_full[acc]));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        constexpr int CPW = BN / (Cfg::EPI_WARPS / 4);  // accumulator columns per warp
        const int cbase = ((warp - 2) >> 2) * CPW;
        constexpr bool TMA_OUT = (sizeof(OutT) == 2);   // bf16: swizzled staging + TMA tile stores; float32: direct stores
        const uint32_t stag0 = smem_base + STAGES * Cfg::STAGE + (uint32_t)(warp - 2) * (4096u * Cfg::STG);
        uint32_t stag = stag0, box = 0;
        // before a staging box is written again the store that last read it must be done with it
        auto next_box = [&]() {
            if (Cfg::STG == 2) {
                stag = stag0 + box * 4096u;
                box ^= 1u;
                if (lane == 0) bulk_wait_group_read1();
            } else {
                if (lane == 0) bulk_wait_group_read0();
            }
            __syncwarp();
        };
        uint32_t acc = 0, acc_phase = 0;
        for (int64_t w = blockIdx.x; w < total_tiles; w += gridDim.x) {
            const int64_t tile = w % tiles_mn;
            OutT *dw = d + (w / tiles_mn) * slice_stride;
            const int64_t m0 = (m_fast ? tile % tiles_m : tile / tiles_n) * BM;
            const int64_t n0 = (m_fast ? tile / tiles_m : tile % tiles_n) * BN;
            if (!mbar_wait_warp<false>(smem_u32(&bar_tmem_full[acc]), acc_phase, abortp)) {
                raise_abort(abortp, status, RDB_STATUS_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            const int64_t row_w = m0 + q * 32;
            if (TMA_OUT) {
#pragma unroll 1
                for (int c0 = cbase; c0 < cbase + CPW; c0 += 64) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0);
                    tmem_ld_32x32(taddr, r0);
                    tmem_ld_32x32(taddr + 32, r1);
                    next_box();
                    tmem_ld_wait();
                    const uint32_t rowaddr = stag + (uint32_t)lane * 128u;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t pk[4], pl[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r0[j * 8 + 2 * e]), __uint_as_float(r0[j * 8 + 2 * e + 1]));
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r1[j * 8 + 2 * e]), __uint_as_float(r1[j * 8 + 2 * e + 1]));
                            pk[e] = *reinterpret_cast<uint32_t *>(&h0);
                            pl[e] = *reinterpret_cast<uint32_t *>(&h1);
                        }
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)((j ^ (lane & 7)) << 4)),
                                     "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)(((4 + j) ^ (lane & 7)) << 4)),
                                     "r"(pl[0]), "r"(pl[1]), "r"(pl[2]), "r"(pl[3]) : "memory");
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (row_w < M && n0 + c0 < N) tma_store_2d(&tmap_d, stag, (int32_t)(n0 + c0), (int32_t)row_w);
                        bulk_commit_group();      // one group per box use, empty or not: next_box() counts groups
                    }
                }
            } else if (f32_tma) {
                // float32 partial products, M a multiple of 128: [32 rows x 32 columns] boxes (128-byte rows) through the same
                // staging; the output is addressed as one [split * M, N] matrix
                const int64_t row_g = (w / tiles_mn) * M + row_w;
#pragma unroll 1
                for (int c0 = cbase; c0 < cbase + CPW; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                    next_box();
                    tmem_ld_wait();
                    const uint32_t rowaddr = stag + (uint32_t)lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)((j ^ (lane & 7)) << 4)),
                                     "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (n0 + c0 < N) tma_store_2d(&tmap_d, stag, (int32_t)(n0 + c0), (int32_t)row_g);
                        bulk_commit_group();
                    }
                }
            } else {
                const int64_t row = row_w + lane;
#pragma unroll 1
                for (int c0 = cbase; c0 < cbase + CPW; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                    tmem_ld_wait();
                    const int64_t col = n0 + c0;
                    const int ncols = (int)((N - col) < 32 ? (N - col) : 32);
                    if (row < M && ncols > 0) store_row32<OutT>(dw + row * ldd + col, r, ncols);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if ((TMA_OUT || f32_tma) && lane == 0) bulk_wait_group0();   // all output tiles written before the CTA retires
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ================================================================================================
// dense_pair_kernel: D[M,N] = op(A) op(B)^T on CTA pairs (tcgen05 cta_group::2), bf16 output
//
// One pair owns a tile of MT*256 rows x 256 columns.  Each pair MMA is 256 x 256 x 16: the even CTA holds rows
// [0,128) and the odd CTA rows [128,256) of the 256-row sub-tile in its TMEM lanes, and each CTA stages only its
// own 128 rows of A and its own 128 of the 256 B rows, so a 64-wide k-block costs a CTA (MT+1)*16 KB of TMA
// traffic for MT*128x256x64 MACs.  MT = 2 fills TMEM with one tile (two accumulators, released one by one to
// the next tile); MT = 1 alternates between the two accumulators so the epilogue overlaps the next main loop.
//
//   warp 0      TMA producer (own A rows, own half of B); the loads of both CTAs complete their transaction bytes on
//               the even CTA's barrier (cta_group::2 form of the load), so the MMA thread waits on one barrier
//   warp 1      MMA issuer (even CTA only); tcgen05.commit frees the stage in both CTAs
//   warps 2-9   epilogue: TMEM -> bf16 -> swizzled staging -> TMA tile stores (two warps per lane quarter)
// ================================================================================================
// the pair kernel's epilogue reads accumulator 0 (the one the next tile's first MMAs wait for) with all four of a warp's
// tcgen05.ld in flight before one wait; accumulator 1, read while 64 converted registers are live, two at a time
constexpr bool DRAIN_WIDE = true;

template <int MT, int D>
struct DensePairCfg {
    static constexpr int BN = 256;
    static constexpr int HALF = BN / 2;
    static constexpr int A_PART = MT * SUB_BYTES;
    static constexpr int B_PART = HALF * BK * 2;
    static constexpr int STAGE = A_PART + B_PART;
    static constexpr int EPI_WARPS = 8;
    static constexpr int FIRST_EPI_WARP = 2;
    static constexpr int END_WARP = FIRST_EPI_WARP + EPI_WARPS;
    static constexpr int THREADS = END_WARP * 32;
    static constexpr int OUT_STAGING = EPI_WARPS * 4096;               // per epilogue warp: one [32 rows x 64 columns] bf16 box
    static constexpr int SMEM_DYN = D * STAGE + OUT_STAGING + 1024;
    static_assert(MT == 1 || MT == 2, "sub-tiles per pair tile");
    static_assert(SMEM_DYN <= 232448 - 512, "shared memory");
};

// Output tensor maps of the pair kernel.  NDST == 1: the one output matrix.  NDST > 1 (the scatter half of a reduce-scatter
// fused into the product): row block j of the output -- rows [j * rows_per_dst, (j + 1) * rows_per_dst) -- is stored into
// destination j, a dense [rows_per_dst x N] matrix that may live in another GPU's memory (plain TMA tile stores over
// NVLink, no multicast); rows_per_dst is a multiple of 32, so no 32-row store box spans two destinations.
template <int NDST>
struct OutMaps {
    CUtensorMap m[NDST];
};

// F32 (split-K): the contraction is cut into `split` slices of whole k-blocks; work item = (slice, tile), and slice s writes its
// float32 partial product into rows [s * M, (s + 1) * M) of the output map, a float32 [split * M, N] matrix (M a multiple of
// 32, so no 32-row store box crosses into the next slice); split_k_reduce_kernel adds the slices in order afterwards.
template <int MT, int D, int A_MN, int B_MN, int NDST, bool F32>
__global__ void __launch_bounds__(DensePairCfg<MT, D>::THREADS, 1)
dense_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ OutMaps<NDST> out, int64_t rows_per_dst, int64_t M, int64_t N, int64_t Kc, int m_fast,
                  int split, int32_t *status, long long *prof) {
    long long pc0 = 0, pc2 = 0;
    using Cfg = DensePairCfg<MT, D>;
    constexpr int BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[D], bar_free[D], bar_tmem_full[2], bar_tmem_empty[2];
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;

    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;   // stage s: A sub-tiles, then this CTA's half of the B tile
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t half = rank & 1;
    const bool leader = (half == 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < D; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);                 // the even CTA's TMA thread; both CTAs' loads complete their bytes here
            mbar_init(smem_u32(&bar_free[s]), 1);                 // one tcgen05.commit from the pair's MMA thread
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bar_tmem_full[s]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[s]), 2 * Cfg::EPI_WARPS);
        }
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_holder), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    volatile int *abortp = &abort_flag;
    pdl_launch_dependents();   // the next kernel of the stream may start its own prologue
    pdl_wait();                // ... and this one touches global memory only after its predecessor has completed

    const int64_t tiles_m = (M + (int64_t)MT * 2 * BM - 1) / ((int64_t)MT * 2 * BM);
    const int64_t tiles_n = (N + BN - 1) / BN;
    const int64_t tiles_mn = tiles_m * tiles_n;
    const int64_t total_tiles = tiles_mn * split;          // work items: (slice, tile)
    const int64_t pair_id = blockIdx.x >> 1;
    const int64_t num_pairs = gridDim.x >> 1;
    const int all_kb = (int)((Kc + BK - 1) / BK);
    const int kb_per = (all_kb + split - 1) / split;
    auto kb_lo = [&](int64_t w) { return (int)(w / tiles_mn) * kb_per; };
    auto kb_hi = [&](int64_t w) { const int hi = ((int)(w / tiles_mn) + 1) * kb_per; return hi < all_kb ? hi : all_kb; };
    // consecutive tiles share the B panel (m_fast) or the A panel: the larger operand is the one streamed once
    auto tile_m = [&](int64_t w) { const int64_t t = w % tiles_mn; return m_fast ? (t % tiles_m) : (t / tiles_n); };
    auto tile_n = [&](int64_t w) { const int64_t t = w % tiles_mn; return m_fast ? (t / tiles_m) : (t % tiles_n); };
    // accumulator and barrier parity used by sub-tile s of this CTA's it-th tile
    auto acc_of = [&](int64_t it, int s) { return MT == 2 ? s : (int)(it & 1); };
    auto par_of = [&](int64_t it) { return (uint32_t)(MT == 2 ? (it & 1) : ((it >> 1) & 1)); };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tmap(&tmap_a);
            prefetch_tmap(&tmap_b);
            PipeState st;
            bool ok = true;
            for (int64_t t = pair_id; t < total_tiles && ok; t += num_pairs) {
                const int32_t m0 = (int32_t)(tile_m(t) * MT * 2 * BM + half * BM);
                const int32_t n0 = (int32_t)(tile_n(t) * BN + half * Cfg::HALF);
                for (int kb = kb_lo(t); kb < kb_hi(t); ++kb) {
                    const long long tw = prof ? clock64() : 0;
                    if (!mbar_wait_cluster(smem_u32(&bar_free[st.idx]), st.phase ^ 1, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (prof) pc0 += clock64() - tw;
                    // both CTAs' loads of a stage complete their bytes on the even CTA's barrier, where the MMA thread waits
                    const uint32_t fb = mapa(smem_u32(&bar_full[st.idx]), rank & ~1u);
                    if (leader) mbar_arrive_expect_tx(smem_u32(&bar_full[st.idx]), 2 * Cfg::STAGE);
                    const uint32_t sa = smem_base + st.idx * Cfg::STAGE;
                    const uint32_t sb = sa + Cfg::A_PART;
#pragma unroll
                    for (int s = 0; s < MT; ++s) {
                        if (A_MN) {
#pragma unroll
                            for (int i = 0; i < BM / 64; ++i)
                                tma_load_2d_pair(sa + s * SUB_BYTES + i * (64 * BK * 2), &tmap_a, fb, m0 + s * 2 * BM + i * 64, kb * BK);
                        } else {
                            tma_load_2d_pair(sa + s * SUB_BYTES, &tmap_a, fb, kb * BK, m0 + s * 2 * BM);
                        }
                    }
                    if (B_MN) {
#pragma unroll
                        for (int i = 0; i < Cfg::HALF / 64; ++i) tma_load_2d_pair(sb + i * (64 * BK * 2), &tmap_b, fb, n0 + i * 64, kb * BK);
                    } else {
                        tma_load_2d_pair(sb, &tmap_b, fb, kb * BK, n0);
                    }
                    st.advance<D>();
                }
            }
            if (prof) prof[blockIdx.x * 16 + 4] = pc0;
            if (!ok) {
                // gave up: let the loads already in flight land before the CTA may retire (their completions go to the
                // even CTA's barriers, so this side can only wait out the time a load can take)
                const long long t0 = clock64();
                while (clock64() - t0 < 4000000LL) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA of the pair)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN, A_MN, B_MN);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 0, A_KSTEP = A_MN ? 2048 : UMMA_K * 2;
            constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 0, B_KSTEP = B_MN ? 2048 : UMMA_K * 2;
            const uint32_t peer = rank ^ 1u;
            PipeState st;
            bool ok = true;
            int64_t it = 0;
            const long long t_start = prof ? clock64() : 0;
            for (int64_t t = pair_id; t < total_tiles && ok; t += num_pairs, ++it) {
                const int kb0 = kb_lo(t), kb1 = kb_hi(t);
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    const long long tw = prof ? clock64() : 0;
                    if (!mbar_wait_cluster(smem_u32(&bar_full[st.idx]), st.phase, abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    if (prof) pc0 += clock64() - tw;
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + st.idx * Cfg::STAGE;
                    const uint32_t b_lo = smem_desc_lo(sa + Cfg::A_PART, B_LBO);
                    auto issue = [&](int s, int k) {
                        const uint32_t a_lo = smem_desc_lo(sa + s * SUB_BYTES, A_LBO);
                        const uint64_t adesc = pack_desc(a_lo + ((k * A_KSTEP) >> 4), desc_hi);
                        const uint64_t bdesc = pack_desc(b_lo + ((k * B_KSTEP) >> 4), desc_hi);
                        umma_bf16_pair(tmem_base + acc_of(it, s) * BN, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
                    };
                    const bool first = (kb == kb0), last = (kb == kb1 - 1);
                    if (MT == 2 && (first || last)) {
                        // tile boundaries, one accumulator after the other: the first k-block of accumulator 0 starts as soon
                        // as the epilogue has drained it (accumulator 1 is still being stored), and the last k-block hands
                        // accumulator 0 to the epilogue while accumulator 1's MMAs still run
#pragma unroll
                        for (int s = 0; s < MT; ++s) {
                            if (first) {
                                const long long te = prof ? clock64() : 0;
                                if (!mbar_wait_cluster(smem_u32(&bar_tmem_empty[acc_of(it, s)]), par_of(it) ^ 1, abortp)) {
                                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                                    ok = false;
                                    break;
                                }
                                tc_fence_after_sync();
                                if (prof) pc2 += clock64() - te;
                            }
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k) issue(s, k);
                            if (last) {
                                umma_commit_pair(smem_u32(&bar_tmem_full[acc_of(it, s)]));
                                umma_commit_pair(mapa(smem_u32(&bar_tmem_full[acc_of(it, s)]), peer));
                            }
                        }
                    } else {
                        if (first) {
                            const long long te = prof ? clock64() : 0;
                            if (!mbar_wait_cluster(smem_u32(&bar_tmem_empty[acc_of(it, 0)]), par_of(it) ^ 1, abortp)) {
                                raise_abort(abortp, status, RDB_STATUS_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            if (prof) pc2 += clock64() - te;
                        }
                        // consecutive MMAs alternate between the accumulators and share the B slice
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
#pragma unroll
                            for (int s = 0; s < MT; ++s) issue(s, k);
                        }
                        if (last) {
                            umma_commit_pair(smem_u32(&bar_tmem_full[acc_of(it, 0)]));
                            umma_commit_pair(mapa(smem_u32(&bar_tmem_full[acc_of(it, 0)]), peer));
                        }
                    }
                    if (!ok) break;
                    umma_commit_pair(smem_u32(&bar_free[st.idx]));
                    umma_commit_pair(mapa(smem_u32(&bar_free[st.idx]), peer));
                    st.advance<D>();
                }
            }
            if (prof) {
                prof[blockIdx.x * 16 + 0] = pc0;
                prof[blockIdx.x * 16 + 2] = pc2;
                prof[blockIdx.x * 16 + 3] = clock64() - t_start;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (8 warps, this CTA's 128 rows)
        // Two phases per tile.  (1) Drain: as soon as an accumulator is complete, every warp copies its 32 rows x 128
        // columns into registers (already rounded to bf16) and hands the accumulator back to the MMA thread -- TMEM is
        // held only for the tcgen05.ld round trips, so the next tile's MMAs start while (2) the registers go through the
        // swizzled staging box and out as TMA tile stores.  One 512 x 256 tile fills all of TMEM, so everything that
        // happens before the hand-back is time the tensor pipe idles; after it, the stores hide under ~16 k-blocks of MMAs.
        const int ew = warp - Cfg::FIRST_EPI_WARP;
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int cg = ew >> 2;                      // which 128 of the 256 accumulator columns
        const uint32_t leader_rank = rank & ~1u;
        const uint32_t stag = smem_base + D * Cfg::STAGE + (uint32_t)ew * 4096u;
        int64_t it = 0;
        bool ok = true;
        for (int64_t t = pair_id; t < total_tiles && ok; t += num_pairs, ++it) {
            const int64_t m0 = tile_m(t) * MT * 2 * BM + half * BM;
            const int64_t n0 = tile_n(t) * BN;
            if (F32) {
                // float32 partial products of a split-K work item: [32 rows x 32 columns] boxes (128-byte rows) through the
                // staging box, straight from TMEM; the accumulator goes back when all of it has been read
                const int64_t row_base = (t / tiles_mn) * M;
#pragma unroll 1
                for (int s = 0; s < MT && ok; ++s) {
                    const int a = acc_of(it, s);
                    if (!mbar_wait_warp<true>(smem_u32(&bar_tmem_full[a]), par_of(it), abortp)) {
                        raise_abort(abortp, status, RDB_STATUS_TIMEOUT_EPILOGUE);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const int64_t row_w = m0 + s * 2 * BM + q * 32;
#pragma unroll 1
                    for (int c0 = cg * 128; c0 < cg * 128 + 128; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + c0), r);
                        if (lane == 0) bulk_wait_group_read0();
                        __syncwarp();
                        tmem_ld_wait();
                        const uint32_t rowaddr = stag + (uint32_t)lane * 128u;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)((j ^ (lane & 7)) << 4)),
                                         "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && row_w < M && n0 + c0 < N) {
                            tma_store_2d(&out.m[0], stag, (int32_t)(n0 + c0), (int32_t)(row_base + row_w));
                            bulk_commit_group();
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(mapa(smem_u32(&bar_tmem_empty[a]), leader_rank));
                }
                continue;
            }
            uint32_t packed[MT][64];                 // [sub-tile][16-byte chunk * 4 + word]: 128 bf16 columns of this lane's row
            unsigned t_full = 0;
#pragma unroll
            for (int s = 0; s < MT; ++s) {
                const int a = acc_of(it, s);
                if (ok && !mbar_wait_warp<true>(smem_u32(&bar_tmem_full[a]), par_of(it), abortp)) {
                    raise_abort(abortp, status, RDB_STATUS_TIMEOUT_EPILOGUE);
                    ok = false;
                }
                if (ok) {
                    tc_fence_after_sync();
                    if (prof && s == 0) t_full = (unsigned)clock();
                    // this warp's part of the accumulator has landed in registers: hand it back to the MMA thread of the pair
                    auto hand_back = [&]() {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote(mapa(smem_u32(&bar_tmem_empty[a]), leader_rank));
                        if (prof && ew == 0 && lane == 0)
                            atomicAdd(reinterpret_cast<unsigned long long *>(prof) + blockIdx.x * 16 + 5 + s, (unsigned long long)((unsigned)clock() - t_full));
                    };
                    if (DRAIN_WIDE && s == 0) {
                        // accumulator 0 is the one the next tile's first MMAs wait for: all four loads in flight at once
                        uint32_t r0[32], r1[32], r2[32], r3[32];
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + cg * 128);
                        tmem_ld_32x32(taddr, r0);
                        tmem_ld_32x32(taddr + 32, r1);
                        tmem_ld_32x32(taddr + 64, r2);
                        tmem_ld_32x32(taddr + 96, r3);
                        tmem_ld_wait();
                        hand_back();          // the values are in registers: the conversion runs under the next tile's MMAs
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r2[2 * j]), __uint_as_float(r2[2 * j + 1]));
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r3[2 * j]), __uint_as_float(r3[2 * j + 1]));
                            packed[s][j] = *reinterpret_cast<uint32_t *>(&h0);
                            packed[s][16 + j] = *reinterpret_cast<uint32_t *>(&h1);
                            packed[s][32 + j] = *reinterpret_cast<uint32_t *>(&h2);
                            packed[s][48 + j] = *reinterpret_cast<uint32_t *>(&h3);
                        }
                    } else {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        uint32_t r0[32], r1[32];
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + cg * 128 + hb * 64);
                        tmem_ld_32x32(taddr, r0);
                        tmem_ld_32x32(taddr + 32, r1);
                        tmem_ld_wait();
                        if (hb == 1) hand_back();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                            packed[s][hb * 32 + j] = *reinterpret_cast<uint32_t *>(&h0);
                            packed[s][hb * 32 + 16 + j] = *reinterpret_cast<uint32_t *>(&h1);
                        }
                    }
                    }
                }
            }
            if (!ok) break;
            const unsigned t_store = prof ? (unsigned)clock() : 0u;
#pragma unroll
            for (int s = 0; s < MT; ++s) {
                const int64_t row_w = m0 + s * 2 * BM + q * 32;    // first row of this warp's 32-row slab
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    const int c0 = cg * 128 + hb * 64;
                    // the previous store of this warp must have finished reading the staging box
                    if (lane == 0) bulk_wait_group_read0();
                    __syncwarp();
                    const uint32_t rowaddr = stag + (uint32_t)lane * 128u;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (uint32_t)((ch ^ (lane & 7)) << 4)),
                                     "r"(packed[s][hb * 32 + ch * 4]), "r"(packed[s][hb * 32 + ch * 4 + 1]),
                                     "r"(packed[s][hb * 32 + ch * 4 + 2]), "r"(packed[s][hb * 32 + ch * 4 + 3]) : "memory");
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row_w < M && n0 + c0 < N) {
                        int di = 0;
                        int64_t row_l = row_w;
                        if (NDST > 1) {
                            di = (int)(row_w / rows_per_dst);
                            row_l = row_w - di * rows_per_dst;
                        }
                        tma_store_2d(&out.m[di], stag, (int32_t)(n0 + c0), (int32_t)row_l);
                        bulk_commit_group();
                    }
                }
            }
            if (prof && ew == 0 && lane == 0) {
                // first epilogue warp of each CTA: cycles from seeing accumulator 0 complete to handing it back [5], to handing
                // accumulator 1 back [6], and spent in the store phase [7], summed over this CTA's tiles
                prof[blockIdx.x * 16 + 7] += (long long)((unsigned)clock() - t_store);
            }
        }
        if (lane == 0) bulk_wait_group0();   // all output tiles written (remote ones included) before the CTA retires
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // no CTA retires (or frees TMEM) while its peer may still use it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ================================================================================================
// host side
// ================================================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
        if (q != cudaDriverEntryPointSuccess) return (EncodeTiledFn) nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// cuTensorMapEncodeTiled needs a CUDA context current on the calling thread.  PyTorch's autograd worker
// threads may not have touched the runtime yet when they call in here (device 0 is never "set"
// explicitly and cached allocations make no API call), so bind the primary context once per thread:
// the runtime adopts the driver context that is already current, or binds its default device otherwise.
static void ensure_context() {
    thread_local bool done = false;
    if (!done) {
        (void)cudaFree(nullptr);
        done = true;
    }
}

// bf16 matrix with `inner` contiguous elements per row, `outer` rows, row pitch ld elements.
static int make_tmap(CUtensorMap *m, const void *base, int64_t inner, int64_t outer, int64_t ld, uint32_t box_inner,
                     uint32_t box_outer, bool f32 = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RDB_ERR_DRIVER;
    ensure_context();
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (getenv("RDB_DEBUG"))
            fprintf(stderr, "randumb_b200: cuTensorMapEncodeTiled -> %d (base %p inner %lld outer %lld ld %lld box %u x %u)\n",
                    (int)r, base, (long long)inner, (long long)outer, (long long)ld, box_inner, box_outer);
        return RDB_ERR_DRIVER_BASE - (int)r;   // keeps the CUresult visible to the caller
    }
    return RDB_OK;
}

static int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool umma_shape_ok_noise(int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, const void *a, const void *d) {
    return M >= 1 && N >= 8 && Kc >= 8 && (N % 8) == 0 && (Kc % 8) == 0 && (lda % 8) == 0 && (ldd % 8) == 0 &&
           aligned16(a) && aligned16(d) && M < (1LL << 31) && N < (1LL << 31) && Kc < (1LL << 31);
}

static long long *g_prof = nullptr;
static size_t g_prof_bytes = 0;
void set_profile_buffer(void *p, size_t bytes) {
    g_prof = reinterpret_cast<long long *>(p);
    g_prof_bytes = p ? bytes : 0;
}

template <int CS, int MT, int BN, int SA, int SB>
static int launch_noise_gemm(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, Sq5Lin lin,
                             int32_t *status, cudaStream_t st) {
    using Cfg = NoiseCfg<CS, MT, BN, SA, SB>;
    CUtensorMap ta;
    int rc = make_tmap(&ta, a, Kc, M, lda, BK, BM);
    if (rc) return rc;
    auto kern = noise_gemm_kernel<CS, MT, BN, SA, SB>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_DYN);
    if (e != cudaSuccess) return (int)e;
    const int64_t ctiles = cdiv64(cdiv64(M, (int64_t)MT * BM), CS) * cdiv64(N, BN);

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_DYN;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;                       // the occupancy query below sees the cluster shape only
    int max_clusters = sm_count() / CS;
    if (CS > 1) {
        cfg.gridDim = dim3(CS);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) max_clusters = n;
        else (void)cudaGetLastError();
    }
    const int64_t nclusters = ctiles < max_clusters ? ctiles : max_clusters;
    cfg.gridDim = dim3((unsigned)(nclusters * CS));
    cfg.numAttrs = 2;
    __nv_bfloat16 *dp = reinterpret_cast<__nv_bfloat16 *>(d);
    long long *prof = (g_prof && g_prof_bytes >= (size_t)cfg.gridDim.x * 16 * sizeof(long long)) ? g_prof : nullptr;
    e = cudaLaunchKernelEx(&cfg, kern, ta, dp, ldd, M, N, Kc, lin, status, prof);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

template <int NP, int D>
static int launch_noise_pair(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, Sq5Lin lin,
                             int32_t *status, cudaStream_t st) {
    using Cfg = PairCfg<NP, D>;
    constexpr int CSZ = 2 * NP;
    CUtensorMap ta, td;
    int rc = make_tmap(&ta, a, Kc, M, lda, BK, BM);
    if (rc) return rc;
    rc = make_tmap(&td, d, N, M, ldd, 64, 32);   // output tiles of 32 rows x 64 columns
    if (rc) return rc;
    auto kern = noise_pair_kernel<NP, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_DYN);
    if (e != cudaSuccess) return (int)e;
    const int64_t ctiles = cdiv64(cdiv64(M, 4 * BM), NP) * cdiv64(N, Cfg::BN);

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_DYN;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CSZ;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;                       // the occupancy query below sees the cluster shape only
    cfg.gridDim = dim3(CSZ);
    int max_clusters = sm_count() / CSZ, n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) max_clusters = n;
    else (void)cudaGetLastError();
    const int64_t nclusters = ctiles < max_clusters ? ctiles : max_clusters;
    cfg.gridDim = dim3((unsigned)(nclusters * CSZ));
    cfg.numAttrs = 2;
    long long *prof = (g_prof && g_prof_bytes >= (size_t)cfg.gridDim.x * 16 * sizeof(long long)) ? g_prof : nullptr;
    e = cudaLaunchKernelEx(&cfg, kern, ta, td, M, N, Kc, lin, status, prof);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// o.noise_tile (RDB_OPT_NOISE_TILE): (cluster size, token sub-tiles, generated rows) per work unit
int umma_gemm_noise(void *d, const void *a, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldd, Sq5Lin lin,
                    int32_t *status, cudaStream_t st, const CallOpts &o) {
    if (M == 0 || N == 0) return RDB_OK;
    int cfg = o.noise_tile;
    // more than one 512-token tile: two CTA pairs per cluster that share every generated stage (half the hashing per SM);
    // a single token tile: one CTA per work unit when there are many of them (short contraction, many generated rows),
    // four pairs splitting the hashing of each stage when there are few (long generated contraction)
    if (cfg == 0) cfg = (M > 4 * BM) ? 8 : (Kc > 4096 ? 9 : 1);
    switch (cfg) {
        case 2: return launch_noise_gemm<1, 2, 256, 3, 3>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 3: return launch_noise_gemm<2, 4, 128, 2, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 4: return launch_noise_gemm<4, 4, 128, 2, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 5: return launch_noise_gemm<4, 2, 256, 3, 3>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 6: return launch_noise_gemm<1, 4, 128, 2, 6>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 7: return launch_noise_pair<1, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 8: return launch_noise_pair<2, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        case 9: return launch_noise_pair<4, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
        default: return launch_noise_gemm<1, 4, 128, 2, 4>(d, a, M, N, Kc, lda, ldd, lin, status, st);
    }
}

bool umma_shape_ok_dense(int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb, int64_t ldd, int d_dtype,
                         int a_kmajor, int b_kmajor, const void *a, const void *b, const void *d) {
    (void)d_dtype;
    // An MN-major operand has its M (or N) extent as the contiguous TMA dimension.
    if (!a_kmajor && (M % 8) != 0) return false;
    if (!b_kmajor && (N % 8) != 0) return false;
    return M >= 1 && N >= 8 && Kc >= 8 && (N % 8) == 0 && (Kc % 8) == 0 && (lda % 8) == 0 &&
           (ldb % 8) == 0 && (ldd % 8) == 0 && aligned16(a) && aligned16(b) && aligned16(d) && M < (1LL << 31) &&
           N < (1LL << 31) && Kc < (1LL << 31);
}

template <int BN, int STAGES, int A_MN, int B_MN, typename OutT>
static int launch_dense(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb,
                        int64_t ldd, int32_t *status, cudaStream_t st, int reserve_sms, int split = 1, int64_t slice_stride = 0) {
    using Cfg = DenseCfg<BN, STAGES>;
    CUtensorMap ta, tb;
    int rc = A_MN ? make_tmap(&ta, a, M, Kc, lda, 64, BK) : make_tmap(&ta, a, Kc, M, lda, BK, BM);
    if (rc) return rc;
    rc = B_MN ? make_tmap(&tb, b, N, Kc, ldb, 64, BK) : make_tmap(&tb, b, Kc, N, ldb, BK, BN);
    if (rc) return rc;
    CUtensorMap td = ta;                       // float32 outputs with ragged row tiles are stored directly: the map is not used
    int f32_tma = 0;
    if (sizeof(OutT) == 2) {
        rc = make_tmap(&td, d, N, M, ldd, 64, 32);   // output tiles of 32 rows x 64 columns
        if (rc) return rc;
    } else if ((M % BM) == 0 && (ldd % 4) == 0 && slice_stride == (split > 1 ? M * ldd : slice_stride)) {
        rc = make_tmap(&td, d, N, (int64_t)split * M, ldd, 32, 32, true);   // float32: 32 x 32 boxes over [split * M, N]
        if (rc) return rc;
        f32_tma = 1;
    }
    auto kern = dense_gemm_kernel<BN, STAGES, A_MN, B_MN, OutT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_DYN);
    if (e != cudaSuccess) return (int)e;
    const int64_t tiles = cdiv64(M, BM) * cdiv64(N, BN) * split;
    int ctas = sm_count() - reserve_sms;   // SMs left without a CTA for a collective that should run beside this launch
    if (ctas < 1) ctas = 1;
    const int grid = (int)(tiles < ctas ? tiles : ctas);
    // tiles that run at the same time share the panel of the larger operand, which is then streamed from memory once
    const int m_fast = (M <= N) ? 1 : 0;
    return launch_pdl(kern, dim3(grid), Cfg::THREADS, Cfg::SMEM_DYN, st, ta, tb, td, reinterpret_cast<OutT *>(d), ldd, M, N, Kc, m_fast,
                      split, slice_stride, f32_tma, status);
}

template <int MT, int D, int A_MN, int B_MN, int NDST, bool F32 = false>
static int launch_dense_pair(void *const *dsts, int64_t rows_per_dst, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc,
                             int64_t lda, int64_t ldb, int64_t ldd, int64_t tiles, int max_pairs, int32_t *status, cudaStream_t st,
                             int reserve_sms, int split = 1) {
    using Cfg = DensePairCfg<MT, D>;
    CUtensorMap ta, tb;
    OutMaps<NDST> out;
    int rc = A_MN ? make_tmap(&ta, a, M, Kc, lda, 64, BK) : make_tmap(&ta, a, Kc, M, lda, BK, BM);
    if (rc) return rc;
    rc = B_MN ? make_tmap(&tb, b, N, Kc, ldb, 64, BK) : make_tmap(&tb, b, Kc, N, ldb, BK, Cfg::HALF);
    if (rc) return rc;
    const int64_t ndst_used = NDST > 1 ? cdiv64(M, rows_per_dst) : 1;
    for (int j = 0; j < NDST; ++j) {
        // output tiles of 32 rows x 64 columns; unused entries repeat the first destination
        const int jj = j < ndst_used ? j : 0;
        const int64_t rows = NDST > 1 ? (M - jj * rows_per_dst < rows_per_dst ? M - jj * rows_per_dst : rows_per_dst) : M;
        rc = F32 ? make_tmap(&out.m[j], dsts[jj], N, (int64_t)split * M, ldd, 32, 32, true)   // float32 [split * M, N], 32 x 32 boxes
                 : make_tmap(&out.m[j], dsts[jj], N, rows, ldd, 64, 32);
        if (rc) return rc;
    }
    auto kern = dense_pair_kernel<MT, D, A_MN, B_MN, NDST, F32>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_DYN);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_DYN;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    int pairs = max_pairs - (reserve_sms + 1) / 2;
    if (pairs < 1) pairs = 1;
    const int64_t npairs = tiles < pairs ? tiles : pairs;
    cfg.gridDim = dim3((unsigned)(npairs * 2));
    // stream the larger operand once: consecutive tiles share the B panel when A is the smaller matrix
    const int m_fast = (M <= N) ? 1 : 0;
    long long *prof = (g_prof && g_prof_bytes >= (size_t)cfg.gridDim.x * 16 * sizeof(long long)) ? g_prof : nullptr;
    e = cudaLaunchKernelEx(&cfg, kern, ta, tb, out, rows_per_dst, M, N, Kc, m_fast, split, status, prof);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// how many CTA pairs can be resident at once (one CTA per SM)
static int max_resident_pairs() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev == cached_dev && cached > 0) return cached;
    auto kern = dense_pair_kernel<2, 4, 0, 0, 1, false>;
    int n = 0, fallback = sm_count() / 2;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DensePairCfg<2, 4>::SMEM_DYN) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.blockDim = dim3(DensePairCfg<2, 4>::THREADS);
        cfg.dynamicSmemBytes = DensePairCfg<2, 4>::SMEM_DYN;
        cfg.gridDim = dim3(2);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
    }
    (void)cudaGetLastError();
    cached_dev = dev;
    cached = n > 0 ? n : fallback;
    return cached;
}

// Whether the CTA-pair kernel (512 x 256 tiles, one tile per pair at a time, epilogue not overlapped) is expected to
// beat the single-CTA kernel (128 x 256 tiles, overlapped epilogue).  Measured on cfg-sized products: the pair kernel
// wins by 7-15 % when its tiles fill the resident pairs evenly, and loses when a short contraction meets a ragged
// last wave.
static bool prefer_dense_pair(int64_t M, int64_t N, int64_t Kc, int P) {
    if (M <= BM || N <= BM) return false;
    const int64_t tiles = cdiv64(M, 4 * BM) * cdiv64(N, 256);
    if (tiles * 5 < (int64_t)P * 4) return false;                       // fewer than 80 % of the pairs would work
    if (tiles <= P) return true;
    const double eff = (double)tiles / (double)(cdiv64(tiles, P) * P);  // share of the last wave that is used
    return eff >= 0.95 || (Kc >= 4096 && eff >= 0.85);
}

template <int A_MN, int B_MN>
static int dense_by_out(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb,
                        int64_t ldd, int d_dtype, int32_t *status, cudaStream_t st, const CallOpts &o) {
    const int rs = o.reserve_sms;
    if (d_dtype == RDB_BF16 && o.dense_pair && M > BM && N > BM) {
        const int P = max_resident_pairs();
        if (o.dense_pair == 2 || prefer_dense_pair(M, N, Kc, P))
            return launch_dense_pair<2, 4, A_MN, B_MN, 1>(&d, M, a, b, M, N, Kc, lda, ldb, ldd, cdiv64(M, 4 * BM) * cdiv64(N, 256), P,
                                                          status, st, rs);
    }
    // at most 128 output columns (a coefficient dimension of 128 or less): 128-column tiles, half the MMA and B traffic
    if (d_dtype == RDB_BF16 && N <= 128)
        return launch_dense<128, 6, A_MN, B_MN, __nv_bfloat16>(d, a, b, M, N, Kc, lda, ldb, ldd, status, st, rs);
    // a contraction of at most three k-blocks (the y and dX of a layer with a small coefficient matrix): every tile is mostly
    // epilogue, so the ring gives a stage up for a second staging box per epilogue warp
    if (d_dtype == RDB_BF16 && Kc <= 3 * BK)
        return launch_dense<256, 3, A_MN, B_MN, __nv_bfloat16>(d, a, b, M, N, Kc, lda, ldb, ldd, status, st, rs);
    if (d_dtype == RDB_BF16)
        return launch_dense<256, 4, A_MN, B_MN, __nv_bfloat16>(d, a, b, M, N, Kc, lda, ldb, ldd, status, st, rs);
    if (d_dtype == RDB_F32) return launch_dense<256, 4, A_MN, B_MN, float>(d, a, b, M, N, Kc, lda, ldb, ldd, status, st, rs);
    return RDB_ERR_DTYPE;
}

// ---- two independent products at the same time on disjoint sets of CTA pairs ------------------------------------------
// dX = g C (tokens x inputs, short contraction) and dC = g^T x (coefficients x inputs, long contraction) both read g and
// nothing of one another.  Alone, each leaves SMs idle when its tiles do not divide by the resident pairs (the headline
// layer: 256 tiles of 16 k-blocks and 32 tiles of 128 k-blocks for 74 pairs), and the single-CTA kernel that fills the SMs
// better pays a third more shared-memory traffic per MMA.  Side by side on p and P - p pairs the two tile lists pack
// (32 pairs x 128 k-blocks next to 42 pairs x 7 tiles x 16 k-blocks).  Costs are in SM cycles at the nominal MMA rate:
// a k-block of a 512 x 256 pair tile is 1024 cycles, of a 128 x 256 single-CTA tile 512 cycles times the measured 1.27.
static double pair_cost(int64_t M, int64_t N, int64_t Kc, int pairs) {
    const int64_t tiles = cdiv64(M, 4 * BM) * cdiv64(N, 256);
    return (double)cdiv64(tiles, pairs) * ((double)cdiv64(Kc, BK) * 1024.0 + 2500.0);   // + ring start and epilogue per tile
}

static double alone_cost(int64_t M, int64_t N, int64_t Kc, int P) {
    const int64_t tiles = cdiv64(M, BM) * cdiv64(N, 256);
    const double single = (double)cdiv64(tiles, sm_count()) * (double)cdiv64(Kc, BK) * 512.0 * 1.27;
    const double pair = pair_cost(M, N, Kc, P);
    return single < pair ? single : pair;
}

// Pairs for the first and the second product when running them side by side is expected to take less than 93 % of
// running them one after the other (`always`: whenever both can run on pairs); false otherwise.  `reserve_sms` SMs stay
// free as in every plain-product launch.
bool dense_beside_plan(int64_t M1, int64_t N1, int64_t Kc1, int64_t M2, int64_t N2, int64_t Kc2, int reserve_sms, bool always,
                       int *pairs1, int *pairs2) {
    if (M1 <= BM || N1 <= BM || M2 <= BM || N2 <= BM || Kc1 < BK || Kc2 < BK) return false;
    const int P = max_resident_pairs() - (reserve_sms + 1) / 2;
    if (P < 2) return false;
    double best = 0.0;
    int best_p = 0;
    for (int p = 1; p < P; ++p) {
        const double c1 = pair_cost(M1, N1, Kc1, p), c2 = pair_cost(M2, N2, Kc2, P - p);
        const double c = c1 > c2 ? c1 : c2;
        if (best_p == 0 || c <= best) { best = c; best_p = p; }   // among equals, the split that leaves no pair without a tile
    }
    if (!always && best > 0.93 * (alone_cost(M1, N1, Kc1, P) + alone_cost(M2, N2, Kc2, P))) return false;
    *pairs1 = best_p;
    *pairs2 = P - best_p;
    return true;
}

// D = op(A) op(B)^T (bf16) on at most `pairs` CTA pairs, whatever the tile count
int umma_gemm_dense_on_pairs(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb,
                             int64_t ldd, int a_kmajor, int b_kmajor, int pairs, int32_t *status, cudaStream_t st) {
    if (M == 0 || N == 0) return RDB_OK;
    const int64_t tiles = cdiv64(M, 4 * BM) * cdiv64(N, 256);
    if (a_kmajor && b_kmajor) return launch_dense_pair<2, 4, 0, 0, 1>(&d, M, a, b, M, N, Kc, lda, ldb, ldd, tiles, pairs, status, st, 0);
    if (a_kmajor) return launch_dense_pair<2, 4, 0, 1, 1>(&d, M, a, b, M, N, Kc, lda, ldb, ldd, tiles, pairs, status, st, 0);
    if (b_kmajor) return launch_dense_pair<2, 4, 1, 0, 1>(&d, M, a, b, M, N, Kc, lda, ldb, ldd, tiles, pairs, status, st, 0);
    return launch_dense_pair<2, 4, 1, 1, 1>(&d, M, a, b, M, N, Kc, lda, ldb, ldd, tiles, pairs, status, st, 0);
}

// ---- split-K: few output tiles, long contraction (dC = g^T x of a layer with a small coefficient matrix) ---------------
// Slices the contraction into `split` pieces that run as independent work items writing float32 partial products
// [split, M, N] into `partials`; split_k_reduce_kernel then sums the slices in a fixed order.
// Which kernel a split product runs on, and in how many slices.
//   CTA pairs: the 512 x 256 tiles would occupy at most half the resident pairs and the contraction is long enough for
//              slices of 64 k-blocks or more (256 in all at least) that together fill at least 80 % of the pairs (the
//              token-sliced z = x C^T of the row-sharded layer at 2 and 4 ranks); shorter slices lose to the single-CTA
//              kernel (ring start-up and an unoverlapped epilogue once per slice: 8 x 32 k-blocks measured 72 against 40 us,
//              2 x 64 of the headline dC 60.7 against 59.8);
//   single CTAs: the same idea on 128-row tiles for everything else with few tiles and a long contraction.
struct SplitPlan {
    int slices;
    bool pair;
};

static SplitPlan split_plan(int64_t M, int64_t N, int64_t Kc) {
    const int64_t kbs = cdiv64(Kc, BK);
    if (M > BM && N > BM && (M % 32) == 0 && kbs >= 256) {
        const int P = max_resident_pairs();
        const int64_t tiles_p = cdiv64(M, 4 * BM) * cdiv64(N, 256);
        if (tiles_p * 2 <= P) {
            int64_t sp = P / tiles_p;
            if (sp > kbs / 64) sp = kbs / 64;
            if (sp > 8) sp = 8;
            if (sp >= 2 && tiles_p * sp * 5 >= (int64_t)P * 4) {
                const int64_t kb_per = cdiv64(kbs, sp);
                return SplitPlan{(int)cdiv64(kbs, kb_per), true};
            }
        }
    }
    const int64_t tiles = cdiv64(M, BM) * cdiv64(N, N <= 128 ? 128 : 256);
    const int sms = sm_count();
    if (tiles * 2 > sms || kbs < 16) return SplitPlan{1, false};
    int64_t s = sms / tiles;                 // one wave of work items
    if (s > kbs / 4) s = kbs / 4;            // at least four k-blocks per slice
    if (s > 16) s = 16;                      // every slice writes and re-reads a float32 copy of the output
    if (s < 2) return SplitPlan{1, false};
    const int64_t kb_per = cdiv64(kbs, s);   // the kernel gives every slice this many k-blocks ...
    return SplitPlan{(int)cdiv64(kbs, kb_per), false};   // ... so this many slices are non-empty
}

int dense_split_k_slices(int64_t M, int64_t N, int64_t Kc) { return split_plan(M, N, Kc).slices; }

template <typename OutT>
__global__ void split_k_reduce_kernel(OutT *__restrict__ out, const float *__restrict__ partials, int64_t n4, int split,
                                      int64_t slice_stride4) {
    const float4 *p = reinterpret_cast<const float4 *>(partials);
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 acc = p[i];
        for (int s = 1; s < split; ++s) {
            const float4 v = p[i + s * slice_stride4];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (sizeof(OutT) == 4) {
            reinterpret_cast<float4 *>(out)[i] = acc;
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            uint2 v;
            v.x = *reinterpret_cast<uint32_t *>(&lo);
            v.y = *reinterpret_cast<uint32_t *>(&hi);
            reinterpret_cast<uint2 *>(out)[i] = v;
        }
    }
}

// d must be densely packed (ldd == N) and N a multiple of 8; partials: split * M * N floats
int umma_gemm_dense_split_k(void *d, const void *a, const void *b, float *partials, int split, int64_t M, int64_t N, int64_t Kc,
                            int64_t lda, int64_t ldb, int d_dtype, int a_kmajor, int b_kmajor, int32_t *status, cudaStream_t st,
                            const CallOpts &o) {
    if (M == 0 || N == 0) return RDB_OK;
    const int64_t stride = M * N;
    const int rs = o.reserve_sms;
    int rc;
    void *pp = partials;
    if (split_plan(M, N, Kc).pair) {
        const int P = max_resident_pairs();
        const int64_t items = cdiv64(M, 4 * BM) * cdiv64(N, 256) * split;
        if (a_kmajor && b_kmajor) rc = launch_dense_pair<2, 4, 0, 0, 1, true>(&pp, M, a, b, M, N, Kc, lda, ldb, N, items, P, status, st, rs, split);
        else if (a_kmajor) rc = launch_dense_pair<2, 4, 0, 1, 1, true>(&pp, M, a, b, M, N, Kc, lda, ldb, N, items, P, status, st, rs, split);
        else if (b_kmajor) rc = launch_dense_pair<2, 4, 1, 0, 1, true>(&pp, M, a, b, M, N, Kc, lda, ldb, N, items, P, status, st, rs, split);
        else rc = launch_dense_pair<2, 4, 1, 1, 1, true>(&pp, M, a, b, M, N, Kc, lda, ldb, N, items, P, status, st, rs, split);
    } else if (N <= 128) {
        if (a_kmajor && b_kmajor) rc = launch_dense<128, 6, 0, 0, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
        else if (a_kmajor) rc = launch_dense<128, 6, 0, 1, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
        else if (b_kmajor) rc = launch_dense<128, 6, 1, 0, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
        else rc = launch_dense<128, 6, 1, 1, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
    } else if (a_kmajor && b_kmajor) rc = launch_dense<256, 4, 0, 0, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
    else if (a_kmajor) rc = launch_dense<256, 4, 0, 1, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
    else if (b_kmajor) rc = launch_dense<256, 4, 1, 0, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
    else rc = launch_dense<256, 4, 1, 1, float>(partials, a, b, M, N, Kc, lda, ldb, N, status, st, rs, split, stride);
    if (rc) return rc;
    const int64_t n4 = stride / 4;
    const int grid = (int)(cdiv64(n4, 256) < 148 * 8 ? cdiv64(n4, 256) : 148 * 8);
    if (d_dtype == RDB_BF16)
        return launch_pdl(split_k_reduce_kernel<__nv_bfloat16>, dim3(grid), 256, 0, st, reinterpret_cast<__nv_bfloat16 *>(d),
                          (const float *)partials, n4, split, stride / 4);
    return launch_pdl(split_k_reduce_kernel<float>, dim3(grid), 256, 0, st, reinterpret_cast<float *>(d), (const float *)partials, n4,
                      split, stride / 4);
}

// D = A op(B)^T on CTA pairs with row block j of D stored into dsts[j] (dense [rows_per_dst x N] bf16 each, possibly in
// peer memory).  A K-major; B K-major or MN-major.
int umma_gemm_dense_scatter(void *const *dsts, int ndst, int64_t rows_per_dst, const void *a, const void *b, int64_t M, int64_t N,
                            int64_t Kc, int64_t lda, int64_t ldb, int b_kmajor, int32_t *status, cudaStream_t st, const CallOpts &o) {
    if (M == 0 || N == 0) return RDB_OK;
    if (ndst < 1 || ndst > RDB_MAX_PEERS || rows_per_dst <= 0 || (rows_per_dst % 32) != 0 || cdiv64(M, rows_per_dst) > ndst)
        return RDB_ERR_PEER;
    const int P = max_resident_pairs();
    const int64_t tiles = cdiv64(M, 4 * BM) * cdiv64(N, 256);
    if (b_kmajor)
        return launch_dense_pair<2, 4, 0, 0, RDB_MAX_PEERS>(dsts, rows_per_dst, a, b, M, N, Kc, lda, ldb, N, tiles, P, status, st, o.reserve_sms);
    return launch_dense_pair<2, 4, 0, 1, RDB_MAX_PEERS>(dsts, rows_per_dst, a, b, M, N, Kc, lda, ldb, N, tiles, P, status, st, o.reserve_sms);
}

int umma_gemm_dense(void *d, const void *a, const void *b, int64_t M, int64_t N, int64_t Kc, int64_t lda, int64_t ldb,
                    int64_t ldd, int d_dtype, int a_kmajor, int b_kmajor, int32_t *status, cudaStream_t st, const CallOpts &o) {
    if (M == 0 || N == 0) return RDB_OK;
    if (a_kmajor && b_kmajor) return dense_by_out<0, 0>(d, a, b, M, N, Kc, lda, ldb, ldd, d_dtype, status, st, o);
    if (a_kmajor && !b_kmajor) return dense_by_out<0, 1>(d, a, b, M, N, Kc, lda, ldb, ldd, d_dtype, status, st, o);
    if (!a_kmajor && b_kmajor) return dense_by_out<1, 0>(d, a, b, M, N, Kc, lda, ldb, ldd, d_dtype, status, st, o);
    return dense_by_out<1, 1>(d, a, b, M, N, Kc, lda, ldb, ldd, d_dtype, status, st, o);
}

}  // namespace rdb
