// Exchange steps of the row-sharded layer over peer memory (NVLink / NVSwitch), written as plain kernels of this
// library: every rank maps the other ranks' exchange buffers into its own address space (the host side hands over the
// pointers) and the kernels here store into them directly.
//
//   peer_barrier_kernel   all ranks have reached this point of their streams (and their earlier stores have landed)
//   peer_copy_kernel      one contiguous block -> the same offset in every listed destination (the all-gather step)
//   peer_scatter_kernel   row block j of a matrix -> destination j (the scatter half of a reduce-scatter)
//   reduce_slots_kernel   sum of `nslots` bf16 blocks in a fixed order, float32 accumulation (the reduce half)
//
// Only plain st.global / ld.global with system-scope release/acquire on the flags cross GPUs: no TMA multicast, no
// multimem.  Every wait is bounded: a rank that does not show up within the limit makes the waiting kernel record
// RDB_STATUS_TIMEOUT_PEER and return, so the context stays usable.  The reference has no counterpart (its only
// collectives are DDP's: modded-nanogpt/train_gpt2.py:346, 441).
#include "common.cuh"

namespace rdb {

struct PeerPtrs {
    void *p[RDB_MAX_PEERS];
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// flags[r] of rank p is written only by rank r.  Epochs only grow, so nothing is ever reset and a slow rank cannot
// miss a value.  One thread per peer: signal it, then wait for its signal.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, unsigned long long epoch, unsigned long long limit_ns,
                                    int32_t *status) {
    const int t = threadIdx.x;
    if (t >= world) return;
    __threadfence_system();   // everything this GPU wrote before (earlier kernels of the stream included) is ordered first
    unsigned long long *theirs = reinterpret_cast<unsigned long long *>(flags.p[t]) + rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(theirs), "l"(epoch) : "memory");
    const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(flags.p[rank]) + t;
    const unsigned long long t0 = global_timer_ns();
    unsigned long long v = 0;
    unsigned spins = 0;
    while (true) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
        if (v >= epoch) break;
        if (((++spins) & 63) == 0 && global_timer_ns() - t0 > limit_ns) {
            if (status) atomicCAS(status, 0, RDB_STATUS_TIMEOUT_PEER);
            break;
        }
    }
}

// dst[d][dst_off + i] = src[i] for every destination d of the list (16-byte units)
__global__ void __launch_bounds__(256) peer_copy_kernel(PeerPtrs dst, int ndst, size_t dst_off16, const uint4 *__restrict__ src,
                                                        size_t n16) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (int d = 0; d < ndst; ++d) reinterpret_cast<uint4 *>(dst.p[d])[dst_off16 + i] = v;
    }
}

// block j (n16 units) of src -> dst[j][dst_off + ...]
__global__ void __launch_bounds__(256) peer_scatter_kernel(PeerPtrs dst, int ndst, size_t dst_off16, const uint4 *__restrict__ src,
                                                           size_t n16) {
    const size_t total = n16 * (size_t)ndst;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t j = i / n16, k = i - j * n16;
        reinterpret_cast<uint4 *>(dst.p[j])[dst_off16 + k] = src[i];
    }
}

// out[i] = bf16( sum_s float(slots[s * stride + i]) ), s ascending; 8 bf16 per thread and step
__global__ void __launch_bounds__(256) reduce_slots_kernel(uint4 *__restrict__ out, const uint4 *__restrict__ slots, size_t stride16,
                                                           int nslots, size_t n16) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < nslots; ++s) {
            const uint4 v = slots[(size_t)s * stride16 + i];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] += __uint_as_float(w[j] << 16);
                acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            p[j] = *reinterpret_cast<uint32_t *>(&h);
        }
        out[i] = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

static int peers_ok(void *const *ptrs, int n) {
    if (!ptrs || n < 1 || n > RDB_MAX_PEERS) return RDB_ERR_PEER;
    for (int i = 0; i < n; ++i)
        if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return RDB_ERR_PEER;
    return RDB_OK;
}

static int grid_blocks(size_t items, int max_blocks) {
    size_t g = (items + 255) / 256;
    const size_t cap = max_blocks > 0 ? (size_t)max_blocks : 148 * 4;
    if (g > cap) g = cap;
    return g < 1 ? 1 : (int)g;
}

}  // namespace rdb

using namespace rdb;

extern "C" int rdb_peer_barrier(void *const *flag_ptrs, int rank, int world, uint64_t epoch, int32_t *status, void *stream) {
    int rc = peers_ok(flag_ptrs, world);
    if (rc) return rc;
    if (rank < 0 || rank >= world || epoch == 0) return RDB_ERR_PEER;
    PeerPtrs f{};
    for (int i = 0; i < world; ++i) f.p[i] = flag_ptrs[i];
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, rank, world, epoch, RDB_PEER_WAIT_LIMIT_NS, status);
    return launch_status();
}

extern "C" int rdb_peer_copy(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, const void *src, size_t nbytes,
                             int max_blocks, void *stream) {
    int rc = peers_ok(dst_ptrs, ndst);
    if (rc) return rc;
    if ((dst_offset_bytes & 15) || (nbytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return RDB_ERR_ALIGN;
    if (nbytes == 0) return RDB_OK;
    if (!src) return RDB_ERR_NULL;
    PeerPtrs d{};
    for (int i = 0; i < ndst; ++i) d.p[i] = dst_ptrs[i];
    peer_copy_kernel<<<grid_blocks(nbytes / 16, max_blocks), 256, 0, (cudaStream_t)stream>>>(d, ndst, dst_offset_bytes / 16,
                                                                                             reinterpret_cast<const uint4 *>(src), nbytes / 16);
    return launch_status();
}

extern "C" int rdb_peer_scatter(void *const *dst_ptrs, int ndst, size_t dst_offset_bytes, const void *src, size_t block_bytes,
                                int max_blocks, void *stream) {
    int rc = peers_ok(dst_ptrs, ndst);
    if (rc) return rc;
    if ((dst_offset_bytes & 15) || (block_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return RDB_ERR_ALIGN;
    if (block_bytes == 0) return RDB_OK;
    if (!src) return RDB_ERR_NULL;
    PeerPtrs d{};
    for (int i = 0; i < ndst; ++i) d.p[i] = dst_ptrs[i];
    peer_scatter_kernel<<<grid_blocks(block_bytes / 16 * ndst, max_blocks), 256, 0, (cudaStream_t)stream>>>(
        d, ndst, dst_offset_bytes / 16, reinterpret_cast<const uint4 *>(src), block_bytes / 16);
    return launch_status();
}

extern "C" int rdb_reduce_slots_bf16(void *out, const void *slots, size_t slot_stride_bytes, int nslots, size_t nbytes,
                                     void *stream) {
    if (nslots < 1 || nslots > RDB_MAX_PEERS) return RDB_ERR_PEER;
    if ((nbytes & 15) || (slot_stride_bytes & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (reinterpret_cast<uintptr_t>(slots) & 15))
        return RDB_ERR_ALIGN;
    if (nbytes == 0) return RDB_OK;
    if (!out || !slots) return RDB_ERR_NULL;
    reduce_slots_kernel<<<grid_blocks(nbytes / 16, 0), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<uint4 *>(out), reinterpret_cast<const uint4 *>(slots), slot_stride_bytes / 16, nslots, nbytes / 16);
    return launch_status();
}
