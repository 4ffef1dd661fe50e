// Peer-memory exchange of the KV-split partial rows: instead of an NCCL all-gather, every rank
// stores its [B, H, D+2] fp32 rows straight into its slot of each peer's gather buffer with plain
// 16-byte stores over NVLink, then bumps a per-source arrival counter on the peer with a
// system-scope atomic.  The consumer side is a one-warp kernel that polls those counters with a
// bounded wait, placed in stream order before the log-sum-exp combine.  No multicast of any kind
// is used; the peer buffers are ordinary device allocations mapped into this process (CUDA IPC /
// symmetric memory), and a remote row lands in local HBM before any CTA consumes it.
//
// Counters are monotonic (never reset): after the s-th exchange every counter holds s * n_ctas.
#include "common.cuh"

namespace attn {

constexpr int kMaxPeers = 16;
constexpr int kPushThreads = 256;
constexpr int kPushVecPerThread = 4;
constexpr long long kWaitCycles = 2000000000LL;

struct PushParams {
    const uint4* src;
    int64_t n_vec;                 // 16-byte vectors
    uint4* dst[kMaxPeers];         // peer buffers, already offset to this rank's slot
    int32_t* flag[kMaxPeers];      // peer counters, already offset to this rank's entry
    int n_peers;
};

__global__ void __launch_bounds__(kPushThreads)
peer_push_kernel(const PushParams p) {
    const int64_t base = (int64_t)blockIdx.x * (kPushThreads * kPushVecPerThread) + threadIdx.x;
    uint4 v[kPushVecPerThread];
#pragma unroll
    for (int k = 0; k < kPushVecPerThread; ++k) {
        const int64_t i = base + (int64_t)k * kPushThreads;
        v[k] = i < p.n_vec ? p.src[i] : make_uint4(0, 0, 0, 0);
    }
    for (int g = 0; g < p.n_peers; ++g) {
#pragma unroll
        for (int k = 0; k < kPushVecPerThread; ++k) {
            const int64_t i = base + (int64_t)k * kPushThreads;
            if (i < p.n_vec) p.dst[g][i] = v[k];
        }
    }
    __threadfence_system();        // my stores are visible system-wide before the counter moves
    __syncthreads();
    if (threadIdx.x < p.n_peers) atomicAdd_system(p.flag[threadIdx.x], 1);
}

// One thread per counter; gives up after kWaitCycles and raises ATTN_B200_FLAG_TIMEOUT.
// With `consume` the thread takes `expected` off its counter once it has been reached (system-scope
// atomic: peers may already be adding the arrivals of their next push), so that the same `expected`
// serves every step and the launch can be replayed from a CUDA graph.
__global__ void wait_flags_kernel(int32_t* flags, int n, int32_t expected, int32_t* err_flag, int consume) {
    const int i = threadIdx.x;
    if (i >= n) return;
    int32_t* f = flags + i;
    const long long t0 = clock64();
    while (true) {
        int32_t v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v - expected >= 0) {
            if (consume) atomicSub_system(f, expected);
            break;
        }
        if (clock64() - t0 > kWaitCycles) {
            if (err_flag) atomicOr(err_flag, ATTN_B200_FLAG_TIMEOUT);
            break;
        }
        __nanosleep(64);
    }
}

}  // namespace attn

using namespace attn;

extern "C" int attn_b200_peer_push_ctas(size_t n_bytes) {
    const int64_t n_vec = (int64_t)(n_bytes / 16);
    return (int)((n_vec + kPushThreads * kPushVecPerThread - 1) / (kPushThreads * kPushVecPerThread));
}

extern "C" int attn_b200_peer_push(const void* src, size_t n_bytes, void* const* peer_dst,
                                   int32_t* const* peer_flag, int n_peers, void* stream) {
    if (!src || !peer_dst || !peer_flag || n_peers <= 0 || n_bytes == 0) return ATTN_B200_EINVAL;
    if (n_peers > kMaxPeers) return ATTN_B200_ETOOLARGE;
    if (n_bytes % 16 || (uintptr_t)src % 16) return ATTN_B200_EINVAL;
    PushParams p;
    p.src = (const uint4*)src;
    p.n_vec = (int64_t)(n_bytes / 16);
    p.n_peers = n_peers;
    for (int g = 0; g < n_peers; ++g) {
        if (!peer_dst[g] || !peer_flag[g] || (uintptr_t)peer_dst[g] % 16) return ATTN_B200_EINVAL;
        p.dst[g] = (uint4*)peer_dst[g];
        p.flag[g] = peer_flag[g];
    }
    peer_push_kernel<<<(unsigned)attn_b200_peer_push_ctas(n_bytes), kPushThreads, 0, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
}

extern "C" int attn_b200_wait_flags(const int32_t* flags, int n_flags, int32_t expected, int32_t* err_flag,
                                    void* stream) {
    if (!flags || n_flags <= 0 || n_flags > 32) return ATTN_B200_EINVAL;
    wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(const_cast<int32_t*>(flags), n_flags, expected, err_flag, 0);
    return (int)cudaGetLastError();
}

extern "C" int attn_b200_wait_flags_consume(int32_t* flags, int n_flags, int32_t count, int32_t* err_flag,
                                            void* stream) {
    if (!flags || n_flags <= 0 || n_flags > 32 || count <= 0) return ATTN_B200_EINVAL;
    wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n_flags, count, err_flag, 1);
    return (int)cudaGetLastError();
}
