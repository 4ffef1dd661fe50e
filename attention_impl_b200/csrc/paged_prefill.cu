// Chunked / prefix-cached prefill through the slot table: several query rows per sequence attend to
// that sequence's KV rows in the paged pools.
//
// Not in the reference (its packed prefill reads K, V next to Q, its paged operator has one query
// row).  This is the operation that unifies the two: the last q_len_b tokens of sequence b are
// queries, all kv_len_b tokens (the prefix from earlier steps plus the chunk itself, already
// appended to the pools) are keys; query i sees key j iff j <= kv_len_b - q_len_b + i.
//
// Generic kernel: one warp per (query row, head), lanes over keys for the scores (kept in shared
// memory), lanes over dims for P*V; fp32 accumulation, true row maximum.  Any dtype / head_dim,
// grouped-query heads; KV length per sequence limited by shared memory (12 288 keys).
#include "common.cuh"

namespace attn {

struct PagedPrefillParams {
    const void* q;
    const void* k_cache;
    const void* v_cache;
    const int32_t* slots;
    const int32_t* kv_offsets;
    const int32_t* q_offsets;
    void* out;
    int B, H, Hkv, D;
    int64_t n_q_tokens, n_kv_tokens, n_slots;
    int max_q_len, max_kv_len;
    float scale;
    int32_t* err_flag;
};

constexpr int kPpWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kPpWarps * 32)
paged_prefill_generic_kernel(const PagedPrefillParams p) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int i = blockIdx.x * kPpWarps + warp;              // query row within the sequence's chunk
    const int64_t qb = b ? p.q_offsets[b - 1] : 0, qe = p.q_offsets[b];
    const int64_t kb = b ? p.kv_offsets[b - 1] : 0, ke = p.kv_offsets[b];
    if (qb < 0 || qe < qb || qe > p.n_q_tokens || kb < 0 || ke < kb || ke > p.n_kv_tokens) {
        if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
        return;
    }
    const int q_len = (int)(qe - qb);
    int kv_len = (int)(ke - kb);
    if (i >= q_len) return;
    if (kv_len > p.max_kv_len) kv_len = p.max_kv_len;
    const int D = p.D, G = p.H / p.Hkv, hk = h / G;
    float* sq = smem + (size_t)warp * (p.D + p.max_kv_len);
    float* sc = sq + p.D;
    const T* Q = (const T*)p.q;
    const T* K = (const T*)p.k_cache;
    const T* V = (const T*)p.v_cache;
    for (int d = lane; d < D; d += 32) sq[d] = to_f32<T>(Q[((qb + i) * p.H + h) * D + d]);
    __syncwarp();
    int jmax = kv_len - q_len + i + 1;                       // keys 0 .. kv_len - q_len + i are visible
    if (jmax < 0) jmax = 0;
    if (jmax > kv_len) jmax = kv_len;
    float mx = -INFINITY;
    for (int j = lane; j < jmax; j += 32) {
        const int64_t s = p.slots[kb + j];
        float acc = -INFINITY;
        if (s >= 0 && s < p.n_slots) {
            const T* kr = K + (s * p.Hkv + hk) * D;
            acc = 0.f;
            for (int d = 0; d < D; ++d) acc = fmaf(sq[d], to_f32<T>(kr[d]), acc);
            acc *= p.scale;
        } else if (p.err_flag) {
            atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
        }
        sc[j] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = group_max<32>(mx);
    float sum = 0.f;
    for (int j = lane; j < jmax; j += 32) {
        const float e = (mx > -INFINITY && sc[j] > -INFINITY) ? __expf(sc[j] - mx) : 0.f;
        sc[j] = e;
        sum += e;
    }
    sum = group_sum<32>(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int j = 0; j < jmax; ++j) {
            const float pj = sc[j];
            if (pj != 0.f) acc = fmaf(pj, to_f32<T>(V[((int64_t)p.slots[kb + j] * p.Hkv + hk) * D + d]), acc);
        }
        ((T*)p.out)[((qb + i) * p.H + h) * D + d] = from_f32<T>(acc * inv);
    }
}

template <typename T>
static int launch_pp(const PagedPrefillParams& p, cudaStream_t st) {
    const size_t smem = (size_t)kPpWarps * (p.D + p.max_kv_len) * sizeof(float);
    if (smem > 200 * 1024) return ATTN_B200_ETOOLARGE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(paged_prefill_generic_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (p.H > 65535 || p.B > 65535) return ATTN_B200_ETOOLARGE;
    dim3 grid((p.max_q_len + kPpWarps - 1) / kPpWarps, p.H, p.B);
    paged_prefill_generic_kernel<T><<<grid, kPpWarps * 32, smem, st>>>(p);
    return (int)cudaGetLastError();
}

int paged_prefill_tc_launch(const PagedPrefillParams& p, int dtype, cudaStream_t st);
bool paged_prefill_tc_supported(const PagedPrefillParams& p, int dtype);

}  // namespace attn

using namespace attn;

extern "C" int attn_b200_paged_prefill(const void* q, const void* k_cache, const void* v_cache, const int32_t* slots,
                                       const int32_t* kv_offsets, const int32_t* q_offsets, void* out, int B,
                                       int64_t n_q_tokens, int64_t n_kv_tokens, int max_q_len, int max_kv_len, int H,
                                       int n_kv_heads, int D, int64_t n_slots, float scale, int dtype,
                                       int force_generic, int32_t* err_flag, void* stream) {
    if (!q || !k_cache || !v_cache || !slots || !kv_offsets || !q_offsets || !out || B <= 0 || H <= 0 || D <= 0 ||
        n_q_tokens < 0 || n_kv_tokens < 0 || n_slots <= 0 || max_q_len < 0 || max_kv_len < 0)
        return ATTN_B200_EINVAL;
    if (n_kv_heads <= 0 || H % n_kv_heads) return ATTN_B200_ESHAPE;
    if (n_q_tokens == 0 || max_q_len == 0) return 0;
    PagedPrefillParams p{q, k_cache, v_cache, slots, kv_offsets, q_offsets, out, B, H, n_kv_heads, D, n_q_tokens,
                         n_kv_tokens, n_slots, max_q_len, max_kv_len, scale, err_flag};
    cudaStream_t st = (cudaStream_t)stream;
    if (!force_generic && paged_prefill_tc_supported(p, dtype)) return paged_prefill_tc_launch(p, dtype, st);
    switch (dtype) {
        case ATTN_B200_F16: return launch_pp<__half>(p, st);
        case ATTN_B200_BF16: return launch_pp<__nv_bfloat16>(p, st);
        case ATTN_B200_F32: return launch_pp<float>(p, st);
        default: return ATTN_B200_EDTYPE;
    }
}

// Tensor-core form (tcgen05, K/V gathered into shared memory by cp.async): prefill_tc.cu
namespace attn {
int paged_prefill_tc_launch_impl(const void* q, const void* k_cache, const void* v_cache, const int32_t* slots,
                                 const int32_t* kv_offsets, const int32_t* q_offsets, void* out, int B,
                                 int64_t n_q_tokens, int64_t n_kv_tokens, int max_q_len, int H, int Hkv, int D,
                                 int64_t n_slots, float scale, int dtype, int32_t* err_flag, cudaStream_t st);
bool paged_prefill_tc_supported(const PagedPrefillParams& p, int dtype) {
    return p.D == 128 && (dtype == ATTN_B200_F16 || dtype == ATTN_B200_BF16);
}
int paged_prefill_tc_launch(const PagedPrefillParams& p, int dtype, cudaStream_t st) {
    return paged_prefill_tc_launch_impl(p.q, p.k_cache, p.v_cache, p.slots, p.kv_offsets, p.q_offsets, p.out, p.B,
                                        p.n_q_tokens, p.n_kv_tokens, p.max_q_len, p.H, p.Hkv, p.D, p.n_slots, p.scale,
                                        dtype, p.err_flag, st);
}
}  // namespace attn
