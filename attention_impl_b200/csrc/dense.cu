// Generic dense / packed attention kernel (any dtype, any head_dim) and the host entry points
// for packed causal prefill and dense masked attention.
//
// This is the compatibility path: it materialises S and P when asked (the reference API returns
// them: paged_attention_kernel.cu:207-208,234, attention_kernel.cu:199-200,228), handles the
// explicit [B, L, L] mask of the naive entry point and the tiny head dims the reference's tests
// use.  Scores are  scale*<q,k> + (mask-1)*fill  (tests/test_naive_attention.py:18-21,
// tests/test_packed_attention.py:14-18); softmax subtracts the true row maximum.
// One warp owns one query row: lanes over keys for the scores (kept in shared memory), lanes over
// dims for P*V.  The tensor-core path for large packed prefill lives in prefill_tc.cu.
#include "common.cuh"

namespace attn {

int prefill_tc_launch(const void* q, const void* k, const void* v, const int32_t* offsets, void* out, int B,
                      int64_t n_tokens, int max_len, int H, int D, float scale, int dtype, int out_f32, int precise,
                      int32_t* err_flag, cudaStream_t st);
bool prefill_tc_supported(int D, int dtype);

struct DenseParams {
    const void* q;
    const void* k;
    const void* v;
    const void* mask;          // [B, L, L] or null
    const int32_t* offsets;    // packed mode: inclusive cumulative lengths; null => dense [B, L]
    void* out;
    void* S;
    void* P;
    int B, H, D;
    int L;                     // dense: sequence length; packed: max_len (leading dim of S/P)
    int64_t n_tokens;
    float scale, fill;
    int causal;
    int32_t* err_flag;
};

constexpr int kDenseWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kDenseWarps * 32)
dense_attention_kernel(const DenseParams p) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int i = blockIdx.x * kDenseWarps + warp;
    int64_t beg;
    int len;
    if (p.offsets) {
        int64_t e = p.offsets[b];
        beg = b ? p.offsets[b - 1] : 0;
        if (beg < 0 || e < beg || e > p.n_tokens) {
            if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
            return;
        }
        len = (int)(e - beg);
        if (len > p.L) {       // max_len understates this sequence: rows past it are not computed
            if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
            len = p.L;
        }
    } else {
        beg = (int64_t)b * p.L;
        len = p.L;
    }
    if (i >= len) return;
    const int D = p.D, HD = p.H * p.D;
    float* sq = smem + (size_t)warp * (p.D + p.L);
    float* sc = sq + p.D;
    const T* Q = (const T*)p.q;
    const T* K = (const T*)p.k;
    const T* V = (const T*)p.v;
    const T* M = (const T*)p.mask;
    for (int d = lane; d < D; d += 32) sq[d] = to_f32<T>(Q[(beg + i) * HD + h * D + d]);
    __syncwarp();
    const bool all_keys = p.S != nullptr || M != nullptr || !p.causal;
    const int jmax = all_keys ? len : i + 1;
    const int64_t sp_row = (((int64_t)b * p.H + h) * p.L + i) * p.L;
    float mx = -INFINITY;
    for (int j = lane; j < jmax; j += 32) {
        const T* kr = K + (beg + j) * HD + h * D;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) acc = fmaf(sq[d], to_f32<T>(kr[d]), acc);
        const float mv = M ? to_f32<T>(M[((int64_t)b * p.L + i) * p.L + j]) : ((p.causal && j > i) ? 0.f : 1.f);
        float s = acc * p.scale;
        if (mv != 1.f) s += (mv - 1.f) * p.fill;
        sc[j] = s;
        mx = fmaxf(mx, s);
        if (p.S) ((T*)p.S)[sp_row + j] = from_f32<T>(s);
    }
    mx = group_max<32>(mx);
    float sum = 0.f;
    for (int j = lane; j < jmax; j += 32) {
        const float e = __expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = group_sum<32>(sum);
    const float inv = 1.f / sum;
    __syncwarp();
    if (p.P)
        for (int j = lane; j < jmax; j += 32) ((T*)p.P)[sp_row + j] = from_f32<T>(sc[j] * inv);
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int j = 0; j < jmax; ++j) acc = fmaf(sc[j], to_f32<T>(V[(beg + j) * HD + h * D + d]), acc);
        ((T*)p.out)[(beg + i) * HD + h * D + d] = from_f32<T>(acc * inv);
    }
}

template <typename T>
static int launch_dense_t(const DenseParams& p, cudaStream_t st) {
    const size_t smem = (size_t)kDenseWarps * (p.D + p.L) * sizeof(float);
    if (smem > 200 * 1024) return ATTN_B200_ETOOLARGE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(dense_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (p.H > 65535 || p.B > 65535) return ATTN_B200_ETOOLARGE;
    dim3 grid((p.L + kDenseWarps - 1) / kDenseWarps, p.H, p.B);
    dense_attention_kernel<T><<<grid, kDenseWarps * 32, smem, st>>>(p);
    return (int)cudaGetLastError();
}

static int launch_dense(const DenseParams& p, int dtype, cudaStream_t st) {
    switch (dtype) {
        case ATTN_B200_F16: return launch_dense_t<__half>(p, st);
        case ATTN_B200_BF16: return launch_dense_t<__nv_bfloat16>(p, st);
        case ATTN_B200_F32: return launch_dense_t<float>(p, st);
        default: return ATTN_B200_EDTYPE;
    }
}

}  // namespace attn

using namespace attn;

extern "C" int attn_b200_varlen_prefill(const void* q, const void* k, const void* v, const int32_t* offsets,
                                        void* out, void* S, void* P, int B, int64_t n_tokens, int max_len, int H,
                                        int D, float scale, int dtype, int out_flags, int force_generic,
                                        int32_t* err_flag, void* stream) {
    const int out_f32 = out_flags & ATTN_B200_PREFILL_OUT_F32, precise = out_flags & ATTN_B200_PREFILL_PRECISE_P;
    if (!q || !k || !v || !offsets || !out || B <= 0 || H <= 0 || D <= 0 || n_tokens < 0 || max_len < 0)
        return ATTN_B200_EINVAL;
    if ((S == nullptr) != (P == nullptr)) return ATTN_B200_EINVAL;
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t out_el = out_f32 ? 4 : (dtype == ATTN_B200_F32 ? 4 : 2);
    if (max_len == 0)          // no sequence has a token: the output is all zeros, as the reference's zeros_like
        return (int)cudaMemsetAsync(out, 0, (size_t)n_tokens * H * D * out_el, st);
    if (!force_generic && !S && prefill_tc_supported(D, dtype))
        return prefill_tc_launch(q, k, v, offsets, out, B, n_tokens, max_len, H, D, scale, dtype, out_f32, precise,
                                 err_flag, st);
    if (out_f32) return ATTN_B200_EDTYPE;
    DenseParams p{q, k, v, nullptr, offsets, out, S, P, B, H, D, max_len, n_tokens, scale, 10000.f, 1, err_flag};
    return launch_dense(p, dtype, st);
}

extern "C" int attn_b200_dense_attention(const void* q, const void* k, const void* v, const void* mask, void* out,
                                         void* S, void* P, int B, int L, int H, int D, float scale, float fill,
                                         int dtype, void* stream) {
    if (!q || !k || !v || !out || B <= 0 || L <= 0 || H <= 0 || D <= 0) return ATTN_B200_EINVAL;
    if ((S == nullptr) != (P == nullptr)) return ATTN_B200_EINVAL;
    DenseParams p{q, k, v, mask, nullptr, out, S, P, B, H, D, L, (int64_t)B * L, scale, fill, 0, nullptr};
    return launch_dense(p, dtype, (cudaStream_t)stream);
}
