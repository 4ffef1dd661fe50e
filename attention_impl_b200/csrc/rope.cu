// In-place rotary embedding (NeoX pairing) for sm_100a.
//
// Semantics follow rotary_embedding.cu:10-36 of the reference: for a head's first
// rot_dim = 2*rot_half dims, x[d] <- x[d]*c - x[d+rh]*s and x[d+rh] <- x[d+rh]*c + x[d]*s with
// c,s = cos/sin[positions[token], d], every product and the sum rounded to the tensor's dtype
// (the reference computes in scalar_t).  Unlike the reference, both partner elements are read
// into registers before either is written, so there is no cross-warp read/write race.
//
// The kernel is pure streaming: per (token, head) it moves 2*rot_dim elements in and out.  The
// vector kernel gives each thread one 16-byte chunk of the first half and its partner chunk of
// the second half (4 loads + 2 table loads in flight per thread), so a warp touches whole
// 128-byte lines.  cos/sin rows are shared by all heads of a token and come from L1/L2.
#include "common.cuh"

namespace attn {

template <typename T> struct RnArith;
template <> struct RnArith<float> {
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float neg(float a) { return -a; }
};
template <> struct RnArith<__half> {
    static __device__ __forceinline__ __half mul(__half a, __half b) { return __hmul_rn(a, b); }
    static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd_rn(a, b); }
    static __device__ __forceinline__ __half neg(__half a) { return __hneg(a); }
};
template <> struct RnArith<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 mul(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat16 neg(__nv_bfloat16 a) { return __hneg(a); }
};
template <typename T2> struct RnArith2;
template <> struct RnArith2<__half2> {
    static __device__ __forceinline__ __half2 mul(__half2 a, __half2 b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ __half2 add(__half2 a, __half2 b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ __half2 neg(__half2 a) { return __hneg2(a); }
};
template <> struct RnArith2<__nv_bfloat162> {
    static __device__ __forceinline__ __nv_bfloat162 mul(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat162 add(__nv_bfloat162 a, __nv_bfloat162 b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat162 neg(__nv_bfloat162 a) { return __hneg2(a); }
};

// 16-bit types, rot_half % 8 == 0, head_dim % 8 == 0: a thread rotates 8 elements and their 8
// partners at a time.  One CTA per token: the position is read once, all index arithmetic is 32-bit
// and a thread walks several (chunk, partner) pairs of the token, q heads first, then k.  (With one
// thread per pair over the whole batch - a 64-bit division and four loads per thread - the same
// arithmetic ran at 0.88 of the measured copy bandwidth against 0.92.)
template <typename T2>
__global__ void __launch_bounds__(256)
rope_token_kernel(uint4* __restrict__ q, uint4* __restrict__ k, const int32_t* __restrict__ positions,
                  const uint4* __restrict__ cos, const uint4* __restrict__ sin, int n_heads_q, int n_heads_k,
                  int head_vec, int half_vec, int64_t max_pos, int32_t* __restrict__ err_flag) {
    const int64_t token = blockIdx.x;
    const int pos = positions[token];
    if (pos < 0 || pos >= max_pos) {
        if (err_flag && threadIdx.x == 0) atomicOr(err_flag, ATTN_B200_FLAG_BAD_POSITION);
        return;
    }
    const uint4* cosr = cos + (int64_t)pos * half_vec;
    const uint4* sinr = sin + (int64_t)pos * half_vec;
    uint4* qrow = q + token * n_heads_q * head_vec;
    uint4* krow = k ? k + token * n_heads_k * head_vec : nullptr;
    const int q_items = n_heads_q * half_vec, items = q_items + n_heads_k * half_vec;
    using A = RnArith2<T2>;
    for (int r = threadIdx.x; r < items; r += blockDim.x) {
        const bool is_q = r < q_items;
        const int rr = is_q ? r : r - q_items;
        const int head = rr / half_vec, c = rr - head * half_vec;
        uint4* base = (is_q ? qrow : krow) + head * head_vec;
        uint4 x1 = base[c], x2 = base[c + half_vec];
        const uint4 cs = __ldg(cosr + c), sn = __ldg(sinr + c);
        T2* a = reinterpret_cast<T2*>(&x1);
        T2* b = reinterpret_cast<T2*>(&x2);
        const T2* cc = reinterpret_cast<const T2*>(&cs);
        const T2* ss = reinterpret_cast<const T2*>(&sn);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const T2 lo = A::add(A::mul(a[i], cc[i]), A::mul(A::neg(b[i]), ss[i]));
            const T2 hi = A::add(A::mul(b[i], cc[i]), A::mul(a[i], ss[i]));
            a[i] = lo;
            b[i] = hi;
        }
        base[c] = x1;
        base[c + half_vec] = x2;
    }
}

// Any dtype / any rot_half: one thread per (token, head, d < rot_half).
template <typename T>
__global__ void __launch_bounds__(256)
rope_scalar_kernel(T* __restrict__ q, T* __restrict__ k, const int32_t* __restrict__ positions,
                   const T* __restrict__ cos, const T* __restrict__ sin, int64_t n_items, int n_heads_q,
                   int n_heads_k, int head_dim, int rot_half, int64_t max_pos, int32_t* __restrict__ err_flag) {
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_items) return;
    const int per_token = (n_heads_q + n_heads_k) * rot_half;
    const int64_t token = g / per_token;
    const int r = (int)(g - token * per_token);
    const int head = r / rot_half;
    const int d = r - head * rot_half;
    const int pos = positions[token];
    if (pos < 0 || pos >= max_pos) {
        if (err_flag) atomicOr(err_flag, ATTN_B200_FLAG_BAD_POSITION);
        return;
    }
    T* base = head < n_heads_q ? q + (token * n_heads_q + head) * head_dim
                               : k + (token * n_heads_k + (head - n_heads_q)) * head_dim;
    const T c = cos[(int64_t)pos * rot_half + d];
    const T s = sin[(int64_t)pos * rot_half + d];
    const T x1 = base[d], x2 = base[d + rot_half];
    using A = RnArith<T>;
    base[d] = A::add(A::mul(x1, c), A::mul(A::neg(x2), s));
    base[d + rot_half] = A::add(A::mul(x2, c), A::mul(x1, s));
}

template <typename T, typename T2>
static int launch_rope(void* q, void* k, const int32_t* positions, const void* cos, const void* sin,
                       int64_t n_tokens, int hq, int hk, int head_dim, int rot_half, int64_t max_pos,
                       int32_t* err_flag, cudaStream_t stream) {
    constexpr bool kVec = sizeof(T) == 2;
    const bool aligned = ((uintptr_t)q % 16 == 0) && (k == nullptr || (uintptr_t)k % 16 == 0) &&
                         ((uintptr_t)cos % 16 == 0) && ((uintptr_t)sin % 16 == 0);
    if (kVec && rot_half % 8 == 0 && head_dim % 8 == 0 && aligned) {
        if constexpr (kVec) {
            const int cph = rot_half / 8;
            if (n_tokens > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
            rope_token_kernel<T2><<<(unsigned)n_tokens, 256, 0, stream>>>(
                (uint4*)q, (uint4*)k, positions, (const uint4*)cos, (const uint4*)sin, hq, hk, head_dim / 8, cph,
                max_pos, err_flag);
        }
    } else {
        const int64_t n_items = n_tokens * (int64_t)(hq + hk) * rot_half;
        const int64_t blocks = (n_items + 255) / 256;
        if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
        rope_scalar_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
            (T*)q, (T*)k, positions, (const T*)cos, (const T*)sin, n_items, hq, hk, head_dim, rot_half, max_pos,
            err_flag);
    }
    return (int)cudaGetLastError();
}

}  // namespace attn

extern "C" int attn_b200_rope_inplace(void* q, void* k, const int32_t* positions, const void* cos,
                                      const void* sin, int64_t n_tokens, int n_heads_q, int n_heads_k,
                                      int head_dim, int rot_half, int64_t max_pos, int dtype, int32_t* err_flag,
                                      void* stream) {
    if (n_tokens == 0) return 0;
    if (!q || !positions || !cos || !sin || n_tokens < 0 || n_heads_q <= 0 || head_dim <= 0 || rot_half <= 0 ||
        max_pos <= 0)
        return ATTN_B200_EINVAL;
    if (2 * rot_half > head_dim) return ATTN_B200_ESHAPE;
    if (!k) n_heads_k = 0;
    if (n_heads_k < 0) return ATTN_B200_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case ATTN_B200_F16:
            return attn::launch_rope<__half, __half2>(q, k, positions, cos, sin, n_tokens, n_heads_q, n_heads_k,
                                                      head_dim, rot_half, max_pos, err_flag, st);
        case ATTN_B200_BF16:
            return attn::launch_rope<__nv_bfloat16, __nv_bfloat162>(q, k, positions, cos, sin, n_tokens, n_heads_q,
                                                                    n_heads_k, head_dim, rot_half, max_pos,
                                                                    err_flag, st);
        case ATTN_B200_F32:
            return attn::launch_rope<float, float2>(q, k, positions, cos, sin, n_tokens, n_heads_q, n_heads_k,
                                                    head_dim, rot_half, max_pos, err_flag, st);
        default:
            return ATTN_B200_EDTYPE;
    }
}
