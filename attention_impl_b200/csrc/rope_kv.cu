// Rotary embedding fused with the KV-cache append: rotate q and k in place (same arithmetic as
// rope.cu) and, in the same pass, store the rotated k and the untouched v of every token into the
// K/V pools at the token's slot, optionally quantised to e4m3 with per-head scales.
//
// The reference leaves the append to its caller: its decode operator takes the current token's
// k and v as separate arguments (paged_attention_kernel.cu:137-146,179-185) and nothing in it
// writes the pools.  This kernel is that missing step; it defines the on-device format the decode
// kernels read ([slots, H*D] rows, block_size = 1).
//
// One thread = one 16-byte chunk (8 elements).  Rotated dims are handled as (chunk, partner chunk)
// pairs by a single thread so that both are read before either is written; dims beyond the
// rotary width of k, and all of v, are plain copies into the pool.
#include "common.cuh"

namespace attn {

template <typename T2> struct Rn2;
template <> struct Rn2<__half2> {
    static __device__ __forceinline__ __half2 mul(__half2 a, __half2 b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ __half2 add(__half2 a, __half2 b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ __half2 neg(__half2 a) { return __hneg2(a); }
    static __device__ __forceinline__ float2 f2(__half2 a) { return __half22float2(a); }
};
template <> struct Rn2<__nv_bfloat162> {
    static __device__ __forceinline__ __nv_bfloat162 mul(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat162 add(__nv_bfloat162 a, __nv_bfloat162 b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ __nv_bfloat162 neg(__nv_bfloat162 a) { return __hneg2(a); }
    static __device__ __forceinline__ float2 f2(__nv_bfloat162 a) { return __bfloat1622float2(a); }
};

// 8 elements -> 8 e4m3 bytes, x * inv_scale rounded to nearest even, saturating at +-448
template <typename T2>
__device__ __forceinline__ uint2 quant8(const uint4& x, float inv_scale) {
    const T2* h = reinterpret_cast<const T2*>(&x);
    uint32_t out[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        const float2 a = Rn2<T2>::f2(h[2 * w]), b = Rn2<T2>::f2(h[2 * w + 1]);
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(a.y * inv_scale), "f"(a.x * inv_scale));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(b.y * inv_scale), "f"(b.x * inv_scale));
        out[w] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    return make_uint2(out[0], out[1]);
}

struct RopeKvParams {
    uint4* q;
    uint4* k;
    const uint4* v;
    const int32_t* positions;
    const int32_t* slots;
    const uint4* cos;
    const uint4* sin;
    void* k_cache;
    void* v_cache;
    const float* k_scale;
    const float* v_scale;
    int64_t n_items, n_slots, max_pos;
    int hq, hk, head_vec, cph;      // head_dim/8, rot_half/8
    int items_per_token;
    int quant;
    int32_t* err_flag;
};

// One CTA per token: position and slot are read once, all index arithmetic is 32-bit, and a thread
// walks several items of the token (its v chunks are loaded before anything is stored, so they are
// in flight while q and k are rotated).  The first form gave every 16-byte chunk of the whole batch
// its own thread (one 64-bit division and one or two loads per thread, threads too short-lived to
// keep the SMs full): 4.7 TB/s against this one's figure in the measurement table.
template <typename T2>
__global__ void __launch_bounds__(256)
rope_write_kv_kernel(const RopeKvParams p) {
    using A = Rn2<T2>;
    // A kernel launched behind this one as a programmatic dependent (the decode's partial kernel)
    // may be scheduled from here on; it reads nothing this kernel writes before its own wait.
    asm volatile("griddepcontrol.launch_dependents;");
    const int64_t token = blockIdx.x;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int cph = p.cph, hv = p.head_vec;
    const int pass_k = hv - 2 * cph;                     // pass-through chunks of a k head

    const int64_t slot = p.slots[token];
    const bool slot_ok = slot >= 0 && slot < p.n_slots;
    if (!slot_ok && p.err_flag && tid == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
    const int pos = p.positions[token];
    const bool pos_ok = pos >= 0 && pos < p.max_pos;
    if (!pos_ok && p.err_flag && tid == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_POSITION);

    uint4* qrow = p.q + token * p.hq * hv;
    uint4* krow = p.k + token * p.hk * hv;
    const uint4* vrow = p.v + token * p.hk * hv;
    // A token with a bad position is left alone altogether (q and k unrotated, nothing appended): a
    // pool row holding the new v beside a stale or unrotated k would be worse than a missing row.
    // A token with a good position and a bad slot is rotated in place and not appended.
    if (!pos_ok) return;
    auto store_cache = [&](void* cache, const float* scale, int head, int vec_in_row, const uint4& val) {
        if (!slot_ok) return;
        const int64_t vec = slot * p.hk * hv + vec_in_row;          // in 8-element units
        if (p.quant) reinterpret_cast<uint2*>(cache)[vec] = quant8<T2>(val, 1.f / scale[head]);
        else reinterpret_cast<uint4*>(cache)[vec] = val;
    };

    // ---- v: plain copy into the pool; up to four chunks per thread and pass, loaded first
    const int v_items = p.hk * hv;
    for (int r0 = tid; r0 < v_items; r0 += 4 * nthr) {
        uint4 vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + i * nthr;
            if (r < v_items) vv[i] = ldg_stream128(vrow + r);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + i * nthr;
            if (r < v_items) store_cache(p.v_cache, p.v_scale, r / hv, r, vv[i]);
        }
    }
    // ---- k dims beyond the rotary width: copies
    for (int r = tid; r < p.hk * pass_k; r += nthr) {
        const int head = r / pass_k, chunk = 2 * cph + (r - head * pass_k);
        store_cache(p.k_cache, p.k_scale, head, head * hv + chunk, krow[head * hv + chunk]);
    }
    // ---- rotated dims of q and k: a thread owns a chunk and its partner chunk (both read before either is written)
    const uint4* cosr = p.cos + (int64_t)pos * cph;
    const uint4* sinr = p.sin + (int64_t)pos * cph;
    const int q_items = p.hq * cph, qk_items = q_items + p.hk * cph;
    for (int r = tid; r < qk_items; r += nthr) {
        const bool is_q = r < q_items;
        const int rr = is_q ? r : r - q_items;
        const int head = rr / cph, c = rr - head * cph;
        uint4* base = (is_q ? qrow : krow) + head * hv;
        uint4 x1 = base[c], x2 = base[c + cph];
        const uint4 cs = __ldg(cosr + c), sn = __ldg(sinr + c);
        T2* a = reinterpret_cast<T2*>(&x1);
        T2* b2 = reinterpret_cast<T2*>(&x2);
        const T2* cc = reinterpret_cast<const T2*>(&cs);
        const T2* ss = reinterpret_cast<const T2*>(&sn);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const T2 lo = A::add(A::mul(a[i], cc[i]), A::mul(A::neg(b2[i]), ss[i]));
            const T2 hi = A::add(A::mul(b2[i], cc[i]), A::mul(a[i], ss[i]));
            a[i] = lo;
            b2[i] = hi;
        }
        base[c] = x1;
        base[c + cph] = x2;
        if (!is_q) {
            store_cache(p.k_cache, p.k_scale, head, head * hv + c, x1);
            store_cache(p.k_cache, p.k_scale, head, head * hv + c + cph, x2);
        }
    }
}

}  // namespace attn

using namespace attn;

extern "C" int attn_b200_rope_write_kv(void* q, void* k, const void* v, const int32_t* positions, const void* cos,
                                       const void* sin, const int32_t* slots, void* k_cache, void* v_cache,
                                       int64_t n_tokens, int n_heads_q, int n_heads_k, int head_dim, int rot_half,
                                       int64_t max_pos, int64_t n_slots, int dtype, int kv_dtype,
                                       const float* k_scale, const float* v_scale, int32_t* err_flag,
                                       void* stream) {
    if (n_tokens == 0) return 0;
    if (!q || !k || !v || !positions || !cos || !sin || !slots || !k_cache || !v_cache || n_tokens < 0 ||
        n_heads_q <= 0 || n_heads_k <= 0 || head_dim <= 0 || rot_half <= 0 || max_pos <= 0 || n_slots <= 0)
        return ATTN_B200_EINVAL;
    if (2 * rot_half > head_dim || rot_half % 8 || head_dim % 8) return ATTN_B200_ESHAPE;
    if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return ATTN_B200_EDTYPE;
    const bool quant = kv_dtype == ATTN_B200_E4M3;
    if (!quant && kv_dtype != dtype) return ATTN_B200_EDTYPE;
    if (quant && (!k_scale || !v_scale)) return ATTN_B200_EINVAL;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)cos | (uintptr_t)sin | (uintptr_t)k_cache |
         (uintptr_t)v_cache) % 16)
        return ATTN_B200_EINVAL;
    RopeKvParams p;
    p.q = (uint4*)q; p.k = (uint4*)k; p.v = (const uint4*)v;
    p.positions = positions; p.slots = slots; p.cos = (const uint4*)cos; p.sin = (const uint4*)sin;
    p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale;
    p.n_slots = n_slots; p.max_pos = max_pos;
    p.hq = n_heads_q; p.hk = n_heads_k; p.head_vec = head_dim / 8; p.cph = rot_half / 8;
    p.items_per_token = n_heads_q * p.cph + n_heads_k * (p.cph + p.head_vec - 2 * p.cph) + n_heads_k * p.head_vec;
    p.n_items = n_tokens * p.items_per_token;
    p.quant = quant; p.err_flag = err_flag;
    const int64_t blocks = n_tokens;                     // one CTA per token
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    if (dtype == ATTN_B200_F16) rope_write_kv_kernel<__half2><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    else rope_write_kv_kernel<__nv_bfloat162><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
}
