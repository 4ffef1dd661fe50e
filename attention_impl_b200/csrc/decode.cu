// KV-paged single-query decode for sm_100a: split-KV partial kernels + log-sum-exp combine.
//
// Semantics (paged_attention_kernel.cu:100-187 of the reference, with a correct softmax): for
// sequence b with cached tokens t in [beg_b, end_b) living in rows slots[t] of the K/V pools, and
// head h:  s_t = scale*<q, K[slots[t], h]>,  s_new = scale*<q, k_new>,  p = softmax(s_0..s_n, s_new),
// out = sum p_t V[slots[t], h] + p_new v_new.
//
// Work decomposition.  The concatenated token stream is cut by a global grid of `chunk` tokens; a
// work unit is the intersection of one grid cell with one sequence, numbered  u = cell + b.  That
// numbering is strictly increasing in (b, cell), needs no host knowledge of the lengths (so no
// device->host sync, unlike the reference launcher's per-sequence .item() loop) and has at most
// n_tokens/chunk + B + 1 ids; ids that correspond to no unit exit at once.  A CTA resolves its
// unit with a binary search over the offsets staged in shared memory.
//
// Fast kernel (16-bit q; 16-bit or e4m3 KV; D in {64,128,256}): one warp per (unit, head), the
// warps of a CTA covering adjacent heads of the SAME tokens so that a CTA streams `warps*D`
// contiguous elements per token.  Each 16-byte slice of a row is owned by one lane; a warp-wide
// 128-bit load fetches 32/LPR rows, and U such loads for K plus U for V are issued back to back
// before any arithmetic (2*U*512 B in flight per warp).  The slot table is read once per tile by
// the warp (coalesced) and broadcast by shuffle; the next tile's slots are prefetched.  Scores are
// reduced over the LPR lanes of a row by xor shuffles, the online-softmax state (m, l, o) is kept
// in the log2 domain in registers.  Each warp writes one partial row [o[D], m, l].
//
// Generic kernel (any dtype / head_dim): one CTA per (unit, head); small-shape compatibility path.
#include "common.cuh"

namespace attn {

constexpr int kMaxStagedB = 2048;

struct DecodeParams {
    const void* q;
    const void* k_cache;
    const void* v_cache;
    const int32_t* slots;
    const int32_t* offsets;
    float* part;  // [n_units, H, D + 2]
    double* S;
    int64_t sp_stride;
    int B, H, D;
    int64_t n_tokens, n_slots;
    int uniform_ctx;
    int chunk;
    float scale_log2;  // scale * log2(e)
    const float* k_scale;
    const float* v_scale;
    int32_t* err_flag;
    int head_groups;
    int Hkv;          // KV heads; H (query heads) = Hkv * G
    int G;            // query heads per KV head
    int block_size;   // tokens per KV block; 1 = `slots` is a per-token table
    int max_blocks;   // block_size > 1: `slots` is a [B, max_blocks] block table
    int tables_ready; // `slots` and `offsets` were complete before the kernel preceding this launch started
};

// Pool row of token `t` (absolute index in the token stream) of the unit's sequence, or -1.
__device__ __forceinline__ int token_slot(const DecodeParams& p, const struct Unit& un, int64_t t);

struct Unit {
    int b;
    int64_t seq_beg, tbeg, tend;
};

// beg(b) for b in [0, B]: start of sequence b in the token stream (beg(B) = total).
struct SeqBounds {
    const int32_t* off;  // global or shared copy; nullptr => uniform
    int64_t uniform_ctx;
    int64_t n_tokens;
    __device__ __forceinline__ int64_t beg(int b) const {
        if (!off) return (int64_t)b * uniform_ctx;
        if (b == 0) return 0;
        int64_t v = off[b - 1];
        return v < 0 ? 0 : (v > n_tokens ? n_tokens : v);
    }
};

__device__ __forceinline__ int token_slot(const DecodeParams& p, const Unit& un, int64_t t) {
    int64_t v;
    if (!p.slots) {
        v = t;
    } else if (p.block_size <= 1) {
        v = p.slots[t];
    } else {
        const int64_t rel = t - un.seq_beg;
        const int64_t blk = rel / p.block_size;
        if (blk >= p.max_blocks) v = -1;
        else {
            const int64_t id = p.slots[(int64_t)un.b * p.max_blocks + blk];
            v = id < 0 ? -1 : id * p.block_size + (rel - blk * p.block_size);
        }
    }
    if (v >= 0 && v < p.n_slots) return (int)v;
    if (p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
    return -1;
}

__device__ __forceinline__ bool resolve_unit(int64_t u, int B, int chunk, const SeqBounds& sb, Unit& out) {
    int lo = 0, hi = B - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (sb.beg(mid) / chunk + mid <= u) lo = mid; else hi = mid - 1;
    }
    const int64_t seq_beg = sb.beg(lo), seq_end = sb.beg(lo + 1);
    const int64_t cell = u - lo;
    const int64_t tb = cell * chunk, te = tb + chunk;
    out.b = lo;
    out.seq_beg = seq_beg;
    out.tbeg = tb > seq_beg ? tb : seq_beg;
    out.tend = te < seq_end ? te : seq_end;
    return out.tbeg < out.tend;
}

__device__ __forceinline__ const int32_t* stage_offsets(const DecodeParams& p, int32_t* s_off) {
    if (!p.offsets) return nullptr;
    if (p.B > kMaxStagedB) return p.offsets;
    for (int i = threadIdx.x; i < p.B; i += blockDim.x) s_off[i] = p.offsets[i];
    __syncthreads();
    return s_off;
}

// ---------------------------------------------------------------------------------------------
// fast kernel
// ---------------------------------------------------------------------------------------------
template <typename KVT, int EPL> struct RowChunk;  // 16 bytes of a KV row -> EPL floats
template <> struct RowChunk<__half, 8> {
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        unpack2(r.x, __half(), f[0], f[1]); unpack2(r.y, __half(), f[2], f[3]);
        unpack2(r.z, __half(), f[4], f[5]); unpack2(r.w, __half(), f[6], f[7]);
    }
};
template <> struct RowChunk<__nv_bfloat16, 8> {
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        unpack2(r.x, __nv_bfloat16(), f[0], f[1]); unpack2(r.y, __nv_bfloat16(), f[2], f[3]);
        unpack2(r.z, __nv_bfloat16(), f[4], f[5]); unpack2(r.w, __nv_bfloat16(), f[6], f[7]);
    }
};
template <> struct RowChunk<__nv_fp8_e4m3, 16> {
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        unpack4_e4m3(r.x, f[0], f[1], f[2], f[3]); unpack4_e4m3(r.y, f[4], f[5], f[6], f[7]);
        unpack4_e4m3(r.z, f[8], f[9], f[10], f[11]); unpack4_e4m3(r.w, f[12], f[13], f[14], f[15]);
    }
};

// Multi-head attention with a per-token slot table (the reference's case and the benchmarked one).
// The general kernel below (grouped-query heads, block tables) computes the same thing with G = 1,
// block_size = 1, but measured 7 % slower on this path (6.40 vs 6.91 TB/s on a 15 GB fp16 case), so
// the specialised form is kept.
// The 32/LPR row groups of a warp take adjacent HEADS of one token, so a warp-wide load is one
// contiguous 512-byte piece of a token's row and a CTA of 8 warps streams 4 KB per token; each
// group keeps its own softmax state and nothing is merged across groups.  A tile is 8 tokens; its
// 8 K-row and 8 V-row loads are issued, then consumed.  With many CTAs per SM in different phases
// the memory pipe stays full: this is the form for long units (large batches, long contexts).
//
// The grid is launched as a programmatic dependent of whatever kernel precedes it on the stream: if
// that kernel releases its dependents early (the combine of the previous decode step and the RoPE /
// cache-append kernel do), this grid's launch latency is spent while it still runs.  Nothing the
// preceding kernel may have written is read before griddepcontrol.wait.  EARLY = true (the caller
// vouches that the slot table and the offsets were complete before the preceding kernel STARTED:
// they came from an upload, not from that kernel) also finds the CTA's unit and fetches its first
// slots before the wait, so that two of the prologue's three dependent round trips overlap the
// preceding kernel's tail.  This grid releases its own dependent (the combine kernel, which reads the
// step's inputs before its own wait) only after its wait: those inputs are complete by then.
template <typename QT, typename KVT, int D, bool EARLY>
__global__ void __launch_bounds__(256)
paged_decode_mha_kernel(const DecodeParams p) {
    constexpr int EPL = 16 / (int)sizeof(KVT);   // elements per lane (one 16-byte slice)
    constexpr int LPR = D / EPL;                 // lanes per row
    constexpr int TPI = 32 / LPR;                // rows per warp-wide load
    constexpr int U = 8;                         // loads in flight per lane and tensor = tokens per tile
    constexpr int TILE = U;
    constexpr int HPW = TPI;                     // heads per warp
    static_assert(LPR >= 1 && LPR <= 32 && TILE <= 32, "unsupported head_dim");

    __shared__ int32_t s_off[kMaxStagedB];
    if constexpr (!EARLY) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;");
    }
    SeqBounds sb{stage_offsets(p, s_off), p.uniform_ctx, p.n_tokens};

    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t u = blockIdx.x / p.head_groups;
    const int sub = lane % LPR, grp = lane / LPR;
    const int h_raw = ((blockIdx.x % p.head_groups) * warps + warp) * HPW + grp;
    Unit un;
    if (!resolve_unit(u, p.B, p.chunk, sb, un) || h_raw - grp >= p.H) {
        // (a CTA without work still takes part in the grid dependency: if every CTA left without waiting,
        // this grid would count as complete, and release its dependent, before its predecessor is)
        if constexpr (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }
    int early_slot = -1;
    if constexpr (EARLY) {
        const int64_t t = un.tbeg + lane;
        if (lane < TILE && t < un.tend) {
            const int64_t v = p.slots ? (int64_t)p.slots[t] : t;
            if (v >= 0 && v < p.n_slots) early_slot = (int)v;
            else if (p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;");
    }
    const bool h_ok = h_raw < p.H;               // trailing groups of the last warp may have no head
    const int h = h_ok ? h_raw : p.H - 1;
    const int64_t row_bytes = (int64_t)p.H * D * sizeof(KVT);
    const char* kbase = (const char*)p.k_cache + ((int64_t)h * D + sub * EPL) * sizeof(KVT);
    const char* vbase = (const char*)p.v_cache + ((int64_t)h * D + sub * EPL) * sizeof(KVT);

    // 16-bit KV: q in fp32, pre-multiplied by scale*log2(e).  e4m3 KV: q stays unscaled in packed
    // fp16 (products with the 4-significant-bit e4m3 values are formed by HFMA2 and the 16
    // products of a lane are summed in fp16 before widening: the error, ~1e-3 of a score's
    // standard deviation, is far below the e4m3 quantisation it rides on); the combined factor
    // scale*log2(e)*k_scale[h] is applied to the reduced fp32 score.
    constexpr bool kFp8 = sizeof(KVT) == 1;
    float qf[kFp8 ? 1 : EPL];
    __half2 q2[kFp8 ? EPL / 2 : 1];
    float qs = p.scale_log2 * (p.k_scale ? p.k_scale[h] : 1.f);
    {
        const QT* qp = (const QT*)p.q + ((int64_t)un.b * p.H + h) * D + sub * EPL;
        if constexpr (kFp8) {
#pragma unroll
            for (int i = 0; i < EPL / 2; ++i) q2[i] = __floats2half2_rn(to_f32<QT>(qp[2 * i]), to_f32<QT>(qp[2 * i + 1]));
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) qf[i] = to_f32<QT>(qp[i]) * qs;
        }
    }
    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.f;

    auto load_slot = [&](int64_t t0) -> int {
        const int64_t t = t0 + lane;
        int s = -1;
        if (lane < TILE && t < un.tend) {
            const int64_t v = p.slots ? (int64_t)p.slots[t] : t;
            if (v >= 0 && v < p.n_slots) s = (int)v;
            else if (p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
        }
        return s;
    };

    int next_slot;
    if constexpr (EARLY) next_slot = early_slot;
    else next_slot = load_slot(un.tbeg);
    for (int64_t t0 = un.tbeg; t0 < un.tend; t0 += TILE) {
        const int my_slot = next_slot;
        uint4 kr[U], vr[U];
        int sl[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            sl[j] = __shfl_sync(0xffffffffu, my_slot, j);
            if (sl[j] >= 0) {
                kr[j] = ldg_stream128(kbase + (int64_t)sl[j] * row_bytes);
            } else {
                kr[j] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (sl[j] >= 0) {
                vr[j] = ldg_stream128(vbase + (int64_t)sl[j] * row_bytes);
            } else {
                vr[j] = make_uint4(0, 0, 0, 0);
            }
        }
        if (t0 + TILE < un.tend) next_slot = load_slot(t0 + TILE);

        float s[U];
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            float acc = 0.f;
            if constexpr (kFp8) {
                const uint32_t w4[4] = {kr[j].x, kr[j].y, kr[j].z, kr[j].w};
                __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __half2 lo, hi;
                    e4m3x4_to_half2x2(w4[i], lo, hi);
                    a0 = __hfma2(q2[2 * i], lo, a0);
                    a1 = __hfma2(q2[2 * i + 1], hi, a1);
                }
                const float2 f = __half22float2(__hadd2(a0, a1));
                acc = group_sum<LPR>(f.x + f.y) * qs;
            } else {
                float kf[EPL];
                RowChunk<KVT, EPL>::unpack(kr[j], kf);
#pragma unroll
                for (int i = 0; i < EPL; ++i) acc = fmaf(qf[i], kf[i], acc);
                acc = group_sum<LPR>(acc);
            }
            s[j] = sl[j] >= 0 ? acc : -INFINITY;
            tmax = fmaxf(tmax, s[j]);
        }
        if (p.S) {
            if (sub == 0) {
#pragma unroll
                for (int j = 0; j < U; ++j)
                    if (sl[j] >= 0)
                        if (h_ok)
                            p.S[((int64_t)un.b * p.H + h) * p.sp_stride + (t0 + j - un.seq_beg)] =
                                (double)(s[j] * kLn2);
            }
        }
        const float m_new = fmaxf(m, tmax);
        if (m_new > -INFINITY) {  // at least one valid row so far
            const float alpha = fast_exp2(m - m_new);
            l *= alpha;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[i] *= alpha;
            if constexpr (kFp8) {
                // p*v summed over the tile's U rows in fp16x2 (p <= 1, |v| <= 448), widened once per tile
                __half2 oa[EPL / 2];
#pragma unroll
                for (int i = 0; i < EPL / 2; ++i) oa[i] = __float2half2_rn(0.f);
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const float pj = fast_exp2(s[j] - m_new);
                    l += pj;
                    const __half2 p2 = __float2half2_rn(pj);
                    const uint32_t w4[4] = {vr[j].x, vr[j].y, vr[j].z, vr[j].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 lo, hi;
                        e4m3x4_to_half2x2(w4[i], lo, hi);
                        oa[2 * i] = __hfma2(p2, lo, oa[2 * i]);
                        oa[2 * i + 1] = __hfma2(p2, hi, oa[2 * i + 1]);
                    }
                }
#pragma unroll
                for (int i = 0; i < EPL / 2; ++i) {
                    const float2 f = __half22float2(oa[i]);
                    o[2 * i] += f.x;
                    o[2 * i + 1] += f.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const float pj = fast_exp2(s[j] - m_new);
                    l += pj;
                    float vf[EPL];
                    RowChunk<KVT, EPL>::unpack(vr[j], vf);
#pragma unroll
                    for (int i = 0; i < EPL; ++i) o[i] = fmaf(pj, vf[i], o[i]);
                }
            }
            m = m_new;
        }
    }
    float* row = p.part + ((int64_t)u * p.H + h) * (D + 2);
    if (h_ok) {
        const float vs = p.v_scale ? p.v_scale[h] : 1.f;
        float2* dst = reinterpret_cast<float2*>(row + sub * EPL);
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) dst[i] = make_float2(o[2 * i] * vs, o[2 * i + 1] * vs);
        if (sub == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m, l);
    }
}


// The 32/LPR row groups of a warp take ADJACENT KV HEADS of one token, so a warp-wide load is one
// contiguous 512-byte piece of the token's row and a CTA of 8 warps streams 4 KB per token; each
// group keeps its own softmax state.  G > 1 (grouped-query attention): the G query heads that share
// a KV head are all served from the one copy of the row held in registers.
template <typename QT, typename KVT, int D, int G>
// CTAs per SM.  G = 1, 2 and (16-bit KV) 4: two CTAs of 128 registers (16 warps per SM): the
// kernel needs the loads of many warps in flight more than it needs the registers (measured at
// G = 2: 3.66 -> 5.34 TB/s, at G = 4: 2.29 -> 3.25; the e4m3 form of G = 4 spills too much at 128
// and G = 8 needs all 255).  Packed fp16 arithmetic for fp16 rows was also measured (G = 4: 3.62):
// not worth the fp16 sums; groups this large want the rows multiplied on the tensor cores.
__global__ void __launch_bounds__(256, (G <= 2 || (G == 4 && sizeof(KVT) == 2)) ? 2 : 1)
paged_decode_fast_kernel(const DecodeParams p) {
    constexpr int EPL = 16 / (int)sizeof(KVT);   // elements per lane (one 16-byte slice)
    constexpr int LPR = D / EPL;                 // lanes per row
    constexpr int HPW = 32 / LPR;                // KV heads per warp
    constexpr int U = G >= 8 ? 2 : (G >= 4 ? 4 : 8);   // row loads in flight per lane and tensor = tokens per tile
    constexpr bool kFp8 = sizeof(KVT) == 1;
    static_assert(LPR >= 1 && LPR <= 32, "unsupported head_dim");

    __shared__ int32_t s_off[kMaxStagedB];
    SeqBounds sb{stage_offsets(p, s_off), p.uniform_ctx, p.n_tokens};

    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t u = blockIdx.x / p.head_groups;
    const int sub = lane % LPR, grp = lane / LPR;
    const int hk_raw = ((blockIdx.x % p.head_groups) * warps + warp) * HPW + grp;
    Unit un;
    if (!resolve_unit(u, p.B, p.chunk, sb, un) || hk_raw - grp >= p.Hkv) return;
    const bool h_ok = hk_raw < p.Hkv;            // trailing groups of the last warp may have no head
    const int hk = h_ok ? hk_raw : p.Hkv - 1;
    const int64_t row_bytes = (int64_t)p.Hkv * D * sizeof(KVT);
    const char* kbase = (const char*)p.k_cache + ((int64_t)hk * D + sub * EPL) * sizeof(KVT);
    const char* vbase = (const char*)p.v_cache + ((int64_t)hk * D + sub * EPL) * sizeof(KVT);

    // 16-bit KV: q in fp32, pre-multiplied by scale*log2(e).  e4m3 KV: q stays unscaled in packed
    // fp16 (products with the 4-significant-bit e4m3 values are formed by HFMA2 and the 16
    // products of a lane are summed in fp16 before widening: the error, ~1e-3 of a score's
    // standard deviation, is far below the e4m3 quantisation it rides on); the combined factor
    // scale*log2(e)*k_scale[hk] is applied to the reduced fp32 score.
    float qf[G][kFp8 ? 1 : EPL];
    __half2 q2[G][kFp8 ? EPL / 2 : 1];
    const float qs = p.scale_log2 * (p.k_scale ? p.k_scale[hk] : 1.f);
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const QT* qp = (const QT*)p.q + ((int64_t)un.b * p.H + hk * G + gi) * D + sub * EPL;
        if constexpr (kFp8) {
#pragma unroll
            for (int i = 0; i < EPL / 2; ++i)
                q2[gi][i] = __floats2half2_rn(to_f32<QT>(qp[2 * i]), to_f32<QT>(qp[2 * i + 1]));
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) qf[gi][i] = to_f32<QT>(qp[i]) * qs;
        }
    }
    float m[G], l[G], o[G][EPL];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        m[gi] = -INFINITY;
        l[gi] = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[gi][i] = 0.f;
    }

    auto load_slot = [&](int64_t t0) -> int {
        const int64_t t = t0 + lane;
        return (lane < U && t < un.tend) ? token_slot(p, un, t) : -1;
    };

    int next_slot = load_slot(un.tbeg);
    for (int64_t t0 = un.tbeg; t0 < un.tend; t0 += U) {
        const int my_slot = next_slot;
        uint4 kr[U], vr[U];
        int sl[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            sl[j] = __shfl_sync(0xffffffffu, my_slot, j);
            kr[j] = sl[j] >= 0 ? ldg_stream128(kbase + (int64_t)sl[j] * row_bytes) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < U; ++j)
            vr[j] = sl[j] >= 0 ? ldg_stream128(vbase + (int64_t)sl[j] * row_bytes) : make_uint4(0, 0, 0, 0);
        if (t0 + U < un.tend) next_slot = load_slot(t0 + U);

        float s[G][U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if constexpr (kFp8) {
                const uint32_t w4[4] = {kr[j].x, kr[j].y, kr[j].z, kr[j].w};
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 lo, hi;
                        e4m3x4_to_half2x2(w4[i], lo, hi);    // 2 conversions: cheaper to redo per query head than to hold
                        a0 = __hfma2(q2[gi][2 * i], lo, a0);
                        a1 = __hfma2(q2[gi][2 * i + 1], hi, a1);
                    }
                    const float2 f = __half22float2(__hadd2(a0, a1));
                    const float acc = group_sum<LPR>(f.x + f.y) * qs;
                    s[gi][j] = sl[j] >= 0 ? acc : -INFINITY;
                }
            } else {
                float kf[EPL];
                RowChunk<KVT, EPL>::unpack(kr[j], kf);
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    float acc = 0.f;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) acc = fmaf(qf[gi][i], kf[i], acc);
                    acc = group_sum<LPR>(acc);
                    s[gi][j] = sl[j] >= 0 ? acc : -INFINITY;
                }
            }
        }
        if (p.S && sub == 0 && h_ok) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi)
#pragma unroll
                for (int j = 0; j < U; ++j)
                    if (sl[j] >= 0)
                        p.S[((int64_t)un.b * p.H + hk * G + gi) * p.sp_stride + (t0 + j - un.seq_beg)] =
                            (double)(s[gi][j] * kLn2);
        }
        float msub[G];      // maximum to subtract (0 while a head has seen no valid row: exp2(-inf - 0) = 0)
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            float tmax = s[gi][0];
#pragma unroll
            for (int j = 1; j < U; ++j) tmax = fmaxf(tmax, s[gi][j]);
            const float m_new = fmaxf(m[gi], tmax);
            const bool live = m_new > -INFINITY;
            const float alpha = live ? fast_exp2(m[gi] - m_new) : 1.f;
            l[gi] *= alpha;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[gi][i] *= alpha;
            m[gi] = m_new;
            msub[gi] = live ? m_new : 0.f;
        }
        if constexpr (kFp8) {
            // p*v summed over the tile's rows in fp16x2 (p <= 1, |v| <= 448), widened once per tile
            __half2 oa[G][EPL / 2];
#pragma unroll
            for (int gi = 0; gi < G; ++gi)
#pragma unroll
                for (int i = 0; i < EPL / 2; ++i) oa[gi][i] = __float2half2_rn(0.f);
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const uint32_t w4[4] = {vr[j].x, vr[j].y, vr[j].z, vr[j].w};
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const float pj = fast_exp2(s[gi][j] - msub[gi]);
                    l[gi] += pj;
                    const __half2 p2 = __float2half2_rn(pj);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 lo, hi;
                        e4m3x4_to_half2x2(w4[i], lo, hi);
                        oa[gi][2 * i] = __hfma2(p2, lo, oa[gi][2 * i]);
                        oa[gi][2 * i + 1] = __hfma2(p2, hi, oa[gi][2 * i + 1]);
                    }
                }
            }
#pragma unroll
            for (int gi = 0; gi < G; ++gi)
#pragma unroll
                for (int i = 0; i < EPL / 2; ++i) {
                    const float2 f = __half22float2(oa[gi][i]);
                    o[gi][2 * i] += f.x;
                    o[gi][2 * i + 1] += f.y;
                }
        } else {
#pragma unroll
            for (int j = 0; j < U; ++j) {
                float vf[EPL];
                RowChunk<KVT, EPL>::unpack(vr[j], vf);
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const float pj = fast_exp2(s[gi][j] - msub[gi]);
                    l[gi] += pj;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) o[gi][i] = fmaf(pj, vf[i], o[gi][i]);
                }
            }
        }
    }
    if (!h_ok) return;
    const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        float* row = p.part + ((int64_t)u * p.H + hk * G + gi) * (D + 2);
        float2* dst = reinterpret_cast<float2*>(row + sub * EPL);
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) dst[i] = make_float2(o[gi][2 * i] * vs, o[gi][2 * i + 1] * vs);
        if (sub == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m[gi], l[gi]);
    }
}

// ---------------------------------------------------------------------------------------------
// whole-sequence kernel: one CTA per (sequence, head), combine in shared memory, ONE launch
// ---------------------------------------------------------------------------------------------
// For batches whose (sequence, head) pairs alone fill the machine and whose sequences are short
// (batch 8 x 32 heads x <= 1024 tokens: 256 CTAs).  The split-KV form spends a third of such a step
// on its second launch and on the partial rows' round trip through L2; here the 8 warps of a CTA
// split the sequence's tokens tile by tile (warp w takes tiles w, w + 8, ...), every warp keeps its
// (m, l, o) in registers, and the eight partial results meet in shared memory, where the current
// token is folded in and the output row is written.  No workspace, no second kernel.  The price is
// imbalance: a CTA lives as long as its sequence is long, so it is the wrong kernel for long or very
// unequal sequences (the host-side heuristic decides; attn_b200_paged_decode_single_launch_ok).
// Lane mapping: a row of D 16-bit elements is LPR = D/8 lanes of 16 bytes; a warp-wide load covers
// TPI = 32/LPR different TOKENS of the CTA's one head; U = 8 such loads for K and 8 for V are in
// flight per tile of TPI*8 tokens.
struct SeqDecodeParams {
    const void* q;
    const void* k_new;
    const void* v_new;
    const void* k_cache;
    const void* v_cache;
    const int32_t* slots;
    const int32_t* offsets;
    void* out;
    int B, H, D;
    int64_t n_tokens, n_slots;
    int uniform_ctx;
    float scale_log2;
    int32_t* err_flag;
};

template <typename QT, int D>
__global__ void __launch_bounds__(256, 2)
paged_decode_seq_kernel(const SeqDecodeParams p) {
    constexpr int EPL = 8;                       // elements per lane (one 16-byte slice of a 16-bit row)
    constexpr int LPR = D / EPL;                 // lanes per row
    constexpr int TPI = 32 / LPR;                // tokens per warp-wide load
    constexpr int U = 8;                         // loads in flight per lane and tensor
    constexpr int TILE = TPI * U;                // tokens per warp and tile
    constexpr int WARPS = 8;
    static_assert(LPR >= 1 && LPR <= 32 && TILE <= 32, "unsupported head_dim");
    __shared__ float s_o[WARPS][D];
    __shared__ float s_ml[WARPS][2];
    __shared__ float s_new_sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const int sub = lane % LPR, tsel = lane / LPR;
    SeqBounds sb{p.offsets, p.uniform_ctx, p.n_tokens};
    const int64_t seq_beg = sb.beg(b), seq_end_raw = sb.beg(b + 1);
    const int64_t seq_end = seq_end_raw > seq_beg ? seq_end_raw : seq_beg;
    const int64_t row_bytes = (int64_t)p.H * D * sizeof(QT);
    const char* kbase = (const char*)p.k_cache + ((int64_t)h * D + sub * EPL) * sizeof(QT);
    const char* vbase = (const char*)p.v_cache + ((int64_t)h * D + sub * EPL) * sizeof(QT);
    const QT* qp = (const QT*)p.q + ((int64_t)b * p.H + h) * D + sub * EPL;

    float qf[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) qf[i] = to_f32<QT>(qp[i]) * p.scale_log2;
    if (warp == 0) {                             // score of the current token (every row group computes the same)
        const QT* kp = (const QT*)p.k_new + ((int64_t)b * p.H + h) * D + sub * EPL;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc = fmaf(qf[i], to_f32<QT>(kp[i]), acc);
        acc = group_sum<LPR>(acc);
        if (lane == 0) s_new_sh = acc;
    }
    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.f;

    auto load_slot = [&](int64_t t0) -> int {    // slots of the TILE tokens from t0, one per lane
        const int64_t t = t0 + lane;
        int s = -1;
        if (lane < TILE && t < seq_end) {
            const int64_t v = p.slots ? (int64_t)p.slots[t] : t;
            if (v >= 0 && v < p.n_slots) s = (int)v;
            else if (p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
        }
        return s;
    };
    const int64_t stride = (int64_t)WARPS * TILE;
    int next_slot = seq_beg + (int64_t)warp * TILE < seq_end ? load_slot(seq_beg + (int64_t)warp * TILE) : -1;
    for (int64_t t0 = seq_beg + (int64_t)warp * TILE; t0 < seq_end; t0 += stride) {
        const int my_slot = next_slot;
        uint4 kr[U], vr[U];
        int sl[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            sl[j] = __shfl_sync(0xffffffffu, my_slot, j * TPI + tsel);
            kr[j] = sl[j] >= 0 ? ldg_stream128(kbase + (int64_t)sl[j] * row_bytes) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < U; ++j)
            vr[j] = sl[j] >= 0 ? ldg_stream128(vbase + (int64_t)sl[j] * row_bytes) : make_uint4(0, 0, 0, 0);
        if (t0 + stride < seq_end) next_slot = load_slot(t0 + stride);

        float s[U];
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            float kf[EPL];
            RowChunk<QT, EPL>::unpack(kr[j], kf);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc = fmaf(qf[i], kf[i], acc);
            acc = group_sum<LPR>(acc);
            s[j] = sl[j] >= 0 ? acc : -INFINITY;
            tmax = fmaxf(tmax, s[j]);
        }
        const float m_new = fmaxf(m, tmax);
        if (m_new > -INFINITY) {
            const float alpha = fast_exp2(m - m_new);
            l *= alpha;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[i] *= alpha;
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const float pj = fast_exp2(s[j] - m_new);
                l += pj;
                float vf[EPL];
                RowChunk<QT, EPL>::unpack(vr[j], vf);
#pragma unroll
                for (int i = 0; i < EPL; ++i) o[i] = fmaf(pj, vf[i], o[i]);
            }
            m = m_new;
        }
    }
    // fold the warp's TPI row groups (same head, different tokens), then the CTA's warps
#pragma unroll
    for (int x = LPR; x < 32; x <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, x);
        const float mn = fmaxf(m, mo);
        const float a = mn > -INFINITY ? fast_exp2(m - mn) : 0.f;      // this side's factor (0 if it saw nothing)
        const float bq = mn > -INFINITY ? fast_exp2(mo - mn) : 0.f;
        l = l * a + __shfl_xor_sync(0xffffffffu, l, x) * bq;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[i] = o[i] * a + __shfl_xor_sync(0xffffffffu, o[i], x) * bq;
        m = mn;
    }
    if (tsel == 0) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) s_o[warp][sub * EPL + i] = o[i];
        if (sub == 0) { s_ml[warp][0] = m; s_ml[warp][1] = l; }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float s_new = s_new_sh;
        float M = s_new;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_ml[w][0]);
        const float w_new = exp2f(s_new - M);
        float L = w_new;
        float acc = w_new * to_f32<QT>(((const QT*)p.v_new)[((int64_t)b * p.H + h) * D + d]);
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = s_ml[w][0];
            const float f = mw > -INFINITY ? exp2f(mw - M) : 0.f;
            L = fmaf(s_ml[w][1], f, L);
            acc = fmaf(s_o[w][d], f, acc);
        }
        ((QT*)p.out)[((int64_t)b * p.H + h) * D + d] = from_f32<QT>(acc / L);
    }
}

template <typename QT>
static int launch_seq(const SeqDecodeParams& p, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.B * p.H;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    switch (p.D) {
        case 64: paged_decode_seq_kernel<QT, 64><<<(unsigned)blocks, 256, 0, st>>>(p); break;
        case 128: paged_decode_seq_kernel<QT, 128><<<(unsigned)blocks, 256, 0, st>>>(p); break;
        case 256: paged_decode_seq_kernel<QT, 256><<<(unsigned)blocks, 256, 0, st>>>(p); break;
        default: return ATTN_B200_ESHAPE;
    }
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// generic kernel: any dtype / head_dim, one CTA per (unit, head)
// ---------------------------------------------------------------------------------------------
template <typename QT, typename KVT>
__global__ void __launch_bounds__(128)
paged_decode_generic_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int32_t s_off[kMaxStagedB];
    __shared__ float s_red[4];
    float* s_q = reinterpret_cast<float*>(smem_raw);       // [D]
    float* s_sc = s_q + p.D;                                // [chunk]
    int32_t* s_slot = reinterpret_cast<int32_t*>(s_sc + p.chunk);  // [chunk]

    SeqBounds sb{stage_offsets(p, s_off), p.uniform_ctx, p.n_tokens};
    const int64_t u = blockIdx.x / p.H;
    const int h = blockIdx.x % p.H;
    Unit un;
    if (!resolve_unit(u, p.B, p.chunk, sb, un)) return;
    const int n = (int)(un.tend - un.tbeg);
    const int D = p.D;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int hk = h / p.G;                               // KV head of this query head
    const float qs = p.scale_log2 * (p.k_scale ? p.k_scale[hk] : 1.f);
    for (int d = tid; d < D; d += blockDim.x)
        s_q[d] = to_f32<QT>(((const QT*)p.q)[((int64_t)un.b * p.H + h) * D + d]) * qs;
    for (int i = tid; i < n; i += blockDim.x) s_slot[i] = token_slot(p, un, un.tbeg + i);
    __syncthreads();
    float lmax = -INFINITY;
    for (int i = tid; i < n; i += blockDim.x) {
        float acc = -INFINITY;
        if (s_slot[i] >= 0) {
            const KVT* kr = (const KVT*)p.k_cache + ((int64_t)s_slot[i] * p.Hkv + hk) * D;
            acc = 0.f;
            for (int d = 0; d < D; ++d) acc = fmaf(s_q[d], to_f32<KVT>(kr[d]), acc);
            if (p.S)
                p.S[((int64_t)un.b * p.H + h) * p.sp_stride + (un.tbeg + i - un.seq_beg)] = (double)(acc * kLn2);
        }
        s_sc[i] = acc;
        lmax = fmaxf(lmax, acc);
    }
    lmax = group_max<32>(lmax);
    if (lane == 0) s_red[warp] = lmax;
    __syncthreads();
    const float m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    __syncthreads();
    float lsum = 0.f;
    for (int i = tid; i < n; i += blockDim.x) {
        const float pj = (m > -INFINITY && s_sc[i] > -INFINITY) ? exp2f(s_sc[i] - m) : 0.f;
        s_sc[i] = pj;
        lsum += pj;
    }
    lsum = group_sum<32>(lsum);
    if (lane == 0) s_red[warp] = lsum;
    __syncthreads();
    const float l = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    float* row = p.part + ((int64_t)u * p.H + h) * (D + 2);
    const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
    for (int d = tid; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < n; ++i)
            if (s_slot[i] >= 0)
                acc = fmaf(s_sc[i], to_f32<KVT>(((const KVT*)p.v_cache)[((int64_t)s_slot[i] * p.Hkv + hk) * D + d]), acc);
        row[d] = acc * vs;
    }
    if (tid == 0) { row[D] = m; row[D + 1] = l; }
}

// ---------------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------------
constexpr int kMaxXchgPeers = 16;
constexpr long long kXchgWaitCycles = 2000000000LL;     // about one second of SM clocks

struct CombineParams {
    const float* parts;   // unit partials [n_units, H, D+2]  or  gathered [n_parts, B, H, D+2]
    int n_parts;          // > 0: gathered mode; 0: unit mode (rows found from offsets/chunk)
    const void* q;
    const void* k_new;    // may be null: new token not folded
    const void* v_new;
    void* out;            // final output [B, H*D] (QT) or null
    float* part_out;      // [B, H, D+2] or null
    double* S;
    double* P;
    int64_t sp_stride;
    const int32_t* offsets;
    int64_t uniform_ctx, n_tokens;
    int B, H, D, chunk;
    float scale_log2;
    int G;                // query heads per KV head: k_new / v_new are [B, (H/G)*D]
    // KV-split exchange (XCHG instantiation only; see the kernel)
    int n_peers;                       // > 0: the partial row goes to peer_dst[g] for every g instead of part_out
    float* peer_dst[kMaxXchgPeers];    // each [B, H, D+2], already offset to this rank's slot
    int32_t* peer_flag[kMaxXchgPeers]; // arrival counter of this rank on peer g
    int32_t* wait_flags;               // non-null: wait until wait_flags[i] >= wait_count for i < n_parts ...
    int32_t wait_count;
    int32_t* done_counter;             // ... and the last CTA to get past the wait takes wait_count off them again
    int32_t* err_flag;
};

// One CTA of four warps per (b, h).  Every warp finds the global maximum and denominator (lanes over
// units, the m and l of a unit loaded together), the numerator's units are dealt to the warps
// round-robin in batches of eight per warp whose loads are all independent and are requested
// together with the (m, l) pairs, and the four partial sums meet in shared memory.  With one warp
// doing all units in turn the combine took as long as the partial kernel on small batches (16.6 us
// against 15.0 at batch 8).
//
// XCHG = true adds the two ends of the cross-GPU KV-split exchange, so that a step is three launches
// (partial kernel, this kernel pushing, this kernel waiting) instead of five:
//  * push (n_peers > 0, unit mode): the (b, h) row [o[D], m, l] is stored into every peer's gather
//    buffer with plain stores over NVLink instead of into part_out; then the CTA publishes them
//    (__threadfence_system) and adds 1 to its counter on every peer (system-scope reduction).  A
//    step adds B*H to each counter.
//  * wait (wait_flags != null, gathered mode): before reading the gathered rows, thread i < n_parts
//    polls wait_flags[i] until it has reached wait_count = B*H.  The wait is bounded (about a
//    second); when it runs out the CTA raises ATTN_B200_FLAG_TIMEOUT and carries on with whatever
//    is there, so the kernel always ends.  Every CTA then takes a ticket on done_counter; the last
//    one (all CTAs are past their wait) takes wait_count off each counter again, which leaves the
//    arrivals of a peer that is already one step ahead, and resets done_counter: every step has
//    the same arguments and can be replayed from a CUDA graph.  Peers' rows land in this GPU's own
//    memory before any CTA reads them; no multicast of any kind is involved.
template <typename QT, bool XCHG>
__global__ void __launch_bounds__(128)
lse_combine_kernel(const CombineParams p) {
    __shared__ float s_acc[4][256];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    // A kernel launched behind this one as a programmatic dependent (the partial kernel of the next
    // decode step) may be scheduled from here on; it reads nothing before its own wait.  Not in the
    // exchange instantiation: what follows a pushing combine is the waiting combine, whose CTAs would
    // sit on the SMs polling their counters while the partial kernel still runs (measured at 8 GPUs
    // from a CUDA graph: 0.994 against 0.941 ms per step).
    if constexpr (!XCHG) asm volatile("griddepcontrol.launch_dependents;");
    if constexpr (XCHG) {
        if (p.wait_flags) {
            if (threadIdx.x < p.n_parts) {
                const int32_t* f = p.wait_flags + threadIdx.x;
                const long long t0 = clock64();
                while (true) {
                    int32_t v;
                    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                    if (v - p.wait_count >= 0) break;
                    if (clock64() - t0 > kXchgWaitCycles) {
                        if (p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_TIMEOUT);
                        break;
                    }
                    __nanosleep(64);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                __threadfence();
                if (atomicAdd(p.done_counter, 1) == (int)gridDim.x - 1) {
                    for (int i = 0; i < p.n_parts; ++i) atomicSub_system(p.wait_flags + i, p.wait_count);
                    *p.done_counter = 0;
                }
            }
        }
    }
    const int64_t w = blockIdx.x;
    const int b = (int)(w / p.H), h = (int)(w % p.H);
    const int D = p.D, RS = D + 2;

    int64_t first, stride;
    int count;
    int64_t n_ctx = 0;
    // (offsets, q and the new token are inputs of the step, not products of the partial kernel:
    // they may be read before the grid dependency is resolved)
    if (p.n_parts > 0) {
        first = (int64_t)b * p.H + h;
        stride = (int64_t)p.B * p.H;
        count = p.n_parts;
    } else {
        SeqBounds sb{p.offsets, p.uniform_ctx, p.n_tokens};
        const int64_t sbeg = sb.beg(b), send = sb.beg(b + 1);
        n_ctx = send > sbeg ? send - sbeg : 0;
        const int64_t c0 = sbeg / p.chunk, c1 = n_ctx > 0 ? (send - 1) / p.chunk : c0 - 1;
        first = (c0 + b) * p.H + h;
        stride = p.H;
        count = (int)(c1 - c0 + 1);
    }
    float s_new = -INFINITY;
    if (p.k_new) {
        const QT* qp = (const QT*)p.q + ((int64_t)b * p.H + h) * D;
        const QT* kp = (const QT*)p.k_new + ((int64_t)b * (p.H / p.G) + h / p.G) * D;
        float acc = 0.f;
        for (int d = lane; d < D; d += 32) acc = fmaf(to_f32<QT>(qp[d]), to_f32<QT>(kp[d]), acc);
        s_new = group_sum<32>(acc) * p.scale_log2;
    }
    float v_pre[2] = {0.f, 0.f};                 // the new token's value at this thread's two dims of the first sweep
    if (p.k_new) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int d = threadIdx.x + 128 * k;
            if (d < D) v_pre[k] = to_f32<QT>(((const QT*)p.v_new)[((int64_t)b * (p.H / p.G) + h / p.G) * D + d]);
        }
    }
    // Launched as a programmatic dependent of the partial kernel (see run_combine): the CTA may have
    // started while that grid was still running; from here on its rows are needed.  Without such a
    // launch relation the instruction returns at once.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // global maximum (log2 domain) and denominator: the first 128 units stay in registers
    constexpr int KR = 4;
    float mr[KR], lr[KR];
#pragma unroll
    for (int k = 0; k < KR; ++k) {
        const int i = lane + 32 * k;
        const bool in = i < count;
        mr[k] = in ? p.parts[(first + i * stride) * RS + D] : -INFINITY;
        lr[k] = in ? p.parts[(first + i * stride) * RS + D + 1] : 0.f;
    }
    // The numerator's rows are requested in batches of KB units per warp, every load of a batch
    // independent of the others, and the first batch together with the (m, l) pairs above: a
    // (sequence, head) of up to 32 units costs ONE round trip to L2 after the grid dependency.
    // (A loop with one unit per iteration paid a round trip per unit, up to seven in a row at
    // batch 8: 5 us of a 22 us step.)
    constexpr int KB = 8;
    float rv[KB][8], mi[KB];
    auto load_batch = [&](int i0, int dbase) {
#pragma unroll
        for (int u = 0; u < KB; ++u) {
            const int i = i0 + 4 * u;
            const bool in = i < count;
            const float* row = p.parts + (first + (in ? i : 0) * stride) * RS;
            mi[u] = in ? row[D] : -INFINITY;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int d = dbase + k * 32 + lane;
                rv[u][k] = (in && d < D) ? row[d] : 0.f;
            }
        }
    };
    load_batch(wid, 0);
    float M = fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3]));
    for (int i = lane + 32 * KR; i < count; i += 32) M = fmaxf(M, p.parts[(first + i * stride) * RS + D]);
    if (p.k_new) M = fmaxf(M, s_new);
    M = group_max<32>(M);
    float L = 0.f;
#pragma unroll
    for (int k = 0; k < KR; ++k)
        if (mr[k] > -INFINITY) L += lr[k] * exp2f(mr[k] - M);
    for (int i = lane + 32 * KR; i < count; i += 32) {
        const float mi = p.parts[(first + i * stride) * RS + D];
        const float li = p.parts[(first + i * stride) * RS + D + 1];
        if (mi > -INFINITY) L += li * exp2f(mi - M);
    }
    L = group_sum<32>(L);
    const float w_new = p.k_new ? exp2f(s_new - M) : 0.f;
    L += w_new;
    // numerator: lanes over dims (stride 32, up to 8 accumulators = 256 dims per sweep); warp `wid`
    // takes units wid, wid + 4, ...
    const float inv = (p.out && L > 0.f) ? 1.f / L : 1.f;
    for (int dbase = 0; dbase < D; dbase += 256) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        for (int i0 = wid; i0 < count; i0 += 4 * KB) {
            if (dbase > 0 || i0 > wid) load_batch(i0, dbase);
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const float wi = mi[u] > -INFINITY ? exp2f(mi[u] - M) : 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(rv[u][k], wi, acc[k]);
            }
        }
        if (dbase > 0) __syncthreads();          // the previous sweep's sums have been read
#pragma unroll
        for (int k = 0; k < 8; ++k) s_acc[wid][k * 32 + lane] = acc[k];
        __syncthreads();
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
            const int dd = threadIdx.x + 128 * k2, d = dbase + dd;
            if (d >= D) continue;
            float a = (s_acc[0][dd] + s_acc[1][dd]) + (s_acc[2][dd] + s_acc[3][dd]);
            if (p.k_new)
                a = fmaf(w_new, dbase == 0 ? v_pre[k2]
                                           : to_f32<QT>(((const QT*)p.v_new)[((int64_t)b * (p.H / p.G) + h / p.G) * D + d]), a);
            if (p.out) ((QT*)p.out)[((int64_t)b * p.H + h) * D + d] = from_f32<QT>(a * inv);
            else if (XCHG && p.n_peers > 0) {
                for (int g = 0; g < p.n_peers; ++g) p.peer_dst[g][((int64_t)b * p.H + h) * RS + d] = a;
            } else p.part_out[((int64_t)b * p.H + h) * RS + d] = a;
        }
    }
    if (!p.out && threadIdx.x == 0) {
        if (XCHG && p.n_peers > 0) {
            for (int g = 0; g < p.n_peers; ++g) {
                p.peer_dst[g][((int64_t)b * p.H + h) * RS + D] = M;
                p.peer_dst[g][((int64_t)b * p.H + h) * RS + D + 1] = L;
            }
        } else {
            p.part_out[((int64_t)b * p.H + h) * RS + D] = M;
            p.part_out[((int64_t)b * p.H + h) * RS + D + 1] = L;
        }
    }
    if constexpr (XCHG) {
        if (p.n_peers > 0) {
            __threadfence_system();        // this thread's stores are visible system-wide before the counter moves
            __syncthreads();
            if (threadIdx.x < p.n_peers) atomicAdd_system(p.peer_flag[threadIdx.x], 1);
        }
    }
    if (p.S && p.out) {
        double* Srow = p.S + ((int64_t)b * p.H + h) * p.sp_stride;
        double* Prow = p.P + ((int64_t)b * p.H + h) * p.sp_stride;
        const double Md = (double)M * (double)kLn2;   // natural-log maximum
        const double Ld = (double)L;
        for (int64_t t = threadIdx.x; t < n_ctx; t += 128) Prow[t] = exp(Srow[t] - Md) / Ld;
        if (threadIdx.x == 0 && p.k_new) {
            Srow[n_ctx] = (double)(s_new * kLn2);
            Prow[n_ctx] = (double)w_new / Ld;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static inline int64_t max_units(int B, int64_t n_tokens, int chunk) { return n_tokens / chunk + B + 1; }
template <typename QT, typename KVT>
static int launch_mha(const DecodeParams& p, int warps, int64_t n_units, cudaStream_t st) {
    const int64_t blocks = n_units * p.head_groups;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3((unsigned)(warps * 32));
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool early = p.tables_ready != 0;
    switch (p.D) {
        case 64: return (int)(early ? cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 64, true>, p)
                                    : cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 64, false>, p));
        case 128: return (int)(early ? cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 128, true>, p)
                                     : cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 128, false>, p));
        case 256: return (int)(early ? cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 256, true>, p)
                                     : cudaLaunchKernelEx(&cfg, paged_decode_mha_kernel<QT, KVT, 256, false>, p));
        default: return ATTN_B200_ESHAPE;
    }
}

#include "decode_gqa.cuh"

// Grouped-query decode on the tensor cores (G = 2, 4 or 8, 16-bit KV of the query's type, head_dim 128).
template <typename T>
static int launch_gqa_mma(DecodeParams& p, int64_t n_units, cudaStream_t st) {
    p.head_groups = (p.Hkv + gqa::kWarps - 1) / gqa::kWarps;
    const int64_t blocks = n_units * p.head_groups;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gqa::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        kernel<<<(unsigned)blocks, gqa::kWarps * 32, gqa::kSmemBytes, st>>>(p);
        return (int)cudaGetLastError();
    };
    return p.G == 2 ? go(paged_decode_gqa_mma_kernel<T, 2>)
                    : p.G == 4 ? go(paged_decode_gqa_mma_kernel<T, 4>) : go(paged_decode_gqa_mma_kernel<T, 8>);
}

template <typename QT>
static int launch_gqa_mma_e4m3(DecodeParams& p, int64_t n_units, cudaStream_t st) {
    p.head_groups = (p.Hkv + gqa::kWarps - 1) / gqa::kWarps;
    const int64_t blocks = n_units * p.head_groups;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gqa::kSmemBytes8);
        if (e != cudaSuccess) return (int)e;
        kernel<<<(unsigned)blocks, gqa::kWarps * 32, gqa::kSmemBytes8, st>>>(p);
        return (int)cudaGetLastError();
    };
    return p.G == 2 ? go(paged_decode_gqa_mma_e4m3_kernel<QT, 2>)
                    : p.G == 4 ? go(paged_decode_gqa_mma_e4m3_kernel<QT, 4>) : go(paged_decode_gqa_mma_e4m3_kernel<QT, 8>);
}

template <typename QT, typename KVT, int G>
static int launch_fast_g(const DecodeParams& p, int warps, int64_t n_units, cudaStream_t st) {
    const int64_t blocks = n_units * p.head_groups;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    switch (p.D) {
        case 64: paged_decode_fast_kernel<QT, KVT, 64, G><<<(unsigned)blocks, warps * 32, 0, st>>>(p); break;
        case 128: paged_decode_fast_kernel<QT, KVT, 128, G><<<(unsigned)blocks, warps * 32, 0, st>>>(p); break;
        case 256: paged_decode_fast_kernel<QT, KVT, 256, G><<<(unsigned)blocks, warps * 32, 0, st>>>(p); break;
        default: return ATTN_B200_ESHAPE;
    }
    return (int)cudaGetLastError();
}

template <typename QT, typename KVT>
static int launch_fast(const DecodeParams& p, int warps, int64_t n_units, cudaStream_t st) {
    switch (p.G) {
        case 1: return launch_fast_g<QT, KVT, 1>(p, warps, n_units, st);
        case 2: return launch_fast_g<QT, KVT, 2>(p, warps, n_units, st);
        case 4: return launch_fast_g<QT, KVT, 4>(p, warps, n_units, st);
        case 8: return launch_fast_g<QT, KVT, 8>(p, warps, n_units, st);
        default: return ATTN_B200_ESHAPE;
    }
}

// rows per warp-wide load = KV heads per warp
static int heads_per_warp(int D, int kv_bytes) { return 32 / (D * kv_bytes / 16); }

template <typename QT, typename KVT>
static int launch_generic(const DecodeParams& p, int64_t n_units, cudaStream_t st) {
    const int64_t blocks = n_units * p.H;
    if (blocks > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    const size_t smem = (size_t)p.D * 4 + (size_t)p.chunk * 8;
    if (smem > 40 * 1024) return ATTN_B200_ESHAPE;
    paged_decode_generic_kernel<QT, KVT><<<(unsigned)blocks, 128, smem, st>>>(p);
    return (int)cudaGetLastError();
}

static bool fast_ok(const DecodeParams& p, int q_dtype, int kv_dtype) {
    if (!(p.D == 64 || p.D == 128 || p.D == 256)) return false;
    if (!(p.G == 1 || p.G == 2 || p.G == 4 || p.G == 8)) return false;
    if (!(q_dtype == ATTN_B200_F16 || q_dtype == ATTN_B200_BF16)) return false;
    if (!(kv_dtype == q_dtype || kv_dtype == ATTN_B200_E4M3)) return false;
    if (((uintptr_t)p.k_cache | (uintptr_t)p.v_cache) % 16) return false;
    return true;
}

static int run_stage1(DecodeParams& p, int q_dtype, int kv_dtype, cudaStream_t st) {
    const int64_t n_units = max_units(p.B, p.n_tokens, p.chunk);
    if (fast_ok(p, q_dtype, kv_dtype)) {
        // every row group of a warp takes its own KV head, so that a warp-wide load is one contiguous
        // 512-byte piece of a token's row (2 heads of 16-bit rows, 4 heads of e4m3 rows at head_dim
        // 128) and a CTA of 8 warps streams 4 KB per token.  Measured against a tokens-per-warp
        // mapping on B200: +17 % for e4m3 KV (0.89 -> 1.04 of the copy peak), +3 % for fp16 KV.
        const int hpw = heads_per_warp(p.D, kv_dtype == ATTN_B200_E4M3 ? 1 : 2);
        int warps = (p.Hkv + hpw - 1) / hpw;
        if (warps > 8) warps = 8;
        p.head_groups = (p.Hkv + warps * hpw - 1) / (warps * hpw);
        if ((p.G == 2 || p.G == 4 || p.G == 8) && kv_dtype == q_dtype && p.D == 128 && !p.S)
            return q_dtype == ATTN_B200_F16 ? launch_gqa_mma<__half>(p, n_units, st)
                                            : launch_gqa_mma<__nv_bfloat16>(p, n_units, st);
        if ((p.G == 2 || p.G == 4 || p.G == 8) && kv_dtype == ATTN_B200_E4M3 && p.D == 128 && !p.S)
            return q_dtype == ATTN_B200_F16 ? launch_gqa_mma_e4m3<__half>(p, n_units, st)
                                            : launch_gqa_mma_e4m3<__nv_bfloat16>(p, n_units, st);
        if (p.G == 1 && p.block_size <= 1) {      // multi-head, per-token slot table: specialised kernel
            if (kv_dtype == ATTN_B200_E4M3)
                return q_dtype == ATTN_B200_F16 ? launch_mha<__half, __nv_fp8_e4m3>(p, warps, n_units, st)
                                                : launch_mha<__nv_bfloat16, __nv_fp8_e4m3>(p, warps, n_units, st);
            return q_dtype == ATTN_B200_F16 ? launch_mha<__half, __half>(p, warps, n_units, st)
                                            : launch_mha<__nv_bfloat16, __nv_bfloat16>(p, warps, n_units, st);
        }
        if (kv_dtype == ATTN_B200_E4M3)
            return q_dtype == ATTN_B200_F16 ? launch_fast<__half, __nv_fp8_e4m3>(p, warps, n_units, st)
                                            : launch_fast<__nv_bfloat16, __nv_fp8_e4m3>(p, warps, n_units, st);
        return q_dtype == ATTN_B200_F16 ? launch_fast<__half, __half>(p, warps, n_units, st)
                                        : launch_fast<__nv_bfloat16, __nv_bfloat16>(p, warps, n_units, st);
    }
    p.head_groups = p.H;
    if (kv_dtype == ATTN_B200_E4M3) {
        if (q_dtype == ATTN_B200_F16) return launch_generic<__half, __nv_fp8_e4m3>(p, n_units, st);
        if (q_dtype == ATTN_B200_BF16) return launch_generic<__nv_bfloat16, __nv_fp8_e4m3>(p, n_units, st);
        return ATTN_B200_EDTYPE;
    }
    if (kv_dtype != q_dtype) return ATTN_B200_EDTYPE;
    switch (q_dtype) {
        case ATTN_B200_F16: return launch_generic<__half, __half>(p, n_units, st);
        case ATTN_B200_BF16: return launch_generic<__nv_bfloat16, __nv_bfloat16>(p, n_units, st);
        case ATTN_B200_F32: return launch_generic<float, float>(p, n_units, st);
        default: return ATTN_B200_EDTYPE;
    }
}

static int run_combine(const CombineParams& c, int q_dtype, cudaStream_t st) {
    const int64_t n_rows = (int64_t)c.B * c.H;       // one CTA per (b, h)
    if (n_rows > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    const unsigned blocks = (unsigned)n_rows;
    const bool xchg = c.n_peers > 0 || c.wait_flags != nullptr;
    // Programmatic dependent launch: the kernel may start while the kernel before it in the stream
    // (the partial kernel, which releases its dependents at its start) is still running; it waits
    // for that grid's completion itself, after its prologue.  Saves the launch gap and one round
    // trip of a step that is a few microseconds long.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (q_dtype) {
        case ATTN_B200_F16:
            return (int)(xchg ? cudaLaunchKernelEx(&cfg, lse_combine_kernel<__half, true>, c)
                              : cudaLaunchKernelEx(&cfg, lse_combine_kernel<__half, false>, c));
        case ATTN_B200_BF16:
            return (int)(xchg ? cudaLaunchKernelEx(&cfg, lse_combine_kernel<__nv_bfloat16, true>, c)
                              : cudaLaunchKernelEx(&cfg, lse_combine_kernel<__nv_bfloat16, false>, c));
        case ATTN_B200_F32:
            if (xchg) return ATTN_B200_EDTYPE;
            return (int)cudaLaunchKernelEx(&cfg, lse_combine_kernel<float, false>, c);
        default: return ATTN_B200_EDTYPE;
    }
}

static int check_common(const void* q, const void* kc, const void* vc, int B, int H, int Hkv, int D, int64_t n_tokens,
                        int64_t n_slots, int block_size, int max_blocks, int chunk, int kv_dtype, const float* ks,
                        const float* vs) {
    if (!q || !kc || !vc || B <= 0 || H <= 0 || D <= 0 || n_tokens < 0 || n_slots <= 0) return ATTN_B200_EINVAL;
    if (Hkv <= 0 || H % Hkv) return ATTN_B200_ESHAPE;
    if (block_size < 1 || (block_size > 1 && max_blocks <= 0)) return ATTN_B200_EINVAL;
    if (chunk < 32 || chunk > 2048 || chunk % 32) return ATTN_B200_ESHAPE;
    if (D > 1024) return ATTN_B200_ESHAPE;
    if (n_tokens > 0x7fffffffLL) return ATTN_B200_ETOOLARGE;
    if (kv_dtype == ATTN_B200_E4M3 && (!ks || !vs)) return ATTN_B200_EINVAL;
    return 0;
}

}  // namespace attn

using namespace attn;

extern "C" size_t attn_b200_paged_decode_workspace_bytes(int B, int H, int D, int64_t n_tokens, int chunk) {
    if (B <= 0 || H <= 0 || D <= 0 || n_tokens < 0 || chunk <= 0) return 0;
    return (size_t)max_units(B, n_tokens, chunk) * H * (D + 2) * sizeof(float);
}

extern "C" int attn_b200_paged_decode_pick_chunk(int B, int H, int D, int64_t n_tokens, int sm_count) {
    if (sm_count <= 0) sm_count = 148;
    // CTAs per unit as launched for 16-bit KV (8 warps, 32/(D/8) heads per warp)
    const int lpr = D > 0 ? D / 8 : 16;
    const int hpw = (lpr >= 1 && lpr <= 32) ? 32 / lpr : 1;
    const int64_t heads_per_cta = 8LL * (hpw > 0 ? hpw : 1);
    const int64_t hg = H > 0 ? (H + heads_per_cta - 1) / heads_per_cta : 1;
    int chunk = 1024;
    // largest chunk that still yields >= 16 CTAs per SM (two resident CTAs x eight waves)
    while (chunk > 32 && (n_tokens / chunk + B) * hg < 16LL * sm_count) chunk >>= 1;
    return chunk;
}

// One CTA per (sequence, head) pays when those CTAs alone fill the machine (at least one per SM,
// at most the two per SM that are resident at once, so that it is a single wave) and the sequences
// are short: a CTA works through its sequence 128 tokens per round.  Lengths are not known on the
// host; the capacity per sequence stands in for them.
extern "C" int attn_b200_paged_decode_single_launch_ok(int B, int H, int n_kv_heads, int D, int64_t n_tokens,
                                                       int block_size, int q_dtype, int kv_dtype, int sm_count) {
    if (sm_count <= 0) sm_count = 148;
    if (B <= 0 || H <= 0 || n_kv_heads != H || block_size > 1 || kv_dtype != q_dtype) return 0;
    if (!(q_dtype == ATTN_B200_F16 || q_dtype == ATTN_B200_BF16) || !(D == 64 || D == 128 || D == 256)) return 0;
    const int64_t ctas = (int64_t)B * H;
    return ctas >= sm_count && ctas <= 2LL * sm_count && n_tokens / B <= 1024;
}

extern "C" int attn_b200_paged_decode_pick_chunk_gqa(int B, int n_kv_heads, int group, int D, int kv_dtype,
                                                     int64_t n_tokens, int sm_count) {
    const bool mma = (group == 2 || group == 4 || group == 8) && D == 128 &&
                     (kv_dtype == ATTN_B200_F16 || kv_dtype == ATTN_B200_BF16 || kv_dtype == ATTN_B200_E4M3);
    if (!mma) return attn_b200_paged_decode_pick_chunk(B, n_kv_heads, D, n_tokens, sm_count);
    // tensor-core kernel: a CTA of 4 warps = 4 KV heads, two CTAs per SM; every unit pays for its Q
    // fragments and for filling its copy pipeline, so long units win as soon as there are a few
    // waves of them (measured at G = 8: chunk 256 4.4 TB/s, 1024 5.0)
    if (sm_count <= 0) sm_count = 148;
    const int64_t hg = (n_kv_heads + gqa::kWarps - 1) / gqa::kWarps;
    int chunk = 1024;
    while (chunk > 64 && (n_tokens / chunk + B) * hg < 4LL * sm_count) chunk >>= 1;
    return chunk;
}

extern "C" int attn_b200_paged_decode(const void* q, const void* k_new, const void* v_new, const void* k_cache,
                                      const void* v_cache, const int32_t* slots, const int32_t* offsets, void* out,
                                      void* workspace, size_t workspace_bytes, double* S, double* P,
                                      int64_t sp_stride, int B, int H, int n_kv_heads, int D, int64_t n_tokens,
                                      int64_t n_slots, int uniform_ctx, int block_size, int max_blocks, int chunk,
                                      float scale, const float* k_scale, const float* v_scale, int q_dtype,
                                      int kv_dtype, int stages, int32_t* err_flag, void* stream) {
    int rc = check_common(q, k_cache, v_cache, B, H, n_kv_heads, D, n_tokens, n_slots, block_size, max_blocks, chunk,
                          kv_dtype, k_scale, v_scale);
    if (rc) return rc;
    if (!out || !k_new || !v_new) return ATTN_B200_EINVAL;
    if ((S == nullptr) != (P == nullptr)) return ATTN_B200_EINVAL;
    if (!offsets && (uniform_ctx < 0 || (int64_t)uniform_ctx * B != n_tokens)) return ATTN_B200_EINVAL;
    const int tables_ready = (stages & ATTN_B200_DECODE_TABLES_READY) ? 1 : 0;
    stages &= ~ATTN_B200_DECODE_TABLES_READY;
    if (stages == 4) {      // single launch: one CTA per (sequence, head), no workspace
        if (S || n_kv_heads != H || block_size > 1 || kv_dtype != q_dtype ||
            !(q_dtype == ATTN_B200_F16 || q_dtype == ATTN_B200_BF16) || !(D == 64 || D == 128 || D == 256) ||
            ((uintptr_t)k_cache | (uintptr_t)v_cache) % 16)
            return ATTN_B200_ESHAPE;
        SeqDecodeParams sp{q, k_new, v_new, k_cache, v_cache, slots, offsets, out, B, H, D, n_tokens, n_slots,
                           uniform_ctx, scale * kLog2e, err_flag};
        return q_dtype == ATTN_B200_F16 ? launch_seq<__half>(sp, (cudaStream_t)stream)
                                        : launch_seq<__nv_bfloat16>(sp, (cudaStream_t)stream);
    }
    if (!workspace) return ATTN_B200_EINVAL;
    if (workspace_bytes < attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens, chunk) ||
        (uintptr_t)workspace % 16)
        return ATTN_B200_EWORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int G = H / n_kv_heads;
    DecodeParams p{q, k_cache, v_cache, slots, offsets, (float*)workspace, S, sp_stride, B, H, D, n_tokens, n_slots,
                   uniform_ctx, chunk, scale * kLog2e, kv_dtype == ATTN_B200_E4M3 ? k_scale : nullptr,
                   kv_dtype == ATTN_B200_E4M3 ? v_scale : nullptr, err_flag, 1, n_kv_heads, G, block_size,
                   max_blocks, tables_ready};
    if (stages < 1 || stages > 3) return ATTN_B200_EINVAL;
    if (stages & 1) {
        rc = run_stage1(p, q_dtype, kv_dtype, st);
        if (rc) return rc;
    }
    if (!(stages & 2)) return 0;
    CombineParams c{(const float*)workspace, 0, q, k_new, v_new, out, nullptr, S, P, sp_stride, offsets,
                    uniform_ctx, n_tokens, B, H, D, chunk, scale * kLog2e, G};      // exchange fields zero
    return run_combine(c, q_dtype, st);
}

extern "C" int attn_b200_paged_decode_partial(const void* q, const void* k_cache, const void* v_cache,
                                              const int32_t* slots, const int32_t* offsets, float* part_out,
                                              void* workspace, size_t workspace_bytes, int B, int H, int n_kv_heads,
                                              int D, int64_t n_tokens, int64_t n_slots, int block_size,
                                              int max_blocks, int chunk, float scale, const float* k_scale,
                                              const float* v_scale, int q_dtype, int kv_dtype, int32_t* err_flag,
                                              void* stream) {
    int rc = check_common(q, k_cache, v_cache, B, H, n_kv_heads, D, n_tokens, n_slots, block_size, max_blocks, chunk,
                          kv_dtype, k_scale, v_scale);
    if (rc) return rc;
    if (!part_out || !workspace || !offsets) return ATTN_B200_EINVAL;
    if (workspace_bytes < attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens, chunk) ||
        (uintptr_t)workspace % 16)
        return ATTN_B200_EWORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int G = H / n_kv_heads;
    DecodeParams p{q, k_cache, v_cache, slots, offsets, (float*)workspace, nullptr, 0, B, H, D, n_tokens, n_slots,
                   0, chunk, scale * kLog2e, kv_dtype == ATTN_B200_E4M3 ? k_scale : nullptr,
                   kv_dtype == ATTN_B200_E4M3 ? v_scale : nullptr, err_flag, 1, n_kv_heads, G, block_size,
                   max_blocks};
    rc = run_stage1(p, q_dtype, kv_dtype, st);
    if (rc) return rc;
    CombineParams c{(const float*)workspace, 0, q, nullptr, nullptr, nullptr, part_out, nullptr, nullptr, 0,
                    offsets, 0, n_tokens, B, H, D, chunk, scale * kLog2e, G};
    return run_combine(c, q_dtype, st);
}

extern "C" int attn_b200_paged_decode_partial_push(const void* q, const void* k_cache, const void* v_cache,
                                                   const int32_t* slots, const int32_t* offsets, void* workspace,
                                                   size_t workspace_bytes, int B, int H, int n_kv_heads, int D,
                                                   int64_t n_tokens, int64_t n_slots, int block_size, int max_blocks,
                                                   int chunk, float scale, const float* k_scale, const float* v_scale,
                                                   int q_dtype, int kv_dtype, float* const* peer_dst,
                                                   int32_t* const* peer_flag, int n_peers, int32_t* err_flag,
                                                   void* stream) {
    int rc = check_common(q, k_cache, v_cache, B, H, n_kv_heads, D, n_tokens, n_slots, block_size, max_blocks, chunk,
                          kv_dtype, k_scale, v_scale);
    if (rc) return rc;
    if (!workspace || !offsets || !peer_dst || !peer_flag || n_peers <= 0) return ATTN_B200_EINVAL;
    if (n_peers > kMaxXchgPeers) return ATTN_B200_ETOOLARGE;
    if (q_dtype != ATTN_B200_F16 && q_dtype != ATTN_B200_BF16) return ATTN_B200_EDTYPE;
    if (workspace_bytes < attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens, chunk) ||
        (uintptr_t)workspace % 16)
        return ATTN_B200_EWORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int G = H / n_kv_heads;
    DecodeParams p{q, k_cache, v_cache, slots, offsets, (float*)workspace, nullptr, 0, B, H, D, n_tokens, n_slots,
                   0, chunk, scale * kLog2e, kv_dtype == ATTN_B200_E4M3 ? k_scale : nullptr,
                   kv_dtype == ATTN_B200_E4M3 ? v_scale : nullptr, err_flag, 1, n_kv_heads, G, block_size,
                   max_blocks};
    rc = run_stage1(p, q_dtype, kv_dtype, st);
    if (rc) return rc;
    CombineParams c{(const float*)workspace, 0, q, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0,
                    offsets, 0, n_tokens, B, H, D, chunk, scale * kLog2e, G};
    c.n_peers = n_peers;
    for (int g = 0; g < n_peers; ++g) {
        if (!peer_dst[g] || !peer_flag[g]) return ATTN_B200_EINVAL;
        c.peer_dst[g] = peer_dst[g];
        c.peer_flag[g] = peer_flag[g];
    }
    return run_combine(c, q_dtype, st);
}

extern "C" int attn_b200_lse_combine_wait(const float* parts, int n_parts, const void* q, const void* k_new,
                                          const void* v_new, void* out, int B, int H, int n_kv_heads, int D,
                                          float scale, int q_dtype, int32_t* flags, int32_t* done_counter,
                                          int32_t* err_flag, void* stream) {
    if (!parts || n_parts <= 0 || !out || B <= 0 || H <= 0 || D <= 0 || !flags || !done_counter) return ATTN_B200_EINVAL;
    if (n_parts > kMaxXchgPeers) return ATTN_B200_ETOOLARGE;
    if (n_kv_heads <= 0 || H % n_kv_heads) return ATTN_B200_ESHAPE;
    if ((k_new == nullptr) != (v_new == nullptr)) return ATTN_B200_EINVAL;
    if (k_new && !q) return ATTN_B200_EINVAL;
    if (q_dtype != ATTN_B200_F16 && q_dtype != ATTN_B200_BF16) return ATTN_B200_EDTYPE;
    CombineParams c{parts, n_parts, q, k_new, v_new, out, nullptr, nullptr, nullptr, 0, nullptr, 0, 0,
                    B, H, D, 32, scale * kLog2e, H / n_kv_heads};
    c.wait_flags = flags;
    c.wait_count = (int32_t)((int64_t)B * H);
    c.done_counter = done_counter;
    c.err_flag = err_flag;
    return run_combine(c, q_dtype, (cudaStream_t)stream);
}

extern "C" int attn_b200_lse_combine(const float* parts, int n_parts, const void* q, const void* k_new,
                                     const void* v_new, void* out, int B, int H, int n_kv_heads, int D, float scale,
                                     int q_dtype, void* stream) {
    if (!parts || n_parts <= 0 || !out || B <= 0 || H <= 0 || D <= 0) return ATTN_B200_EINVAL;
    if (n_kv_heads <= 0 || H % n_kv_heads) return ATTN_B200_ESHAPE;
    if ((k_new == nullptr) != (v_new == nullptr)) return ATTN_B200_EINVAL;
    if (k_new && !q) return ATTN_B200_EINVAL;
    CombineParams c{parts, n_parts, q, k_new, v_new, out, nullptr, nullptr, nullptr, 0, nullptr, 0, 0,
                    B, H, D, 32, scale * kLog2e, H / n_kv_heads};
    return run_combine(c, q_dtype, (cudaStream_t)stream);
}
