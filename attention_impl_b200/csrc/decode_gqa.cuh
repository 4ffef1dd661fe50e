// Split-KV partial kernel for grouped-query decode (G = 2, 4 or 8 query heads per KV head, 16-bit KV,
// head_dim 128) with the row products on the tensor cores.  Included by decode.cu after its
// parameter block and unit helpers.
//
// Why: the CUDA-core kernel does the arithmetic of MHA per token and query head while the bytes
// shrink by G; from G = 4 up it is bound by instruction issue (3.2 TB/s at G = 4, 1.2 at G = 8).
// Here a warp owns one KV head and its G query heads and walks the unit's tokens 16 at a time:
//   S[16 x 16] = Q[16 x 128] K^T   16 x mma.sync.m16n8k16 (rows >= G of Q are zero)
//   online softmax on the rows it owns (row = lane / 4; the 4 lanes of a row hold 4 tokens each)
//   O[16 x 128] += P[16 x 16] V    16 x mma.sync.m16n8k16, P taken straight from the S fragments
// (mma.sync, not tcgen05: M is 2 to 8 rows; a 128-row tcgen05 tile would be 94 % padding or more.
// G = 2 is memory bound either way; the gain there, 5.3 -> 5.95 TB/s, comes from the copy pipeline.)
//
// Data movement.  Lane (n = lane / 4, c = lane % 4) copies, for tokens n and 8 + n of the tile,
// the 16-byte chunks (4 j + c), j = 0..3, of the head's K row and V row with cp.async into a
// 3-stage ring in shared memory that is private to the warp - and later reads back exactly the
// chunks it copied, so no thread ever waits for another (cp.async.wait_group is all the
// synchronisation there is) and 16 KB per warp are in flight regardless of registers.
//
// Fragments.  A dot product does not care in which order the dims are visited, so the 8 k-slices of
// the MMA use the dims in the order the lanes hold them: slice 2j + e takes, from lane (n, c), the
// dims (4j + c) * 8 + 4e + {0, 1} as k = 2c, 2c + 1 and + {2, 3} as k = 2c + 8, 2c + 9; Q's A
// fragments are loaded once with the same mapping.  For P V the B operand wants pairs of TOKENS per
// register: movmatrix.trans turns the 8-token x 8-dim block that the lanes hold row-wise (one
// register per lane) into that form.  The output columns come out so that lane (row, c) owns the
// same 32 dims of its row that it loaded.
#pragma once

namespace gqa {

constexpr int kWarps = 4;            // warps (= KV heads) per CTA
constexpr int kStages = 3;           // tiles in flight per warp
constexpr int kTile = 16;            // tokens per tile
constexpr int kStageBytes = kTile * 512;   // K and V rows of a tile for one head (fp16/bf16, D = 128)
constexpr int kSmemBytes = kWarps * kStages * kStageBytes;

template <typename T> struct Mma;
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float x, float y) {
        const __half2 h = __floats2half2_rn(x, y);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float x, float y) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

}  // namespace gqa

template <typename T, int G>
__global__ void __launch_bounds__(gqa::kWarps * 32, 2)
paged_decode_gqa_mma_kernel(const DecodeParams p) {
    using namespace gqa;
    constexpr int D = 128;
    extern __shared__ __align__(16) unsigned char ring_raw[];
    __shared__ int32_t s_off[kMaxStagedB];
    SeqBounds sb{stage_offsets(p, s_off), p.uniform_ctx, p.n_tokens};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = lane >> 2, c = lane & 3;
    const int64_t u = blockIdx.x / p.head_groups;
    const int hk = (int)(blockIdx.x % p.head_groups) * kWarps + warp;
    Unit un;
    if (!resolve_unit(u, p.B, p.chunk, sb, un) || hk >= p.Hkv) return;

    // Q as A fragments (rows >= G stay zero): slice s = 2j + e, registers {k = 2c.., k = 2c+8..}
    uint32_t aq[8][2];
    {
        const bool row_ok = n < G;
        const T* qrow = (const T*)p.q + ((int64_t)un.b * p.H + hk * G + (row_ok ? n : 0)) * D;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(qrow + (4 * j + c) * 8 + 4 * e);
                aq[2 * j + e][0] = row_ok ? src[0] : 0u;
                aq[2 * j + e][1] = row_ok ? src[1] : 0u;
            }
    }
    const int64_t row_bytes = (int64_t)p.Hkv * D * sizeof(T);
    const char* kbase = (const char*)p.k_cache + ((int64_t)hk * D + c * 8) * sizeof(T);
    const char* vbase = (const char*)p.v_cache + ((int64_t)hk * D + c * 8) * sizeof(T);
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_raw) + warp * kStages * kStageBytes + lane * 16;

    const int nt = (int)((un.tend - un.tbeg + kTile - 1) / kTile);
    // slot of token `lane` of a tile (lanes 0..15), or -1
    auto tile_slot = [&](int t) -> int {
        const int64_t tok = un.tbeg + (int64_t)t * kTile + lane;
        return (t < nt && lane < kTile && tok < un.tend) ? token_slot(p, un, tok) : -1;
    };
    // copies of tile t into stage t % kStages; returns the validity bits of its 16 tokens
    auto issue = [&](int t, int my_slot) -> unsigned {
        const uint32_t base = ring + (t % kStages) * kStageBytes;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const int sl = __shfl_sync(0xffffffffu, my_slot, grp * 8 + n);
            const int64_t off = (int64_t)(sl >= 0 ? sl : 0) * row_bytes;
            const int nb = sl >= 0 ? 16 : 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                cp_async_16(base + ((grp * 2 + 0) * 4 + j) * 512, kbase + off + j * 64, nb);
                cp_async_16(base + ((grp * 2 + 1) * 4 + j) * 512, vbase + off + j * 64, nb);
            }
        }
        return __ballot_sync(0xffffffffu, my_slot >= 0) & 0xffffu;
    };

    float oacc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) oacc[i][k] = 0.f;
    float m = -INFINITY, l = 0.f;

    // pipeline: tiles t+1 and t+2 are in flight while tile t is multiplied
    unsigned v0 = 0, v1 = 0, v2 = 0;        // validity bits of the tiles computed next, after that, and just issued
    int next_slot = tile_slot(0);
    {
        const int s0 = next_slot;
        next_slot = tile_slot(1);
        v0 = issue(0, s0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int s1 = next_slot;
        next_slot = tile_slot(2);
        if (nt > 1) v1 = issue(1, s1);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int t = 0; t < nt; ++t) {
        {
            const int s2 = next_slot;
            next_slot = tile_slot(t + 3);
            v2 = 0;
            if (t + 2 < nt) v2 = issue(t + 2, s2);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        const uint32_t base = ring + (t % kStages) * kStageBytes;
        const unsigned vb = v0;
        v0 = v1;
        v1 = v2;

        // S = Q K^T for the tile's two groups of 8 tokens
        float sacc[2][4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
            for (int k = 0; k < 4; ++k) sacc[grp][k] = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 kc;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(kc.x), "=r"(kc.y), "=r"(kc.z), "=r"(kc.w)
                             : "r"(base + ((grp * 2 + 0) * 4 + j) * 512));
                const uint32_t a0[4] = {aq[2 * j][0], 0u, aq[2 * j][1], 0u};
                const uint32_t a1[4] = {aq[2 * j + 1][0], 0u, aq[2 * j + 1][1], 0u};
                Mma<T>::run(sacc[grp], a0, kc.x, kc.y);
                Mma<T>::run(sacc[grp], a1, kc.z, kc.w);
            }
        }
        // this lane's four scores of row n: tokens grp*8 + 2c + {0, 1}
        float sc[4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bool ok = (vb >> (grp * 8 + 2 * c + i)) & 1u;
                sc[grp * 2 + i] = ok ? sacc[grp][i] * p.scale_log2 : -INFINITY;
            }
        float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m, tmax);
        const float msub = m_new > -INFINITY ? m_new : 0.f;     // no valid token yet: exp2(-inf - 0) = 0
        const float alpha = fast_exp2(m - msub);
        float pr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pr[i] = fast_exp2(sc[i] - msub);
        l = l * alpha + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            oacc[i][0] *= alpha;
            oacc[i][1] *= alpha;
        }
        // O += P V: P's A fragments are the score fragments (tokens 2c, 2c+1 of group 0 are k = 2c, 2c+1;
        // of group 1, k = 2c + 8, 2c + 9)
        const uint32_t pa[4] = {Mma<T>::pack(pr[0], pr[1]), 0u, Mma<T>::pack(pr[2], pr[3]), 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 va, vb4;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(va.x), "=r"(va.y), "=r"(va.z), "=r"(va.w)
                         : "r"(base + ((0 * 2 + 1) * 4 + j) * 512));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(vb4.x), "=r"(vb4.y), "=r"(vb4.z), "=r"(vb4.w)
                         : "r"(base + ((1 * 2 + 1) * 4 + j) * 512));
            const uint32_t w0[4] = {va.x, va.y, va.z, va.w}, w1[4] = {vb4.x, vb4.y, vb4.z, vb4.w};
#pragma unroll
            for (int r = 0; r < 4; ++r)
                Mma<T>::run(oacc[j * 4 + r], pa, movmatrix_trans(w0[r]), movmatrix_trans(w1[r]));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the four lanes of a row hold disjoint tokens: fold their denominators
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (n < G) {
        const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
        float* row = p.part + ((int64_t)u * p.H + hk * G + n) * (D + 2);
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r)
                *reinterpret_cast<float2*>(row + (4 * j + c) * 8 + 2 * r) =
                    make_float2(oacc[j * 4 + r][0] * vs, oacc[j * 4 + r][1] * vs);
        if (c == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m, l);
    }
}

// The same kernel for e4m3 pools: a token's row of a head is 128 bytes = 8 chunks of 16 dims, lane
// (n, c) copies chunks 4j + c (j = 0, 1); a 32-bit word of a chunk (4 e4m3) becomes two fp16 pairs
// (cvt.rn.f16x2.e4m3x2), which are the two B registers of one k-slice for Q K^T and two 8-dim output
// blocks for P V.  The MMAs are fp16 for either query type (q is converted once, as the CUDA-core
// e4m3 kernels do); the per-head scales enter the score and the output.
namespace gqa {
constexpr int kStageBytes8 = kTile * 256;
constexpr int kSmemBytes8 = kWarps * kStages * kStageBytes8;
}  // namespace gqa

template <typename QT, int G>
__global__ void __launch_bounds__(gqa::kWarps * 32, 2)
paged_decode_gqa_mma_e4m3_kernel(const DecodeParams p) {
    using namespace gqa;
    using M16 = Mma<__half>;
    constexpr int D = 128;
    extern __shared__ __align__(16) unsigned char ring_raw[];
    __shared__ int32_t s_off[kMaxStagedB];
    SeqBounds sb{stage_offsets(p, s_off), p.uniform_ctx, p.n_tokens};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = lane >> 2, c = lane & 3;
    const int64_t u = blockIdx.x / p.head_groups;
    const int hk = (int)(blockIdx.x % p.head_groups) * kWarps + warp;
    Unit un;
    if (!resolve_unit(u, p.B, p.chunk, sb, un) || hk >= p.Hkv) return;

    // Q as fp16 A fragments: slice s = 4j + e takes dims (4j + c) * 16 + 4e + {0, 1} and + {2, 3}
    uint32_t aq[8][2];
    {
        const bool row_ok = n < G;
        const QT* qrow = (const QT*)p.q + ((int64_t)un.b * p.H + hk * G + (row_ok ? n : 0)) * D;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const QT* src = qrow + (4 * j + c) * 16 + 4 * e;
                aq[4 * j + e][0] = row_ok ? M16::pack(to_f32<QT>(src[0]), to_f32<QT>(src[1])) : 0u;
                aq[4 * j + e][1] = row_ok ? M16::pack(to_f32<QT>(src[2]), to_f32<QT>(src[3])) : 0u;
            }
    }
    const float qs = p.scale_log2 * (p.k_scale ? p.k_scale[hk] : 1.f);
    const int64_t row_bytes = (int64_t)p.Hkv * D;
    const char* kbase = (const char*)p.k_cache + (int64_t)hk * D + c * 16;
    const char* vbase = (const char*)p.v_cache + (int64_t)hk * D + c * 16;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_raw) + warp * kStages * kStageBytes8 + lane * 16;

    const int nt = (int)((un.tend - un.tbeg + kTile - 1) / kTile);
    auto tile_slot = [&](int t) -> int {
        const int64_t tok = un.tbeg + (int64_t)t * kTile + lane;
        return (t < nt && lane < kTile && tok < un.tend) ? token_slot(p, un, tok) : -1;
    };
    auto issue = [&](int t, int my_slot) -> unsigned {
        const uint32_t base = ring + (t % kStages) * kStageBytes8;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const int sl = __shfl_sync(0xffffffffu, my_slot, grp * 8 + n);
            const int64_t off = (int64_t)(sl >= 0 ? sl : 0) * row_bytes;
            const int nb = sl >= 0 ? 16 : 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                cp_async_16(base + ((grp * 2 + 0) * 2 + j) * 512, kbase + off + j * 64, nb);
                cp_async_16(base + ((grp * 2 + 1) * 2 + j) * 512, vbase + off + j * 64, nb);
            }
        }
        return __ballot_sync(0xffffffffu, my_slot >= 0) & 0xffffu;
    };

    float oacc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) oacc[i][k] = 0.f;
    float m = -INFINITY, l = 0.f;

    unsigned v0 = 0, v1 = 0, v2 = 0;
    int next_slot = tile_slot(0);
    {
        const int s0 = next_slot;
        next_slot = tile_slot(1);
        v0 = issue(0, s0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int s1 = next_slot;
        next_slot = tile_slot(2);
        if (nt > 1) v1 = issue(1, s1);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int t = 0; t < nt; ++t) {
        {
            const int s2 = next_slot;
            next_slot = tile_slot(t + 3);
            v2 = 0;
            if (t + 2 < nt) v2 = issue(t + 2, s2);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        const uint32_t base = ring + (t % kStages) * kStageBytes8;
        const unsigned vb = v0;
        v0 = v1;
        v1 = v2;

        float sacc[2][4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
            for (int k = 0; k < 4; ++k) sacc[grp][k] = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t w[4];
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                             : "r"(base + ((grp * 2 + 0) * 2 + j) * 512));
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __half2 lo, hi;
                    e4m3x4_to_half2x2(w[e], lo, hi);
                    const uint32_t a[4] = {aq[4 * j + e][0], 0u, aq[4 * j + e][1], 0u};
                    M16::run(sacc[grp], a, *reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                }
            }
        }
        float sc[4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bool ok = (vb >> (grp * 8 + 2 * c + i)) & 1u;
                sc[grp * 2 + i] = ok ? sacc[grp][i] * qs : -INFINITY;
            }
        float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m, tmax);
        const float msub = m_new > -INFINITY ? m_new : 0.f;
        const float alpha = fast_exp2(m - msub);
        float pr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pr[i] = fast_exp2(sc[i] - msub);
        l = l * alpha + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            oacc[i][0] *= alpha;
            oacc[i][1] *= alpha;
        }
        const uint32_t pa[4] = {M16::pack(pr[0], pr[1]), 0u, M16::pack(pr[2], pr[3]), 0u};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t w0[4], w1[4];
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w0[0]), "=r"(w0[1]), "=r"(w0[2]), "=r"(w0[3])
                         : "r"(base + ((0 * 2 + 1) * 2 + j) * 512));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w1[0]), "=r"(w1[1]), "=r"(w1[2]), "=r"(w1[3])
                         : "r"(base + ((1 * 2 + 1) * 2 + j) * 512));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half2 lo0, hi0, lo1, hi1;
                e4m3x4_to_half2x2(w0[e], lo0, hi0);
                e4m3x4_to_half2x2(w1[e], lo1, hi1);
                M16::run(oacc[(j * 4 + e) * 2 + 0], pa, movmatrix_trans(*reinterpret_cast<const uint32_t*>(&lo0)),
                         movmatrix_trans(*reinterpret_cast<const uint32_t*>(&lo1)));
                M16::run(oacc[(j * 4 + e) * 2 + 1], pa, movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi0)),
                         movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi1)));
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (n < G) {
        const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
        float* row = p.part + ((int64_t)u * p.H + hk * G + n) * (D + 2);
        // output block (j, e, h) of this lane: dims (4j + c) * 16 + 4e + 2h + {0, 1}
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<float2*>(row + (4 * j + c) * 16 + 4 * e + 2 * hh) =
                        make_float2(oacc[(j * 4 + e) * 2 + hh][0] * vs, oacc[(j * 4 + e) * 2 + hh][1] * vs);
        if (c == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m, l);
    }
}
