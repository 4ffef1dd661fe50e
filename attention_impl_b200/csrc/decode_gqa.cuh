// Split-KV partial kernel for grouped-query decode (G = 2, 4 or 8 query heads per KV head, 16-bit KV,
// head_dim 128) with the row products on the tensor cores.  Included by decode.cu after its
// parameter block and unit helpers.
//
// Why: the CUDA-core kernel does the arithmetic of MHA per token and query head while the bytes
// shrink by G; from G = 4 up it is bound by instruction issue (3.2 TB/s at G = 4, 1.2 at G = 8).
// Here a warp owns one KV head and its G query heads and walks the unit's tokens 16 at a time, with
// the KEYS as the M dimension of the MMAs (with the heads as M half of every A fragment was padding
// for G <= 8 and a tile cost 32 MMAs instead of 16):
//   S^T[16 keys x 8 heads] = K[16 x 128] Q^T      8 x mma.sync.m16n8k16 (heads >= G of Q are zero)
//   online softmax per head: lane (n, c) holds keys n, 8 + n of heads 2c, 2c + 1; the maximum over
//   the keys is three shuffles over n
//   O^T[128 dims x 8 heads] += V^T[128 x 16] P^T  8 x mma.sync.m16n8k16; P^T is the transposed score
//   fragment (two movmatrix), V^T the transposed 8-key x 8-dim blocks the lanes hold (four per MMA)
// (mma.sync, not tcgen05: N is 2 to 8 heads; a 128-row tcgen05 tile would be mostly padding.
// G = 2 is memory bound either way; the gain there, 5.3 -> 5.95 TB/s, comes from the copy pipeline.)
//
// Data movement.  Lane (n = lane / 4, c = lane % 4) copies, for tokens n and 8 + n of the tile,
// the 16-byte chunks (4 j + c), j = 0..3, of the head's K row and V row with cp.async into a
// 3-stage ring in shared memory that is private to the warp - and later reads back exactly the
// chunks it copied, so no thread ever waits for another (cp.async.wait_group is all the
// synchronisation there is) and 16 KB per warp are in flight regardless of registers.
//
// Fragments.  A dot product does not care in which order the dims are visited, so the 8 k-slices of
// the first product use the dims in the order the lanes hold them: slice 2j + e takes, from lane
// (n, c), for keys n and 8 + n (the A rows), the dims (4j + c) * 8 + 4e + {0, 1} as k = 2c, 2c + 1 and
// + {2, 3} as k = 2c + 8, 2c + 9; Q^T's B fragments (head n of lane (n, c)) are loaded once with the
// same mapping.  For the second product the A operand wants pairs of KEYS per register:
// movmatrix.trans turns the 8-key x 8-dim block that the lanes hold row-wise (one register per lane)
// into that form; the 16 rows of output block (j, e) are the dims (4j + r/2) * 8 + 4e + r%2 (r = 0..7,
// first word of the pair) and + 2 (second word).
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

    // Q^T as B fragments of head n (heads >= G stay zero): slice s = 2j + e, registers {k = 2c.., k = 2c+8..}
    uint32_t bq[8][2];
    {
        const bool row_ok = n < G;
        const T* qrow = (const T*)p.q + ((int64_t)un.b * p.H + hk * G + (row_ok ? n : 0)) * D;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(qrow + (4 * j + c) * 8 + 4 * e);
                bq[2 * j + e][0] = row_ok ? src[0] : 0u;
                bq[2 * j + e][1] = row_ok ? src[1] : 0u;
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
    auto lds128 = [](uint32_t addr, uint32_t (&w)[4]) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    };

    // O^T accumulators: block (j, e) = oacc[2j + e]: {dim row n, head 2c | head 2c+1 | dim row 8+n, head 2c | head 2c+1}
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) oacc[i][k] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // heads 2c and 2c + 1 (l: this lane's keys only)

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

        // S^T = K Q^T: rows = keys n, 8 + n; columns = heads 2c, 2c + 1
        float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w0[4], w1[4];          // key n, key 8 + n: chunk 4j + c
            lds128(base + ((0 * 2 + 0) * 4 + j) * 512, w0);
            lds128(base + ((1 * 2 + 0) * 4 + j) * 512, w1);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t a[4] = {w0[2 * e], w1[2 * e], w0[2 * e + 1], w1[2 * e + 1]};
                Mma<T>::run(sacc, a, bq[2 * j + e][0], bq[2 * j + e][1]);
            }
        }
        const bool ok0 = (vb >> n) & 1u, ok1 = (vb >> (8 + n)) & 1u;
        float pr[4];                         // (key n, head 2c), (key n, 2c+1), (key 8+n, 2c), (key 8+n, 2c+1)
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float s0 = ok0 ? sacc[i] * p.scale_log2 : -INFINITY, s1 = ok1 ? sacc[2 + i] * p.scale_log2 : -INFINITY;
            float tmax = fmaxf(s0, s1);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
            const float m_new = fmaxf(m[i], tmax);
            const float msub = m_new > -INFINITY ? m_new : 0.f;     // no valid token yet: exp2(-inf - 0) = 0
            alpha[i] = fast_exp2(m[i] - msub);
            pr[i] = fast_exp2(s0 - msub);
            pr[2 + i] = fast_exp2(s1 - msub);
            l[i] = l[i] * alpha[i] + (pr[i] + pr[2 + i]);
            m[i] = m_new;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            oacc[i][0] *= alpha[0];
            oacc[i][1] *= alpha[1];
            oacc[i][2] *= alpha[0];
            oacc[i][3] *= alpha[1];
        }
        // P^T as the B operand: transpose the 8-key x 8-head blocks of the score fragment
        const uint32_t pb0 = movmatrix_trans(Mma<T>::pack(pr[0], pr[1]));      // head n; keys 2c, 2c + 1
        const uint32_t pb1 = movmatrix_trans(Mma<T>::pack(pr[2], pr[3]));      // head n; keys 8 + 2c, 9 + 2c
        // O^T += V^T P^T: A = transposed 8-key x 8-dim blocks (word 2e -> rows 0..7, word 2e + 1 -> rows 8..15)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w0[4], w1[4];
            lds128(base + ((0 * 2 + 1) * 4 + j) * 512, w0);
            lds128(base + ((1 * 2 + 1) * 4 + j) * 512, w1);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t a[4] = {movmatrix_trans(w0[2 * e]), movmatrix_trans(w0[2 * e + 1]),
                                       movmatrix_trans(w1[2 * e]), movmatrix_trans(w1[2 * e + 1])};
                Mma<T>::run(oacc[2 * j + e], a, pb0, pb1);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the eight lanes with this lane's c hold disjoint keys: fold their denominators
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 4);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
    }
    const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int hq = 2 * c + i;
        if (hq >= G) continue;
        float* row = p.part + ((int64_t)u * p.H + hk * G + hq) * (D + 2);
        // block (j, e): row n of the first word's block is dim (4j + n/2) * 8 + 4e + n%2, of the second word's + 2
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int d = (4 * j + (n >> 1)) * 8 + 4 * e + (n & 1);
                row[d] = oacc[2 * j + e][i] * vs;
                row[d + 2] = oacc[2 * j + e][2 + i] * vs;
            }
        if (n == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m[i], l[i]);
    }
}

// The kernel for e4m3 pools, with the KEYS as the M dimension of the MMAs.
//
// A token's row of a head is 128 bytes = 8 chunks of 16 dims; lane (n, c) copies chunks 4j + c
// (j = 0, 1) of tokens n and 8 + n of the tile and reads back what it copied, as above.  With the
// query heads as M (the 16-bit kernel's form) half of every A fragment is padding for G <= 8 and a
// 16-key tile costs 32 MMAs, about half of the instruction issue time of this conversion-heavy
// kernel.  Here a tile is
//   S^T[16 keys x 8 heads] = K[16 x 128] Q^T      8 x mma.sync.m16n8k16 (fp16; heads >= G are zero)
//   O^T[128 dims x 8 heads] += V^T[128 x 16] P^T  8 x mma.sync.m16n8k16
// 16 MMAs.  K is the A operand straight from the converted words: for k-slice s = 4j + e lane (n, c)
// supplies, for keys n and 8 + n, the dims (4j + c) * 16 + 4e + {0, 1} (k = 2c, 2c + 1) and + {2, 3}
// (k = 2c + 8, 2c + 9); Q^T is the B operand with the same dim order (b0, b1 of lane (h, c) = those
// dims of head h).  The score fragment of lane (n, c) is (key n | key 8 + n) x (heads 2c, 2c + 1):
// a lane tracks the running maximum and denominator of its two heads, the maximum over the keys is
// three shuffles over n.  P^T as the B operand of the second product is the transposed score
// fragment: two movmatrix.  V^T as its A operand is the transposed 8-key x 8-"dim" blocks the lanes
// hold (four movmatrix per MMA, as many as before); the 16 rows of output block (j, e) are the dims
// (4j + r/2) * 16 + 4e + r%2 (rows r = 0..7, from the words' low halves) and + 2 (rows 8..15, high
// halves).  The MMAs are fp16 for either query type; the per-head scales enter the score and the output.
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

    // Q^T as fp16 B fragments of head n: slice s = 4j + e holds dims (4j + c) * 16 + 4e + {0, 1} and + {2, 3}
    uint32_t bq[8][2];
    {
        const bool row_ok = n < G;
        const QT* qrow = (const QT*)p.q + ((int64_t)un.b * p.H + hk * G + (row_ok ? n : 0)) * D;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const QT* src = qrow + (4 * j + c) * 16 + 4 * e;
                bq[4 * j + e][0] = row_ok ? M16::pack(to_f32<QT>(src[0]), to_f32<QT>(src[1])) : 0u;
                bq[4 * j + e][1] = row_ok ? M16::pack(to_f32<QT>(src[2]), to_f32<QT>(src[3])) : 0u;
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
    auto lds128 = [](uint32_t addr, uint32_t (&w)[4]) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    };
    auto u32 = [](const __half2& h) { return *reinterpret_cast<const uint32_t*>(&h); };

    // O^T accumulators: block (j, e) = oacc[4j + e]: {dim row n, head 2c | head 2c+1 | dim row 8+n, head 2c | head 2c+1}
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) oacc[i][k] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // heads 2c and 2c + 1 (l: this lane's keys only)

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

        // S^T = K Q^T: rows = keys n, 8 + n; columns = heads 2c, 2c + 1
        float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t w0[4], w1[4];          // key n, key 8 + n: chunk 4j + c
            lds128(base + ((0 * 2 + 0) * 2 + j) * 512, w0);
            lds128(base + ((1 * 2 + 0) * 2 + j) * 512, w1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half2 lo0, hi0, lo1, hi1;
                e4m3x4_to_half2x2(w0[e], lo0, hi0);
                e4m3x4_to_half2x2(w1[e], lo1, hi1);
                const uint32_t a[4] = {u32(lo0), u32(lo1), u32(hi0), u32(hi1)};
                M16::run(sacc, a, bq[4 * j + e][0], bq[4 * j + e][1]);
            }
        }
        const bool ok0 = (vb >> n) & 1u, ok1 = (vb >> (8 + n)) & 1u;
        float pr[4];                         // (key n, head 2c), (key n, 2c+1), (key 8+n, 2c), (key 8+n, 2c+1)
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float s0 = ok0 ? sacc[i] * qs : -INFINITY, s1 = ok1 ? sacc[2 + i] * qs : -INFINITY;
            float tmax = fmaxf(s0, s1);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
            const float m_new = fmaxf(m[i], tmax);
            const float msub = m_new > -INFINITY ? m_new : 0.f;     // no valid token yet: exp2(-inf - 0) = 0
            alpha[i] = fast_exp2(m[i] - msub);
            pr[i] = fast_exp2(s0 - msub);
            pr[2 + i] = fast_exp2(s1 - msub);
            l[i] = l[i] * alpha[i] + (pr[i] + pr[2 + i]);
            m[i] = m_new;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            oacc[i][0] *= alpha[0];
            oacc[i][1] *= alpha[1];
            oacc[i][2] *= alpha[0];
            oacc[i][3] *= alpha[1];
        }
        // P^T as the B operand: transpose the 8-key x 8-head blocks of the score fragment
        const uint32_t pb0 = movmatrix_trans(M16::pack(pr[0], pr[1]));      // head n; keys 2c, 2c + 1
        const uint32_t pb1 = movmatrix_trans(M16::pack(pr[2], pr[3]));      // head n; keys 8 + 2c, 9 + 2c
        // O^T += V^T P^T: A = transposed 8-key x 8-dim blocks (low halves -> rows 0..7, high -> rows 8..15)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t w0[4], w1[4];
            lds128(base + ((0 * 2 + 1) * 2 + j) * 512, w0);
            lds128(base + ((1 * 2 + 1) * 2 + j) * 512, w1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half2 lo0, hi0, lo1, hi1;
                e4m3x4_to_half2x2(w0[e], lo0, hi0);
                e4m3x4_to_half2x2(w1[e], lo1, hi1);
                const uint32_t a[4] = {movmatrix_trans(u32(lo0)), movmatrix_trans(u32(hi0)), movmatrix_trans(u32(lo1)),
                                       movmatrix_trans(u32(hi1))};
                M16::run(oacc[4 * j + e], a, pb0, pb1);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the eight lanes with this lane's c hold disjoint keys: fold their denominators
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 4);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
    }
    const float vs = p.v_scale ? p.v_scale[hk] : 1.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int hq = 2 * c + i;
        if (hq >= G) continue;
        float* row = p.part + ((int64_t)u * p.H + hk * G + hq) * (D + 2);
        // block (j, e): row n of the low-half block is dim (4j + n/2) * 16 + 4e + n%2, of the high-half block + 2
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = (4 * j + (n >> 1)) * 16 + 4 * e + (n & 1);
                row[d] = oacc[4 * j + e][i] * vs;
                row[d + 2] = oacc[4 * j + e][2 + i] * vs;
            }
        if (n == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m[i], l[i]);
    }
}
