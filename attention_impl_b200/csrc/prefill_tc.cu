// Causal prefill on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators, operands
// staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle).
//
// Semantics: paged_attention_kernel.cu:15-98 of the reference (per sequence slice of the packed
// buffer, key j visible to query i iff j <= i, softmax of scale*QK^T, O = P V), evaluated flash
// style: S and P never leave the SM.  Two kernels share one pipeline (a pair of 128-row query
// tiles per work item, one softmax thread per query row, P and O resident in tensor memory):
//   prefill_tc2p_kernel      persistent: one CTA per SM draws pairs from a counter
//   paged_prefill_tc_kernel  K/V gathered through a slot table (chunked / prefix-cached prefill)
// Every mbarrier wait is bounded (about one second of SM clocks); on expiry the kernel raises
// ATTN_B200_FLAG_TIMEOUT, all roles leave their loops, outstanding copies are given a bounded
// wait, TMEM is freed and the CTA returns.  CTAs that start after a timeout exit at once.
#include <cuda.h>
#include <cstdlib>
#include <atomic>
#include <mutex>
#include <type_traits>

#include "tcgen05_utils.cuh"

namespace attn {

namespace tc {

constexpr int BM = 128;          // query rows per CTA
constexpr int BN = 128;          // keys per tile
constexpr int HD = 128;          // head_dim
constexpr int SUB_BYTES = 128 * 128;   // one [128 rows x 64 elements] swizzled sub-tile (16-bit elements)
constexpr int TILE_BYTES = 2 * SUB_BYTES;
constexpr int STAGES = 2;
struct Params {
    const int32_t* offsets;
    void* out;
    int B, H;
    int64_t n_tokens;
    int n_qtiles;
    float scale_log2;
    int out_f32;
    int32_t* err_flag;
    int* launch_abort;   // this launch's abort word (LaunchState::abort)
    int split_rows;      // query rows below this index in their sequence carry P as two terms (see `split`)
};

// =============================================================================================
// The pair kernel: two query tiles per CTA, P kept in tensor memory, O accumulated in tensor memory.
//
//   warps 0-3 / 4-7   softmax warpgroup 0 / 1, one 128-row query tile each (rows q0.. / q0+128..)
//   warp 8            TMA producer: both Q tiles, then K and V tiles into separate 2-stage rings
//   warps 10-11       idle (they complete the third warpgroup so that setmaxnreg can move registers)
//   warp 9            MMA issuer.  Per key tile j:  PV0_j, QK0_{j+1}, PV1_j, QK1_{j+1}, so that one
//                     warpgroup's softmax runs while the tensor pipe works for the other.
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512).  A thread reads its whole
// S row into registers (one wait), then overwrites the first 64 columns of the same S region with P
// in the input type, two per 32-bit column; the PV MMA takes A from tensor memory and B = V from
// shared memory.  O is
// accumulated by the MMA itself.  The running maximum used for P is only advanced when a row's
// new maximum exceeds it by more than 8 in the log2 domain, so P stays below 2^8; only then is O
// read back, scaled and written again (rare after the first tiles).  The true maximum never enters
// the result:
// O and l are consistent with the reference maximum, and O/l is formed in the epilogue.
// =============================================================================================
//
// `split`.  P is rounded to the input type for the P.V MMA: 2^-9 per probability for bf16.  Over
// many keys those roundings average out (for N(0,1) inputs the output error of a row with n visible
// keys is about 1.9e-3 / sqrt(n) rms), but the first rows of a sequence see only a few keys and
// reach 8e-3 max-abs, beyond the 2e-3 the fp16 path meets everywhere.  So the work item that holds
// a sequence's first 256 query rows writes P as TWO terms, hi = round(p) and lo = round(p - hi),
// and the MMA thread issues P.V for both (columns 0..63 and 64..127 of the S region): 2^-17 per
// probability there.  That item is 3 of a sequence's ~150 tile steps; the rest is unchanged.
// What remains for bf16 is the rounding of a single dominant probability: an outlier score in a
// row of a few hundred keys takes p ~ 0.3, and 0.3 * 2^-9 * |v| reaches 3.4e-3 (p99.9 is 4e-4).
// Params::split_rows = 256 is that default; a caller who wants 2e-3 everywhere asks for two terms
// on every row (split_rows = INT_MAX: half as many P.V MMAs again and a second pass over P).
constexpr int THREADS2 = 384;   // 3 warpgroups: softmax 0, softmax 1, {TMA, MMA, 2 idle warps}
// Registers per thread after setmaxnreg.  The CTA's pool is what it was launched with: 65536 / threads
// rounded down to a multiple of 8, times the thread count.  A setmaxnreg.inc that asks for more than
// the pool holds never returns (the kernel hangs), so the identity is checked here and not by trying.
constexpr int kRegsSoftmax2 = 216, kRegsOther2 = 72;     // 224 / 56 before: +1.6 %, the MMA thread spills less
static_assert(8 * 32 * kRegsSoftmax2 + 4 * 32 * kRegsOther2 <= THREADS2 * ((65536 / THREADS2) / 8 * 8),
              "setmaxnreg targets exceed the CTA's register pool");

// Staged read-out of an output tile (16-bit output, all 128 rows of the tile inside the sequence):
// the warpgroup packs its rows into a private 16 KB shared-memory buffer in the 128-byte-swizzled
// layout of a [128 rows x 64 columns] TMA box and one thread stores the box with
// cp.async.bulk.tensor (two boxes per tile).  Written straight from registers, every 16-byte store
// instruction of a warp touches 32 different rows, 8 KB apart: 32 sectors per instruction, about two
// thousand LSU clocks per tile, as long as a whole key-tile step; staged, it is a few hundred.
struct OutStage {
    unsigned char* buf;          // 16 KB, 1024-byte aligned, private to the warpgroup: 4 KB per warp
    const CUtensorMap* map;      // output tensor [n_tokens, H*128], box 32 columns x 32 rows, 64-byte swizzle
    int row0;                    // first row of the tile in the packed buffer
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(src)) : "memory");
}

// One softmax thread = one query row (TMEM lane) of a 128-row tile: walks the key tiles, turns S into
// P in place, keeps the running maximum lazily, and writes the normalised output row at the end.
// `qpos` is the row's position in key coordinates (keys 0..qpos are visible): its index within the
// sequence for the packed prefill, kv_len - q_len + index for a chunk over a cached prefix.
template <typename T, int kPolyOf8, bool kStaged>
__device__ __forceinline__ void softmax_row(unsigned long long* s_full, unsigned long long* p_half,
                                            unsigned long long* p_full,
                                            unsigned long long* o_full, uint32_t s_addr, uint32_t o_addr, int nk,
                                            int qpos, int r, const Params& p, AbortBox* wc,
                                            bool row_valid, int64_t out_row, int h, bool split, int c0 = 0,
                                            unsigned long long* o_free = nullptr, const OutStage* stage = nullptr) {
    // c0: tiles this warpgroup has processed before this call (persistent kernels keep their
    // barriers across work items, so the phase of tile j is (c0 + j) & 1); o_free, if given, is
    // signalled once the accumulator has been read out and may be overwritten by the next item.
    {
        float m_ref = -INFINITY, l = 0.f;
        // P <= 2^kLazy: far inside the range of fp16 and bf16, and O is rescaled rarely.
        constexpr float kLazy = 8.f;
        bool ok = true;
        for (int j = 0; j < nk; ++j) {
            if (!(ok = mbar_wait(s_full, (c0 + j) & 1, wc))) break;
            tc_fence_after();
            float sv[BN];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32_nowait(s_addr + c * 32, sv + c * 32);
            tmem_ld_wait();
            // key (j*BN + i) is visible to this row iff it is <= qpos (the row's position among the keys)
            const int lim = qpos - j * BN;
            if (lim < BN - 1) {
#pragma unroll
                for (int i = 0; i < BN; ++i)
                    if (i > lim) sv[i] = -INFINITY;
            }
            // eight independent chains, then a tree: a single 128-long dependent chain would cost
            // its full latency with only two softmax warps per scheduler to hide it
            float mx8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(sv[i], sv[8 + i]);
#pragma unroll
            for (int i = 16; i < BN; i += 16)
#pragma unroll
                for (int k = 0; k < 8; ++k) mx8[k] = max3(mx8[k], sv[i + k], sv[i + 8 + k]);
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                                   fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            const float m_new = fmaxf(m_ref, mx * p.scale_log2);
            // advance the reference maximum only when some row of the warp outgrew it by 2^8
            if (__any_sync(0xffffffffu, m_new > m_ref + kLazy)) {
                if (j > 0) {
                    const float alpha = fast_exp2(m_ref - m_new);
                    l *= alpha;
                    if (!(ok = mbar_wait(o_full, (c0 + j - 1) & 1, wc))) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float ov[32];
                        tmem_ld32(o_addr + c * 32, ov);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] *= alpha;
                        tmem_st32(o_addr + c * 32, reinterpret_cast<const uint32_t*>(ov));
                    }
                    tmem_st_wait();
                }
                m_ref = m_new;
            }
            // P = 2^(s*scale - m_ref), rounded to the input type.  (fp16 inputs once took the packed
            // ex2.approx.f16x2 with fp16 row sums: its two results per operation cost the
            // special-function unit as much as two fp32 ex2, and the fp32 form measured 842 against
            // 756 TFLOP/s.)
            float rs = 0.f;
            {
                // fp32 ex2, the remaining fp32 arithmetic as packed pairs (f32x2).  A
                // warp's 128 exponentials occupy the special-function unit for 1024 clocks (4 lanes
                // per clock per scheduler), so kPolyOf8 of every 8 elements take a cubic on the
                // FMA pipe instead (2 in the packed kernels; 0 in the paged kernel, whose gather warps
                // share the schedulers: measured 895 against 820 TFLOP/s).
                float rs4[4] = {0.f, 0.f, 0.f, 0.f};
                const float nm = -m_ref;
                // the four probabilities of elements c*64 + i .. + 3; the second pass of `split` calls
                // this again and must get the very same bits (hi is re-derived there from p)
                auto probs4 = [&](int c, int i, float& p0, float& p1, float& p2, float& p3) {
                    float x0, x1, x2, x3;
                    fma2(x0, x1, sv[c * 64 + i], sv[c * 64 + i + 1], p.scale_log2, p.scale_log2, nm, nm);
                    fma2(x2, x3, sv[c * 64 + i + 2], sv[c * 64 + i + 3], p.scale_log2, p.scale_log2, nm, nm);
                    p0 = fast_exp2(x0);
                    p1 = fast_exp2(x1);
                    if (kPolyOf8 == 4 || (kPolyOf8 == 2 && (i & 4)) || (kPolyOf8 == 1 && (i & 12) == 12)) {
                        exp2_poly2(p2, p3, x2, x3);
                    } else {
                        p2 = fast_exp2(x2);
                        p3 = fast_exp2(x3);
                    }
                };
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t pk[32];
#pragma unroll
                    for (int i = 0; i < 64; i += 4) {
                        float p0, p1, p2, p3;
                        probs4(c, i, p0, p1, p2, p3);
                        add2(rs4[0], rs4[1], rs4[0], rs4[1], p0, p1);
                        add2(rs4[2], rs4[3], rs4[2], rs4[3], p2, p3);
                        pk[i >> 1] = pack2<T>(p0, p1);
                        pk[(i >> 1) + 1] = pack2<T>(p2, p3);
                    }
                    tmem_st32(s_addr + c * 32, pk);
                    if (c == 0 && p_half) {
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(p_half);
                    }
                }
                if (split) {
                    // Second term of P for rows with few visible keys (see the note on `split` above
                    // the kernels): lo = p - hi with hi = round(p) exactly as stored above, rounded to
                    // the input type, into columns 64..127 of the S region (free: the whole S row is in
                    // registers).  Cold path: the first item of a sequence, or every item on request.
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t pk[32];
#pragma unroll
                        for (int i = 0; i < 64; i += 4) {
                            float p0, p1, p2, p3, h0, h1, h2, h3;
                            probs4(c, i, p0, p1, p2, p3);
                            unpack2(pack2<T>(p0, p1), T(), h0, h1);
                            unpack2(pack2<T>(p2, p3), T(), h2, h3);
                            pk[i >> 1] = pack2<T>(p0 - h0, p1 - h1);
                            pk[(i >> 1) + 1] = pack2<T>(p2 - h2, p3 - h3);
                        }
                        tmem_st32(s_addr + 64 + c * 32, pk);
                    }
                }
                rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            }
            l += rs;
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(p_full);
        }
        if (ok && nk > 0) ok = mbar_wait(o_full, (c0 + nk - 1) & 1, wc);
        if (ok && nk > 0) {
            tc_fence_after();
            const bool valid = row_valid;
            const float inv = 1.f / l;
            const int64_t row = out_row;
            if (kStaged && stage->buf) {
                // Whole tile inside the sequence, 16-bit output: through shared memory and TMA, every
                // warp by itself.  A warp's 4 KB of staging are two buffers of [32 rows x 32
                // columns]; the row's four quarters go through them in turn, each followed by the
                // warp's own TMA store, and a buffer is rewritten once the store that read it two
                // quarters earlier has finished reading (cp.async.bulk.wait_group.read 1).  Nothing
                // waits for the last two stores here: the next read-out (or the end of the kernel)
                // does.  No barrier across warps is involved.
                float ov[HD];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32_nowait(o_addr + c * 32, ov + c * 32);
                tmem_ld_wait();
                if (o_free) {                  // the accumulator is in registers: the next item may overwrite it
                    tc_fence_before();
                    mbar_arrive(o_free);
                }
                const int lr = r & 31, wq = (r >> 5) & 3;
                unsigned char* const wbuf = stage->buf + wq * 4096;
                if (lr == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous read-out's stores
                __syncwarp();
#pragma unroll
                for (int qt = 0; qt < 4; ++qt) {
                    unsigned char* const sub = wbuf + (qt & 1) * 2048;
                    if (qt >= 2) {
                        if (lr == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        __syncwarp();
                    }
                    const uint32_t sbase = smem_u32(sub) + (uint32_t)lr * 64u;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {              // 16-byte chunk c of this row's 32 columns
                        const float* o8 = ov + qt * 32 + c * 8;
                        const uint32_t dst = sbase + (uint32_t)((c ^ ((lr >> 1) & 3)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                     "r"(pack2<T>(o8[0] * inv, o8[1] * inv)), "r"(pack2<T>(o8[2] * inv, o8[3] * inv)),
                                     "r"(pack2<T>(o8[4] * inv, o8[5] * inv)), "r"(pack2<T>(o8[6] * inv, o8[7] * inv))
                                     : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lr == 0) {
                        tma_store_2d(stage->map, sub, h * HD + qt * 32, stage->row0 + wq * 32);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float ov[32];
                tmem_ld32(o_addr + c * 32, ov);
                if (c == 3 && o_free) {        // the accumulator is in registers: the next item may overwrite it
                    tc_fence_before();
                    mbar_arrive(o_free);
                }
                if (!valid) continue;
                if (p.out_f32) {
                    float4* dst = reinterpret_cast<float4*>((float*)p.out + (row * p.H + h) * HD + c * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dst[i] = make_float4(ov[4 * i] * inv, ov[4 * i + 1] * inv, ov[4 * i + 2] * inv, ov[4 * i + 3] * inv);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>((T*)p.out + (row * p.H + h) * HD + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        dst[i] = make_uint4(pack2<T>(ov[8 * i] * inv, ov[8 * i + 1] * inv),
                                            pack2<T>(ov[8 * i + 2] * inv, ov[8 * i + 3] * inv),
                                            pack2<T>(ov[8 * i + 4] * inv, ov[8 * i + 5] * inv),
                                            pack2<T>(ov[8 * i + 6] * inv, ov[8 * i + 7] * inv));
                }
            }
            }
        }
        }
}

// =============================================================================================
// Persistent form of the pair kernel.
//
// The pair kernel spends about two of a CTA's ~ten key-tile periods outside its steady state: set-up and
// the first TMA round trip before any softmax can run, the read-out of O at the end, and the last
// key tile of the pair, which only the upper query tile needs (the other warpgroup idles).  Here
// the grid is one CTA per SM and every CTA walks work items (a pair of query tiles of one
// (sequence, head)), heaviest pairs first, handed out by an atomic counter: the producer thread
// draws the next non-empty item and publishes it to the other roles through a 4-deep ring in
// shared memory.  Barriers, tensor memory and the K/V rings live across items; every role keeps
// running counters for the barrier phases.
//
// One MMA thread serves the two warpgroups in a fixed alternating order (P.V_a, Q.K_a', P.V_b,
// Q.K_b'), which keeps one warpgroup's softmax over the other's MMAs.  The last key tile of an
// item is needed by the upper query tile only; the warpgroup with the lower tile has finished, and
// the first Q.K of its tile in the NEXT item is issued at that moment (its Q tile and the first K
// tile of the next item are fetched ahead for this), so it runs one key tile ahead.  The two query
// tiles of a pair are given to the warpgroups in alternating order from item to item: the early
// starter takes the upper tile, which has one key tile more, and both finish together.
// =============================================================================================

// Per-launch state in global memory: the work counter of the persistent kernel and the abort word
// that a CTA sets when one of its bounded waits runs out.  Launches in flight at the same time (on
// different streams) must not share a slot, so each launch takes the next of kLaunchSlots slots in
// rotation and zeroes it on its own stream.
struct LaunchState {
    unsigned long long work;
    int abort;
    int pad;
};
constexpr int kLaunchSlots = 64;
static __device__ LaunchState g_launch[kLaunchSlots];

struct Item2p {
    int tp, h, b, L, q0, n0, n1, nmax;
    int t0;            // index of the lower query tile (the upper one, if any, is t0 + 1)
    int64_t seq_beg;
    bool valid;
};

struct SmemLayout2p {
    alignas(1024) unsigned char q[2][TILE_BYTES];
    alignas(1024) unsigned char k[STAGES][TILE_BYTES];
    alignas(1024) unsigned char v[STAGES][TILE_BYTES];
    alignas(1024) unsigned char o_stage[2][SUB_BYTES];     // output staging, one [128 x 64] box per warpgroup
    alignas(8) unsigned long long q_full[2], q_empty[2];
    // item[n & 3] = n-th item of this CTA, decoded (tp < 0: no more work), published by the producer:
    // the other roles start an item from shared memory and never wait for the offsets to come from
    // global memory.  The producer draws item n only after it has issued every K/V tile of item
    // n-1, which needs both streams and therefore both softmax warpgroups to be inside item n-1 or
    // later; slot n & 3 was last read at the start of item n-4, so it is free.
    unsigned long long item_full[4];
    Item2p item[4];
    unsigned long long s_full[2], p_half[2], p_full[2], o_full[2], o_free[2];
    unsigned long long k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    unsigned int tmem_base;
    AbortBox box;
};

// Work item -> (pair index, head, sequence).  (sequence, head) combinations are taken in groups of
// ITEM_GROUP; inside a group the pair index is the slowest coordinate, so the heaviest pairs of the
// group come first while the CTAs running at any moment share the K/V of a few dozen (sequence,
// head) combinations, which stay in L2 (with the pair index slowest over ALL combinations every CTA
// would stream its own K/V from DRAM: measured 814 against 960 TFLOP/s).
//
// Pairing.  A sequence of nq query tiles is cut into pairs from its END: with nq odd, pair 0 is tile 0
// alone and pair tp >= 1 holds tiles 2 tp - 1 and 2 tp; with nq even pair tp holds tiles 2 tp and
// 2 tp + 1.  The tile without a partner keeps one warpgroup idle for as many rounds as it has key
// tiles: one round for tile 0, but nq rounds for the last tile, which is where pairing from the start
// would leave it (3.4 % of the workload's rounds).  A sequence longer than the caller's max_seqlen is
// paired from the start, so that the rows covered are the first n_qtiles pairs' as the zero-fill of
// the rest assumes.
constexpr int ITEM_GROUP = 16;
__device__ __forceinline__ Item2p decode_item(const Params& p, int64_t id) {
    Item2p it;
    const int per_group = p.n_qtiles * ITEM_GROUP;
    const int grp = (int)(id / per_group), r = (int)(id - (int64_t)grp * per_group);
    const int x = r / ITEM_GROUP, hb = grp * ITEM_GROUP + (r - x * ITEM_GROUP);
    it.tp = p.n_qtiles - 1 - x;
    it.valid = true;
    if (hb >= p.H * p.B) {          // padding of the last group: an empty item
        it.L = 0; it.q0 = 1; it.b = it.h = 0; it.n0 = it.n1 = it.nmax = 0; it.seq_beg = 0; it.t0 = 0;
        return it;
    }
    it.b = hb / p.H;
    it.h = hb - it.b * p.H;
    it.seq_beg = it.b ? p.offsets[it.b - 1] : 0;
    const int64_t seq_end = p.offsets[it.b];
    it.valid = !(it.seq_beg < 0 || seq_end < it.seq_beg || seq_end > p.n_tokens);
    it.L = it.valid ? (int)(seq_end - it.seq_beg) : 0;
    const int nq = (it.L + BM - 1) / BM;                     // query (and key) tiles of the sequence
    const int odd = it.L <= p.n_qtiles * 2 * BM ? (nq & 1) : 0;
    it.t0 = it.tp == 0 ? 0 : 2 * it.tp - odd;
    const int t1 = 2 * it.tp + 1 - odd;                      // upper tile (tp = 0 of an odd count: none)
    it.q0 = it.t0 * BM;
    it.n0 = it.t0 < nq ? it.t0 + 1 : 0;                      // key tiles of the lower query tile (0: no such tile)
    it.n1 = (t1 > it.t0 && t1 < nq) ? t1 + 1 : 0;            // of the upper one (0: none)
    it.nmax = it.n1 > it.n0 ? it.n1 : it.n0;
    return it;
}
// In the CTA's n-th item warpgroup w takes the upper query tile iff (w ^ n) & 1.
__device__ __forceinline__ int upper_of(int w, int n) { return (w ^ n) & 1; }

template <typename T>
__global__ void __launch_bounds__(THREADS2, 1)
prefill_tc2p_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                    const Params p, const int64_t n_items, unsigned long long* work_counter) {
    extern __shared__ unsigned char smem_raw[];
    SmemLayout2p& sm = *reinterpret_cast<SmemLayout2p*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (*(volatile int*)p.launch_abort) return;
    AbortBox* const wc = &sm.box;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&sm.item_full[i], 1);
        for (int w = 0; w < 2; ++w) {
            mbar_init(&sm.q_full[w], 1);
            mbar_init(&sm.q_empty[w], 1);
            mbar_init(&sm.s_full[w], 1);
            mbar_init(&sm.p_half[w], 128);
            mbar_init(&sm.p_full[w], 128);
            mbar_init(&sm.o_full[w], 1);
            mbar_init(&sm.o_free[w], 128);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        sm.box.abort = 0;
        sm.box.launch_abort = p.launch_abort;
        sm.box.err_flag = p.err_flag;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    // producer bookkeeping for the drain on abort: K/V tiles and Q tiles issued in total
    int g_issued_k = 0, g_issued_v = 0, q_issued[2] = {0, 0};
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther2));
    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int g = 0;        // key tiles issued so far (all items): ring stage g & 1, use (g >> 1)
            int n_it = 0;     // items published so far
            bool ok = true;
            while (ok) {
                // draw the next non-empty item (empty ones: pairs past the end of a short sequence)
                Item2p it = {};
                long long id;
                do {
                    id = (long long)atomicAdd(work_counter, 1ull);
                    if (id >= n_items) { id = -1; break; }
                    it = decode_item(p, id);
                    if (!it.valid && p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
                } while (!it.valid || it.n0 == 0);
                if (id < 0) it.tp = -1;
                sm.item[n_it & 3] = it;
                mbar_arrive(&sm.item_full[n_it & 3]);
                if (id < 0) break;
                const int col0 = it.h * HD;
                auto load_q = [&](int w) -> bool {       // query tile of warpgroup w, once its buffer is free
                    const int u = upper_of(w, n_it);
                    if ((u ? it.n1 : it.n0) == 0) return true;
                    if (q_issued[w] > 0 && !mbar_wait(&sm.q_empty[w], (q_issued[w] - 1) & 1, wc)) return false;
                    const int row = (int)(it.seq_beg + it.q0 + u * BM);
                    mbar_expect_tx(&sm.q_full[w], TILE_BYTES);
                    tma_load_2d(sm.q[w], &map_q, col0, row, &sm.q_full[w]);
                    tma_load_2d(sm.q[w] + SUB_BYTES, &map_q, col0 + 64, row, &sm.q_full[w]);
                    ++q_issued[w];
                    return true;
                };
                // The warpgroup that had the lower tile in the previous item (and takes the upper
                // one now) finished first: its Q buffer is free first, and it starts this item
                // first.  Order: its Q, K tile 0, the other Q, V tile 0, then the remaining tiles.
                const int w_first = (n_it & 1) ? 0 : 1;      // upper_of(w_first, n_it) == 1
                if (!(ok = load_q(w_first))) break;
                for (int j = 0; j < it.nmax; ++j, ++g) {
                    const int s = g & 1;
                    const uint32_t ph = ((g - STAGES) >> 1) & 1;
                    const int row = (int)(it.seq_beg + (int64_t)j * BN);
                    if (g >= STAGES && !(ok = mbar_wait(&sm.k_empty[s], ph, wc))) break;
                    mbar_expect_tx(&sm.k_full[s], TILE_BYTES);
                    tma_load_2d(sm.k[s], &map_k, col0, row, &sm.k_full[s]);
                    tma_load_2d(sm.k[s] + SUB_BYTES, &map_k, col0 + 64, row, &sm.k_full[s]);
                    g_issued_k = g + 1;
                    if (j == 0 && !(ok = load_q(w_first ^ 1))) break;
                    if (g >= STAGES && !(ok = mbar_wait(&sm.v_empty[s], ph, wc))) break;
                    mbar_expect_tx(&sm.v_full[s], TILE_BYTES);
                    tma_load_2d(sm.v[s], &map_v, col0, row, &sm.v_full[s]);
                    tma_load_2d(sm.v[s] + SUB_BYTES, &map_v, col0 + 64, row, &sm.v_full[s]);
                    g_issued_v = g + 1;
                }
                ++n_it;
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
        constexpr uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);
        constexpr uint32_t idesc_pv = idesc_qk | (1u << 16);
        if (elect_one()) {
            const uint64_t qd[2] = {smem_desc(smem_u32(sm.q[0]), 16, 1024), smem_desc(smem_u32(sm.q[1]), 16, 1024)};
            const uint64_t kd[2] = {smem_desc(smem_u32(sm.k[0]), 16, 1024), smem_desc(smem_u32(sm.k[1]), 16, 1024)};
            const uint64_t vd[2] = {smem_desc(smem_u32(sm.v[0]), SUB_BYTES, 1024), smem_desc(smem_u32(sm.v[1]), SUB_BYTES, 1024)};
            auto issue_qk = [&](int w, int stage) {      // S_w = Q_w K^T, K in ring stage `stage`
                const uint64_t a = qd[w], b2 = kd[stage];
                const uint32_t d = tmem + w * 128;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t off16 = ((kk >> 2) * SUB_BYTES + (kk & 3) * 32) >> 4;
                    umma_f16(d, a + off16, b2 + off16, idesc_qk, kk > 0);
                }
                umma_commit(&sm.s_full[w]);
            };
            // O_w (+)= P_w V, 64 keys per call; with `split` the second call adds the lo term of all 128 keys
            auto issue_pv = [&](int w, int stage, int half, bool first, bool split) {
                const uint64_t b2 = vd[stage];
                const uint32_t d = tmem + 256 + w * 128, a = tmem + w * 128;
#pragma unroll
                for (int k4 = 0; k4 < BN / 32; ++k4) {
                    const int kk = half * (BN / 32) + k4;
                    umma_f16_ts(d, a + kk * 8, b2 + ((kk * 2048) >> 4), idesc_pv, (!first || kk > 0) ? 1u : 0u);
                }
                if (half && split) {        // cold path: a rolled loop keeps the issuing thread's register count down
#pragma unroll 1
                    for (int kk = 0; kk < BN / 16; ++kk)
                        umma_f16_ts(d, a + 64 + kk * 8, b2 + (uint64_t)(kk * (2048 >> 4)), idesc_pv, 1u);
                }
                if (half) umma_commit(&sm.o_full[w]);
            };
            int g = 0, n = 0;
            int c[2] = {0, 0};        // tiles processed per warpgroup (phase of s_full / p_half / p_full / o_full)
            int uses[2] = {0, 0};     // items in which the warpgroup had work (phase of q_full / o_free)
            bool early = false;       // the upper tile's first Q.K of item n was issued during item n-1
            bool ok = true;
            while (ok) {
                if (!(ok = mbar_wait_spin(&sm.item_full[n & 3], (n >> 2) & 1, wc))) break;
                const Item2p it = sm.item[n & 3];
                if (it.tp < 0) break;
                // Within an item the warpgroup with the upper query tile is served first in every
                // round: it has one key tile more and (after an early start) is one tile ahead.
                const int wu = (n & 1) ? 0 : 1, wl = wu ^ 1;
                int nw[2];
                nw[wu] = it.n1;
                nw[wl] = it.n0;
                if (!(ok = mbar_wait_spin(&sm.k_full[g & 1], (g >> 1) & 1, wc))) break;
                if (it.n1 > 0 && !early) {
                    if (!(ok = mbar_wait_spin(&sm.q_full[wu], uses[wu] & 1, wc))) break;
                    tc_fence_after();
                    issue_qk(wu, g & 1);
                }
                if (!(ok = mbar_wait_spin(&sm.q_full[wl], uses[wl] & 1, wc))) break;
                tc_fence_after();
                issue_qk(wl, g & 1);
                umma_commit(&sm.k_empty[g & 1]);
                if (it.n0 == 1) umma_commit(&sm.q_empty[wl]);
                early = false;
                for (int j = 0; ok && j < it.nmax; ++j) {
                    const int s = (g + j) & 1;
                    const uint32_t ph = ((g + j) >> 1) & 1;
                    if (j == it.nmax - 1 && it.n1 > 0) {
                        // Last key tile: only the upper query tile needs it.  The other warpgroup
                        // takes the upper tile of the next item: start that item's first Q.K now
                        // if the item, its Q tile and its first K tile are already there.  (Polling
                        // for them while waiting for P, and a second MMA thread so that each
                        // warpgroup advances by itself, were both measured: short sequences gain,
                        // but the alternation of the two warpgroups is lost and long ones lose more.)
                        const int G1 = g + it.nmax;
                        if (mbar_test(&sm.item_full[(n + 1) & 3], ((n + 1) >> 2) & 1)) {
                            if (sm.item[(n + 1) & 3].tp >= 0 && sm.item[(n + 1) & 3].n1 > 0 && mbar_test(&sm.q_full[wl], (uses[wl] + 1) & 1) &&
                                mbar_test(&sm.k_full[G1 & 1], (G1 >> 1) & 1)) {
                                tc_fence_after();
                                issue_qk(wl, G1 & 1);
                                early = true;
                            }
                        }
                    }
                    for (int t = 0; t < 2 && ok; ++t) {
                        const int w = t ? wl : wu;
                        if (j < nw[w]) {
                            if (j == 0 && uses[w] > 0) {     // the previous item's O must have been read out
                                if (!(ok = mbar_wait_spin(&sm.o_free[w], (uses[w] - 1) & 1, wc))) break;
                            }
                            if (!(ok = mbar_wait_spin(&sm.p_half[w], (c[w] + j) & 1, wc))) break;
                            if (t == 0 || j >= nw[wu]) { if (!(ok = mbar_wait_spin(&sm.v_full[s], ph, wc))) break; }
                            tc_fence_after();
                            issue_pv(w, s, 0, j == 0, false);
                            if (!(ok = mbar_wait_spin(&sm.p_full[w], (c[w] + j) & 1, wc))) break;
                            tc_fence_after();
                            issue_pv(w, s, 1, j == 0, it.q0 < p.split_rows);
                        }
                        if (t == 1) umma_commit(&sm.v_empty[s]);
                        if (j + 1 < nw[w]) {
                            const int s1 = (g + j + 1) & 1;
                            if (t == 0 || j + 1 >= nw[wu]) {
                                if (!(ok = mbar_wait_spin(&sm.k_full[s1], ((g + j + 1) >> 1) & 1, wc))) break;
                            }
                            tc_fence_after();
                            issue_qk(w, s1);
                            if (j + 2 == nw[w]) umma_commit(&sm.q_empty[w]);     // last Q.K of this warpgroup's tile
                        }
                        if (t == 1 && j + 1 < it.nmax) umma_commit(&sm.k_empty[(g + j + 1) & 1]);
                    }
                }
                for (int w = 0; w < 2; ++w) {
                    c[w] += nw[w];
                    uses[w] += nw[w] > 0;
                }
                g += it.nmax;
                ++n;
            }
        }
        __syncwarp();
    }
    } else {
        // ------------------------------------------------------------------ softmax warpgroups
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax2));
        const int w = warp >> 2;
        const int r = threadIdx.x & 127;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + w * 128, o_addr = lane_base + 256 + w * 128;
        int c0 = 0;
        for (int n_it = 0;; ++n_it) {
            if (!mbar_wait(&sm.item_full[n_it & 3], (n_it >> 2) & 1, wc)) break;
            const Item2p it = sm.item[n_it & 3];
            if (it.tp < 0) break;
            if (wc->abort) break;
            const int u = upper_of(w, n_it);
            const int nk = u ? it.n1 : it.n0;
            if (nk == 0) continue;
            const int tq = it.t0 + u;
            // staged read-out when the tile lies wholly inside the sequence and the output is 16-bit
            const bool whole = it.q0 + u * BM + BM <= it.L && !p.out_f32;
            const OutStage stage{whole ? sm.o_stage[w] : nullptr, &map_o, (int)(it.seq_beg + it.q0 + u * BM)};
            softmax_row<T, 2, true>(&sm.s_full[w], &sm.p_half[w], &sm.p_full[w], &sm.o_full[w], s_addr, o_addr, nk, tq * BM + r, r, p,
                              wc, it.q0 + u * BM + r < it.L, it.seq_beg + it.q0 + u * BM + r, it.h, it.q0 < p.split_rows, c0,
                              &sm.o_free[w], &stage);
            c0 += nk;
        }
        // the staged read-out leaves its last stores in flight: shared memory stays until they have read it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    // ---------------------------------------------------------------------- teardown
    if (warp == 8 && lane == 0 && sm.box.abort) {
        // give the copies still in flight a bounded time to land before shared memory is released
        const long long t0 = clock64();
        for (int w = 0; w < 2; ++w)
            if (q_issued[w] > 0) while (!mbar_try(&sm.q_full[w], (q_issued[w] - 1) & 1) && clock64() - t0 < WAIT_CYCLES) {}
        for (int gg = g_issued_k > STAGES ? g_issued_k - STAGES : 0; gg < g_issued_k; ++gg)
            while (!mbar_try(&sm.k_full[gg & 1], (gg >> 1) & 1) && clock64() - t0 < WAIT_CYCLES) {}
        for (int gg = g_issued_v > STAGES ? g_issued_v - STAGES : 0; gg < g_issued_v; ++gg)
            while (!mbar_try(&sm.v_full[gg & 1], (gg >> 1) & 1) && clock64() - t0 < WAIT_CYCLES) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}


// =============================================================================================
// Paged form of the pair kernel: the K and V tiles are GATHERED through the slot table.
//
// Chunked / prefix-cached prefill: sequence b's query rows are its last q_len tokens (packed in q),
// its keys are the pool rows slots[kv_beg .. kv_beg + kv_len) (prefix and chunk); query i sees key
// j iff j <= kv_len - q_len + i.  Everything downstream of shared memory is the pair kernel (two query
// tiles per CTA, S -> P in tensor memory, O accumulated by the MMA).  What changes is the producer
// of K/V: a fourth warpgroup (warps 12-13 for K, 14-15 for V) copies the 128 rows of a tile with
// 16-byte cp.async (16 consecutive lanes = one 256-byte row, so a warp instruction reads two whole
// rows) into the same 128-byte-swizzled layout TMA would have produced; rows past the end of the
// sequence are zero-filled.  The 16 lanes of a row need the same slots: each loads and checks two
// of the group's 32 slots per tile and the copies take them by shuffle (with every lane loading
// and checking all 32 itself the gather warps' instructions slowed the softmax warps on the same
// schedulers: 686 against 895 TFLOP/s).  A tile is published (fence.proxy.async + mbarrier arrive by the
// stream's 64 threads) once it has landed.  Grouped-query heads: query head h reads KV head h / (H / Hkv).
// =============================================================================================
constexpr int THREADS_PG = 512;
constexpr int kRegsSoftmaxPg = 208, kRegsOtherPg = 56, kRegsGatherPg = 40;     // 200 / 56 / 56 before: +1.1 %
static_assert(8 * 32 * kRegsSoftmaxPg + 4 * 32 * kRegsOtherPg + 4 * 32 * kRegsGatherPg <=
                  THREADS_PG * ((65536 / THREADS_PG) / 8 * 8),
              "setmaxnreg targets exceed the CTA's register pool");
constexpr int KSTAGES_PG = 2;    // K tiles in flight (3 fit in shared memory and were measured: 854 against 935 TFLOP/s)

struct PagedTcParams {
    const int32_t* slots;
    const int32_t* kv_offsets;
    const int32_t* q_offsets;
    const void* k_cache;
    const void* v_cache;
    int Hkv;
    int64_t n_kv_tokens, n_slots;
};

struct SmemLayoutPg {
    alignas(1024) unsigned char q[2][TILE_BYTES];
    alignas(1024) unsigned char k[KSTAGES_PG][TILE_BYTES];
    alignas(1024) unsigned char v[STAGES][TILE_BYTES];
    alignas(8) unsigned long long q_full;
    unsigned long long s_full[2], p_half[2], p_full[2], o_full[2];
    unsigned long long k_full[KSTAGES_PG], k_empty[KSTAGES_PG], v_full[STAGES], v_empty[STAGES];
    unsigned int tmem_base;
    AbortBox box;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(THREADS_PG, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const Params p, const PagedTcParams pg) {
    extern __shared__ unsigned char smem_raw[];
    SmemLayoutPg& sm = *reinterpret_cast<SmemLayoutPg*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int tp = p.n_qtiles - 1 - (int)blockIdx.x;       // pair of query tiles, late pairs first
    const int64_t q_beg = b ? pg.q_offsets[b - 1] : 0, q_end = pg.q_offsets[b];
    const int64_t kv_beg = b ? pg.kv_offsets[b - 1] : 0, kv_end = pg.kv_offsets[b];
    if (q_beg < 0 || q_end < q_beg || q_end > p.n_tokens || kv_beg < 0 || kv_end < kv_beg ||
        kv_end > pg.n_kv_tokens || (kv_end - kv_beg) < (q_end - q_beg)) {
        if (p.err_flag && threadIdx.x == 0) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
        return;
    }
    const int q_len = (int)(q_end - q_beg), kv_len = (int)(kv_end - kv_beg);
    const int q0 = tp * 2 * BM;
    if (q0 >= q_len) return;
    if (*(volatile int*)p.launch_abort) return;
    const int shift = kv_len - q_len;
    // key tiles per warpgroup: up to the tile that holds its last row's last visible key
    auto tiles_for = [&](int w) {
        const int first = q0 + w * BM;
        if (first >= q_len) return 0;
        const int last = first + BM - 1 < q_len - 1 ? first + BM - 1 : q_len - 1;
        return (shift + last) / BN + 1;
    };
    const int n0 = tiles_for(0), n1 = tiles_for(1);
    const int nmax = n1 > n0 ? n1 : n0;
    AbortBox* const wc = &sm.box;
    // two-term P where rows see few keys: the chunk's first 256 rows, unless a prefix of >= 256
    // cached tokens already gives every row that many keys
    const bool split = tp == 0 && shift < 2 * BM;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int w = 0; w < 2; ++w) {
            mbar_init(&sm.s_full[w], 1);
            mbar_init(&sm.p_half[w], 128);
            mbar_init(&sm.p_full[w], 128);
            mbar_init(&sm.o_full[w], 1);
        }
        for (int s = 0; s < KSTAGES_PG; ++s) {
            mbar_init(&sm.k_full[s], 64);
            mbar_init(&sm.k_empty[s], 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.v_full[s], 64);
            mbar_init(&sm.v_empty[s], 1);
        }
        sm.box.abort = 0;
        sm.box.launch_abort = p.launch_abort;
        sm.box.err_flag = p.err_flag;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    // Registers: launched with 128 per thread (16 warps); 8 * 208 (softmax) + 4 * 56 (TMA, MMA) + 4 * 40
    // (gather) = 16 * 128.  (200 / 56 / 56 before: +1.1 %, the softmax row spills less.)
    if (warp >= 12) {
        // ------------------------------------------------------------------ gather producers
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsGatherPg));
        // Two independent streams: warps 12-13 copy the K tiles, warps 14-15 the V tiles.  Each
        // stream loops  wait for its stage -> issue the tile's copies -> wait for them -> publish
        // (fence.proxy.async + arrive by its 64 threads), so K_j is on its way as soon as
        // Q*K(j-2) has finished and never waits behind a V stage.
        const int tid = threadIdx.x - 384;
        const bool v_stream = tid >= 64;
        const int t64 = tid & 63;
        const int c = t64 & 15, rsub = t64 >> 4;              // 16-byte chunk of a row, row within a pass (4 rows)
        const int hk = h / (p.H / pg.Hkv);
        const int64_t row_bytes = (int64_t)pg.Hkv * HD * 2;
        const char* base = (const char*)(v_stream ? pg.v_cache : pg.k_cache) + (int64_t)hk * HD * 2 + c * 16;
        const uint32_t dst_off = (c >> 3) * SUB_BYTES;
        unsigned long long* full = v_stream ? sm.v_full : sm.k_full;
        unsigned long long* empty = v_stream ? sm.v_empty : sm.k_empty;
        unsigned char (*stage)[TILE_BYTES] = v_stream ? sm.v : sm.k;
        const int n_stages = v_stream ? STAGES : KSTAGES_PG;
        // A thread copies chunk c of the 32 rows q*4 + rsub (q = 0..31) of a tile.  The 16 threads
        // of a row group need the same 32 slots: thread c loads and checks the slots of rows q = c
        // and q = c + 16 (ahead of the wait for the stage), and the copies take them from there by
        // shuffle, which keeps the gather's share of the schedulers' issue slots small.
        auto tile_slots = [&](int j, int& sa, int& sb) {
            bool bad = false;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int kvpos = j * BN + (c + 16 * i) * 4 + rsub;
                const bool live = kvpos < kv_len;
                const int v = live ? __ldg(pg.slots + kv_beg + kvpos) : -1;
                const bool in_range = v >= 0 && v < pg.n_slots;
                bad |= live && !in_range;
                (i ? sb : sa) = in_range ? v : -1;
            }
            if (bad && p.err_flag) atomicOr(p.err_flag, ATTN_B200_FLAG_BAD_SLOT);
        };
        // destination of row q*4 + rsub, chunk c, in the 128-byte-swizzled tile: the row's low three
        // bits are (q&1)*4 + rsub, so there are only two swizzle terms per thread and everything
        // else is a compile-time offset
        const uint32_t swz_even = rsub * 128 + ((((uint32_t)c & 7) ^ (uint32_t)rsub) << 4);
        const uint32_t swz_odd = rsub * 128 + ((((uint32_t)c & 7) ^ (uint32_t)(4 + rsub)) << 4);
        bool ok = true;
        for (int j = 0; j < nmax; ++j) {
            const int s = j % n_stages;
            int sa, sb;
            tile_slots(j, sa, sb);
            if (j >= n_stages) ok = mbar_wait(&empty[s], ((j - n_stages) / n_stages) & 1, wc);
            if (!__all_sync(0xffffffffu, ok)) break;
            const uint32_t sbase = smem_u32(stage[s]) + dst_off;
            const uint32_t be = sbase + swz_even, bo = sbase + swz_odd;
#pragma unroll
            for (int q = 0; q < 32; ++q) {
                const int v = __shfl_sync(0xffffffffu, q < 16 ? sa : sb, q & 15, 16);
                const uint32_t dst = ((q & 1) ? bo : be) + (uint32_t)q * 512u;
                cp_async16(dst, base + (int64_t)(v >= 0 ? v : 0) * row_bytes, v >= 0 ? 16 : 0);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&full[s]);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOtherPg));
        if (warp == 8) {
            // -------------------------------------------------------------- TMA: the two Q tiles
            if (lane == 0) {
                const int col0 = h * HD;
                mbar_expect_tx(&sm.q_full, 2 * TILE_BYTES);
                for (int w = 0; w < 2; ++w) {
                    tma_load_2d(sm.q[w], &map_q, col0, (int)(q_beg + q0 + w * BM), &sm.q_full);
                    tma_load_2d(sm.q[w] + SUB_BYTES, &map_q, col0 + 64, (int)(q_beg + q0 + w * BM), &sm.q_full);
                }
            }
        } else if (warp == 9) {
            // -------------------------------------------------------------- MMA issuer
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);
            constexpr uint32_t idesc_pv = idesc_qk | (1u << 16);
            const int nw[2] = {n0, n1};
            if (elect_one()) {
                const uint64_t qd[2] = {smem_desc(smem_u32(sm.q[0]), 16, 1024), smem_desc(smem_u32(sm.q[1]), 16, 1024)};
                const uint64_t kd[KSTAGES_PG] = {smem_desc(smem_u32(sm.k[0]), 16, 1024), smem_desc(smem_u32(sm.k[1]), 16, 1024)};
                const uint64_t vd[2] = {smem_desc(smem_u32(sm.v[0]), SUB_BYTES, 1024), smem_desc(smem_u32(sm.v[1]), SUB_BYTES, 1024)};
                auto issue_qk = [&](int w, int j) {
                    const uint64_t a = qd[w], b2 = kd[j % KSTAGES_PG];
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        const uint32_t off16 = ((kk >> 2) * SUB_BYTES + (kk & 3) * 32) >> 4;
                        umma_f16(tmem + w * 128, a + off16, b2 + off16, idesc_qk, kk > 0);
                    }
                    umma_commit(&sm.s_full[w]);
                };
                auto issue_pv = [&](int w, int j, int half) {
                    const uint64_t b2 = vd[j & 1];
                    const uint32_t d = tmem + 256 + w * 128, a = tmem + w * 128;
#pragma unroll
                    for (int k4 = 0; k4 < BN / 32; ++k4) {
                        const int kk = half * (BN / 32) + k4;
                        umma_f16_ts(d, a + kk * 8, b2 + ((kk * 2048) >> 4), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    if (half && split) {      // the lo term of P (columns 64..127 of the S region), all 128 keys
#pragma unroll 1
                        for (int kk = 0; kk < BN / 16; ++kk)
                            umma_f16_ts(d, a + 64 + kk * 8, b2 + (uint64_t)(kk * (2048 >> 4)), idesc_pv, 1u);
                    }
                    if (half) umma_commit(&sm.o_full[w]);
                };
                bool ok = mbar_wait_spin(&sm.q_full, 0, wc) &&
                          mbar_wait_spin(&sm.k_full[0], 0, wc);
                if (ok) {
                    tc_fence_after();
                    issue_qk(0, 0);
                    if (n1 > 0) issue_qk(1, 0);
                    umma_commit(&sm.k_empty[0]);
                }
                for (int j = 0; ok && j < nmax; ++j) {
                    const int s = j & 1;
                    const uint32_t ph = (j >> 1) & 1;
                    for (int w = 0; w < 2 && ok; ++w) {
                        if (j < nw[w]) {
                            if (!(ok = mbar_wait_spin(&sm.p_half[w], j & 1, wc))) break;
                            if (w == 0 || j >= n0) { if (!(ok = mbar_wait_spin(&sm.v_full[s], ph, wc))) break; }
                            tc_fence_after();
                            issue_pv(w, j, 0);
                            if (!(ok = mbar_wait_spin(&sm.p_full[w], j & 1, wc))) break;
                            tc_fence_after();
                            issue_pv(w, j, 1);
                        }
                        if (w == 1) umma_commit(&sm.v_empty[s]);
                        if (j + 1 < nw[w]) {
                            if (w == 0 || j + 1 >= n0) {
                                if (!(ok = mbar_wait_spin(&sm.k_full[(j + 1) % KSTAGES_PG], ((j + 1) / KSTAGES_PG) & 1, wc))) break;
                            }
                            tc_fence_after();
                            issue_qk(w, j + 1);
                        }
                        if (w == 1 && j + 1 < nmax) umma_commit(&sm.k_empty[(j + 1) % KSTAGES_PG]);
                    }
                }
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ softmax warpgroups
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmaxPg));
        const int w = warp >> 2;
        const int r = threadIdx.x & 127;
        const int nk = w ? n1 : n0;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int qi = q0 + w * BM + r;                    // row within the chunk
        softmax_row<T, 0, false>(&sm.s_full[w], &sm.p_half[w], &sm.p_full[w], &sm.o_full[w], lane_base + w * 128, lane_base + 256 + w * 128,
                       nk, shift + qi, r, p, wc, qi < q_len, q_beg + qi, h, split);
    }
    // ---------------------------------------------------------------------- teardown
    if (warp == 8 && lane == 0 && sm.box.abort) {
        const long long t0 = clock64();
        while (!mbar_try(&sm.q_full, 0) && clock64() - t0 < WAIT_CYCLES) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}
// Rows no query tile writes: those past the last sequence, and (when the caller's max_len is too
// small, which also raises ATTN_B200_FLAG_BAD_OFFSETS) the rows of a sequence beyond max_len rounded
// up to a pair of query tiles.  They are zeroed so that the output never carries uninitialised
// memory (the reference returns zeros there, zeros_like(V)).
__global__ void zero_uncovered_rows_kernel(void* out, const int32_t* offsets, int B, int64_t n_tokens, int max_len,
                                           int64_t row_bytes, int32_t* err_flag) {
    const int64_t vec_per_row = row_bytes / 16;
    const int64_t covered = (int64_t)((max_len + 2 * BM - 1) / (2 * BM)) * (2 * BM);
    auto clampt = [&](int64_t v) { return v < 0 ? (int64_t)0 : (v > n_tokens ? n_tokens : v); };
    auto zero_rows = [&](int64_t beg, int64_t end) {
        uint4* base = reinterpret_cast<uint4*>((char*)out + beg * row_bytes);
        const int64_t n_vec = (end - beg) * vec_per_row;
        for (int64_t i = threadIdx.x; i < n_vec; i += blockDim.x) base[i] = make_uint4(0, 0, 0, 0);
    };
    // CTA x takes sequences x, x + gridDim.x, ...; pseudo-sequence B is the tail past offsets[B-1]
    for (int b = blockIdx.x; b <= B; b += gridDim.x) {
        const int64_t beg = b ? clampt(offsets[b - 1]) : 0;
        const int64_t end = b < B ? clampt(offsets[b]) : n_tokens;
        if (end <= beg) continue;
        if (b == B) { zero_rows(beg, end); continue; }
        if (end - beg > covered) {
            if (err_flag && threadIdx.x == 0) atomicOr(err_flag, ATTN_B200_FLAG_BAD_OFFSETS);
            zero_rows(beg + covered, end);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// [n_tokens, H*128] 16-bit row-major.  Loads: box = 64 elements (128 B) x 128 rows, 128-byte swizzle;
// the output's stores (`store_box`): 32 elements (64 B) x 32 rows, 64-byte swizzle.
// A tensor map is a pure function of (base, n_tokens, H, dtype, box), so the last few are kept per
// host thread: a serving loop that calls with the same buffers pays for the encoding once.
static int make_map(CUtensorMap* map, const void* base, int64_t n_tokens, int H, int dtype, bool store_box = false) {
    struct Entry { const void* base; int64_t n_tokens; int H, dtype; bool store_box, used; CUtensorMap map; };
    constexpr int kEntries = 8;
    static thread_local Entry cache[kEntries] = {};
    static thread_local unsigned next = 0;
    for (const Entry& e : cache)
        if (e.used && e.base == base && e.n_tokens == n_tokens && e.H == H && e.dtype == dtype && e.store_box == store_box) {
            *map = e.map;
            return 0;
        }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)H * HD, (cuuint64_t)n_tokens};
    const cuuint64_t strides[1] = {(cuuint64_t)H * HD * 2};
    const cuuint32_t box[2] = {store_box ? 32u : 64u, store_box ? 32u : 128u};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dtype == ATTN_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          store_box ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    cache[next++ % kEntries] = Entry{base, n_tokens, H, dtype, store_box, true, *map};
    return 0;
}

// Per-device facts looked up once: the device address of g_launch, the SM count, and whether the
// kernels' dynamic shared-memory limits have been raised.
constexpr int kMaxDevices = 64;
struct DeviceState {
    LaunchState* launch_base = nullptr;
    int n_sm = 0;
    bool attrs_set = false;
};
static std::mutex g_dev_mu;
static DeviceState g_dev[kMaxDevices];

template <typename K>
static cudaError_t raise_smem(K kernel, int bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

static int device_state(DeviceState* out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ATTN_B200_ETOOLARGE;
    std::lock_guard<std::mutex> lock(g_dev_mu);
    DeviceState& d = g_dev[dev];
    if (!d.launch_base) {
        void* base = nullptr;
        if ((e = cudaGetSymbolAddress(&base, g_launch)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&d.n_sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        d.launch_base = static_cast<LaunchState*>(base);
    }
    if (!d.attrs_set) {
        if ((e = raise_smem(prefill_tc2p_kernel<__nv_bfloat16>, (int)sizeof(SmemLayout2p) + 1024)) != cudaSuccess ||
            (e = raise_smem(prefill_tc2p_kernel<__half>, (int)sizeof(SmemLayout2p) + 1024)) != cudaSuccess ||
            (e = raise_smem(paged_prefill_tc_kernel<__nv_bfloat16>, (int)sizeof(SmemLayoutPg) + 1024)) != cudaSuccess ||
            (e = raise_smem(paged_prefill_tc_kernel<__half>, (int)sizeof(SmemLayoutPg) + 1024)) != cudaSuccess)
            return (int)e;
        d.attrs_set = true;
    }
    *out = d;
    return 0;
}

// Takes the next of the kLaunchSlots launch-state slots and zeroes it on the launch's stream.
static int take_launch_slot(const DeviceState& d, cudaStream_t st, LaunchState** slot) {
    static std::atomic<unsigned> next_slot{0};
    *slot = d.launch_base + (next_slot.fetch_add(1) % kLaunchSlots);
    return (int)cudaMemsetAsync(*slot, 0, sizeof(LaunchState), st);
}

}  // namespace tc

bool prefill_tc_supported(int D, int dtype) {
    return D == tc::HD && (dtype == ATTN_B200_F16 || dtype == ATTN_B200_BF16);
}

int prefill_tc_launch(const void* q, const void* k, const void* v, const int32_t* offsets, void* out, int B,
                      int64_t n_tokens, int max_len, int H, int D, float scale, int dtype, int out_f32, int precise,
                      int32_t* err_flag, cudaStream_t st) {
    using namespace tc;
    if (D != HD) return ATTN_B200_ESHAPE;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) % 16) return ATTN_B200_EINVAL;
    if (n_tokens > 0x7fffffffLL || B > 65535 || H > 65535) return ATTN_B200_ETOOLARGE;
    CUtensorMap mq, mk, mv, mo;
    int rc;
    if ((rc = make_map(&mq, q, n_tokens, H, dtype)) || (rc = make_map(&mk, k, n_tokens, H, dtype)) ||
        (rc = make_map(&mv, v, n_tokens, H, dtype)))
        return rc;
    // the staged read-out stores 16-bit tiles through this map (fp32 output takes the direct path:
    // the map then describes the buffer as if it were 16-bit and is never used)
    if ((rc = make_map(&mo, out, n_tokens, H, dtype, true))) return rc;
    DeviceState d;
    LaunchState* slot = nullptr;
    if ((rc = device_state(&d)) || (rc = take_launch_slot(d, st, &slot))) return rc;
    Params p{offsets, out, B, H, n_tokens, (max_len + 2 * BM - 1) / (2 * BM), scale * kLog2e, out_f32, err_flag,
             &slot->abort, precise ? 0x7fffffff : 2 * BM};
    const int64_t row_bytes = (int64_t)H * HD * (out_f32 ? 4 : 2);
    zero_uncovered_rows_kernel<<<64, 256, 0, st>>>(out, offsets, B, n_tokens, max_len, row_bytes, err_flag);
    const int64_t n_items = (((int64_t)H * B + ITEM_GROUP - 1) / ITEM_GROUP) * ITEM_GROUP * p.n_qtiles;
    if (n_items == 0) return (int)cudaGetLastError();
    const int smem_p = (int)sizeof(SmemLayout2p) + 1024;
    const unsigned ctas = (unsigned)(n_items < d.n_sm ? n_items : d.n_sm);
    if (dtype == ATTN_B200_BF16)
        prefill_tc2p_kernel<__nv_bfloat16><<<ctas, THREADS2, smem_p, st>>>(mq, mk, mv, mo, p, n_items, &slot->work);
    else
        prefill_tc2p_kernel<__half><<<ctas, THREADS2, smem_p, st>>>(mq, mk, mv, mo, p, n_items, &slot->work);
    return (int)cudaGetLastError();
}


// ---- paged (chunked) prefill launcher, called from paged_prefill.cu
int paged_prefill_tc_launch_impl(const void* q, const void* k_cache, const void* v_cache, const int32_t* slots,
                                 const int32_t* kv_offsets, const int32_t* q_offsets, void* out, int B,
                                 int64_t n_q_tokens, int64_t n_kv_tokens, int max_q_len, int H, int Hkv, int D,
                                 int64_t n_slots, float scale, int dtype, int32_t* err_flag, cudaStream_t st) {
    using namespace tc;
    if (D != HD || (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16)) return ATTN_B200_ESHAPE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16) return ATTN_B200_EINVAL;
    if (n_q_tokens > 0x7fffffffLL || B > 65535 || H > 65535) return ATTN_B200_ETOOLARGE;
    CUtensorMap mq;
    int rc = make_map(&mq, q, n_q_tokens, H, dtype);
    if (rc) return rc;
    DeviceState d;
    LaunchState* slot = nullptr;
    if ((rc = device_state(&d)) || (rc = take_launch_slot(d, st, &slot))) return rc;
    const int smem = (int)sizeof(SmemLayoutPg) + 1024;
    Params p{q_offsets, out, B, H, n_q_tokens, (max_q_len + 2 * BM - 1) / (2 * BM), scale * kLog2e, 0, err_flag,
             &slot->abort, 2 * BM};
    PagedTcParams pg{slots, kv_offsets, q_offsets, k_cache, v_cache, Hkv, n_kv_tokens, n_slots};
    zero_uncovered_rows_kernel<<<64, 256, 0, st>>>(out, q_offsets, B, n_q_tokens, max_q_len, (int64_t)H * HD * 2, err_flag);
    if (p.n_qtiles == 0) return (int)cudaGetLastError();
    dim3 grid(p.n_qtiles, H, B);
    if (dtype == ATTN_B200_BF16)
        paged_prefill_tc_kernel<__nv_bfloat16><<<grid, THREADS_PG, smem, st>>>(mq, p, pg);
    else
        paged_prefill_tc_kernel<__half><<<grid, THREADS_PG, smem, st>>>(mq, p, pg);
    return (int)cudaGetLastError();
}

}  // namespace attn
