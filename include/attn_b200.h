/*
 * attn_b200.h — C ABI of libattn_b200.so: sm_100a kernels for the attention hot path of
 * ita9naiwa/attention-impl (paged single-query decode, packed causal prefill, dense masked
 * attention, single-query over a contiguous cache, rotary embedding).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise.
 *  - Data tensors are dense row-major.  "[rows, H*D]" means one row per token with all heads
 *    contiguous (the reference's layout, paged_attention_kernel.cu:132).
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, no call synchronises.
 *  - Return value: 0 = ok; negative = argument error (ATTN_B200_E*); positive = cudaError_t of
 *    a failed launch.  attn_b200_strerror() renders either.
 *  - Outputs and scratch are allocated by the caller; no entry point allocates or frees device memory.
 *    The library's device image holds three small fixed arrays of its own (every device that loads
 *    it carries them until the process exits): 64 launch-state slots of 16 bytes for the tensor-core
 *    prefill kernels (work counter + abort word, taken in rotation, so at most 64 such launches may
 *    be in flight at once), and the ATTN_B200_STATIC_SCRATCH_BYTES array that only
 *    attn_b200_paged_decode_static_scratch uses.
 *  - `err_flag` (optional, may be NULL): device int32 that kernels OR a bit into when they meet an
 *    out-of-range slot / position; the offending row is skipped, never dereferenced.
 */
#ifndef ATTN_B200_H
#define ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(ATTN_B200_BUILD) && defined(__GNUC__)
#define ATTN_B200_API __attribute__((visibility("default")))
#else
#define ATTN_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum {
    ATTN_B200_F16 = 0,
    ATTN_B200_BF16 = 1,
    ATTN_B200_F32 = 2,
    ATTN_B200_E4M3 = 3 /* KV pools only */
};

/* argument errors */
enum {
    ATTN_B200_EINVAL = -1,       /* null pointer / non-positive size */
    ATTN_B200_EDTYPE = -2,       /* unsupported element type for this entry point */
    ATTN_B200_ESHAPE = -3,       /* head_dim / rot_half / chunk not supported */
    ATTN_B200_EWORKSPACE = -4,   /* scratch buffer too small */
    ATTN_B200_ETOOLARGE = -5     /* size beyond a documented limit */
};

/* bits a kernel may set in *err_flag */
enum {
    ATTN_B200_FLAG_BAD_SLOT = 1,     /* cache_indices entry outside [0, n_slots) */
    ATTN_B200_FLAG_BAD_POSITION = 2, /* positions entry outside [0, max_pos) */
    ATTN_B200_FLAG_BAD_OFFSETS = 4,  /* offsets not non-decreasing / beyond n_tokens */
    ATTN_B200_FLAG_TIMEOUT = 8       /* a bounded in-kernel wait ran out; the kernel gave up cleanly */
};

ATTN_B200_API const char* attn_b200_strerror(int status);
/* ABI version of this header (4); bumped on any change of a signature or of an argument's meaning. */
ATTN_B200_API int attn_b200_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * Rotary embedding, in place on q and k.
 * Replaces rotary_embedding_inplace (rotary_embedding.cu:40-77, kernel :10-36).
 *   q [n_tokens, n_heads_q*head_dim], k [n_tokens, n_heads_k*head_dim]   (dtype)
 *   positions int32 [n_tokens]; cos, sin [max_pos, rot_half] (dtype)
 * For d < rot_half:  x[d]        <- fl(fl(x[d]*c) + fl(-x[d+rot_half]*s))
 *                    x[d+rot_half] <- fl(fl(x[d+rot_half]*c) + fl(x[d]*s)),  c,s = cos/sin[pos, d]
 * each product and the sum rounded to `dtype` separately (no FMA contraction), dims >= 2*rot_half
 * untouched.  k may be NULL (n_heads_k ignored).  dtype: F16, BF16, F32.
 */
ATTN_B200_API int attn_b200_rope_inplace(void* q, void* k, const int32_t* positions, const void* cos, const void* sin,
                           int64_t n_tokens, int n_heads_q, int n_heads_k, int head_dim, int rot_half,
                           int64_t max_pos, int dtype, int32_t* err_flag, void* stream);

/* Rotary embedding fused with the KV-cache append.  No counterpart in the reference: its decode
 * operator receives the current token's k, v as arguments (paged_attention_kernel.cu:137-146,
 * 179-185) and leaves writing them into the pools to the caller; this is that step.
 *   q [n_tokens, n_heads_q*head_dim], k, v [n_tokens, n_heads_k*head_dim]  (dtype F16/BF16)
 *   slots int32 [n_tokens]: pool row of each token;  k_cache, v_cache [n_slots, n_heads_k*head_dim]
 *   in `dtype`, or E4M3 with k_scale, v_scale float [n_heads_k] (stored value = rn_e4m3(x / scale)).
 * q and k are rotated in place exactly as attn_b200_rope_inplace does; rotated k and v are stored
 * at their slot.  rot_half and head_dim must be multiples of 8.  Out-of-range slots/positions set
 * err_flag bits and skip the store. */
ATTN_B200_API int attn_b200_rope_write_kv(void* q, void* k, const void* v, const int32_t* positions,
                                          const void* cos, const void* sin, const int32_t* slots, void* k_cache,
                                          void* v_cache, int64_t n_tokens, int n_heads_q, int n_heads_k,
                                          int head_dim, int rot_half, int64_t max_pos, int64_t n_slots, int dtype,
                                          int kv_dtype, const float* k_scale, const float* v_scale,
                                          int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------------------------------
 * KV-paged single-query decode (block_size = 1 slot table).
 * Replaces paged_kv_attention_forward (paged_attention_kernel.cu:237-294, kernel :100-187) and,
 * with slots == NULL and offsets == NULL, kv_attention_forward (attention_kernel.cu:231-280,
 * kernel :96-185).
 *   q, k_new, v_new, out  [B, H*D]            (q_dtype: F16, BF16, F32)
 *   k_cache, v_cache      [n_slots, H*D]      (kv_dtype: q_dtype, or E4M3 with F16/BF16 q)
 *   slots   int32 [n_tokens]  slot of the t-th token of the concatenated sequences, or NULL
 *                             for the identity table (token t lives in row t)
 *   offsets int32 [B]         INCLUSIVE cumulative context lengths, or NULL for a uniform
 *                             length `uniform_ctx` (then n_tokens == B*uniform_ctx)
 *   k_scale, v_scale float [H] per-head dequantisation scales (E4M3 only, else NULL)
 *   S, P    double [B, H, sp_stride]  optional (both or neither): scaled scores and
 *           probabilities, the new token's entry at index ctx_b; entries beyond are NOT written
 *           (pass zeroed buffers, as the reference does).  sp_stride >= max ctx + 1.
 * Per (b, h): softmax over the ctx_b cached tokens plus the new token (k_new, v_new) of
 * `scale * <q, k>`; out = sum p * v.  Context tokens are cut into chunks of `chunk` tokens on a
 * global grid; each (chunk, head) is reduced by one warp into an (m, l, o) partial in
 * `workspace`, then attn_b200_lse_combine-style reduction folds the partials and the new token.
 * `chunk` must be a multiple of 32 in [32, 2048]; use attn_b200_paged_decode_pick_chunk.
 * `workspace` needs attn_b200_paged_decode_workspace_bytes(...) bytes, 16-byte aligned; it needs
 * no initialisation and holds nothing between calls.
 * `stages`: 3 runs both kernels (the normal call); 1 runs only the partial kernel, 2 only the
 * combine kernel (same arguments) so that a profiler or benchmark can put events between them;
 * 4 is the single-launch form: one CTA per (sequence, head) whose warps split the sequence's tokens
 * and combine in shared memory (`workspace` may be NULL, `chunk` is only range-checked).  It exists
 * for multi-head attention (n_kv_heads == H) with a per-token table, 16-bit q and pools of q's type,
 * head_dim 64 / 128 / 256 and S == NULL (anything else: ATTN_B200_ESHAPE), and it pays only when B*H
 * CTAs fill the machine in one wave and the sequences are short:
 * attn_b200_paged_decode_single_launch_ok() says when.
 * The combine kernel is launched as a programmatic dependent of the partial kernel (its launch and
 * prologue overlap that kernel's tail; it waits for the partial rows itself).  The multi-head partial
 * kernel is in turn launched as a programmatic dependent of whatever kernel precedes the call on
 * `stream`, and reads nothing before that kernel has completed, so this is invisible to the caller.
 * ATTN_B200_DECODE_TABLES_READY or-ed into `stages` (3 | ATTN_B200_DECODE_TABLES_READY) is the
 * caller's statement that `slots` and `offsets` were complete BEFORE the kernel preceding this call
 * on `stream` started (they came from an upload or an earlier kernel, not from that one): the partial
 * kernel then reads them while that kernel may still be running, which hides two of its three
 * dependent round trips.  Everything else (q, the pools, k_new, v_new) may still be written by the
 * preceding kernel.  Without the flag nothing is assumed.
 * Extensions beyond the reference (which is multi-head, block_size = 1):
 *   n_kv_heads  KV heads (H % n_kv_heads == 0); k_new, v_new, k_cache, v_cache then have n_kv_heads*D
 *               columns and query head h reads KV head h / (H / n_kv_heads).  Pass H for MHA.
 *   block_size  tokens per KV block.  1: `slots` is the per-token table above.  > 1: `slots` is a
 *               block table int32 [B, max_blocks]; token t of sequence b lives in pool row
 *               slots[b*max_blocks + t/block_size]*block_size + t%block_size.
 */
enum { ATTN_B200_DECODE_TABLES_READY = 0x100 };
ATTN_B200_API int attn_b200_paged_decode(const void* q, const void* k_new, const void* v_new, const void* k_cache,
                           const void* v_cache, const int32_t* slots, const int32_t* offsets, void* out,
                           void* workspace, size_t workspace_bytes, double* S, double* P, int64_t sp_stride,
                           int B, int H, int n_kv_heads, int D, int64_t n_tokens, int64_t n_slots,
                           int uniform_ctx, int block_size, int max_blocks, int chunk, float scale,
                           const float* k_scale, const float* v_scale, int q_dtype, int kv_dtype, int stages,
                           int32_t* err_flag, void* stream);

ATTN_B200_API size_t attn_b200_paged_decode_workspace_bytes(int B, int H, int D, int64_t n_tokens, int chunk);
/* Non-zero when the single-launch form (`stages` = 4) exists for this case and is expected to beat
 * the two-launch form: sm_count <= B*H <= 2*sm_count and at most 1024 tokens of capacity per sequence on
 * average (a CTA lives as long as its sequence is long: one long sequence among short ones would
 * hold the step). */
ATTN_B200_API int attn_b200_paged_decode_single_launch_ok(int B, int H, int n_kv_heads, int D, int64_t n_tokens,
                                                          int block_size, int q_dtype, int kv_dtype, int sm_count);
/* Heuristic chunk length: enough (chunk, head-group) work items to fill `sm_count` SMs. */
ATTN_B200_API int attn_b200_paged_decode_pick_chunk(int B, int H, int D, int64_t n_tokens, int sm_count);
/* The same for grouped-query heads: `group` query heads per KV head, `kv_dtype` of the pools.  Groups
 * of 2, 4 and 8 at head_dim 128 run on the tensor cores and prefer longer chunks. */
ATTN_B200_API int attn_b200_paged_decode_pick_chunk_gqa(int B, int n_kv_heads, int group, int D, int kv_dtype,
                                                        int64_t n_tokens, int sm_count);

/* Same first stage as attn_b200_paged_decode, but the second stage writes, per (b, h), one
 * partial row  [m (log2 domain), l, o[D] (un-normalised)]  of D+2 floats into
 * part_out [B, H, D+2] instead of the final output, and does NOT fold the new token.  This is
 * what one rank of a KV-split group computes over its own slice of every sequence.
 * No counterpart in the reference (it has no split-KV). */
ATTN_B200_API int attn_b200_paged_decode_partial(const void* q, const void* k_cache, const void* v_cache,
                                   const int32_t* slots, const int32_t* offsets, float* part_out,
                                   void* workspace, size_t workspace_bytes, int B, int H, int n_kv_heads, int D,
                                   int64_t n_tokens, int64_t n_slots, int block_size, int max_blocks, int chunk,
                                   float scale, const float* k_scale, const float* v_scale, int q_dtype,
                                   int kv_dtype, int32_t* err_flag, void* stream);

/* Log-sum-exp combine of n_parts partial sets  parts [n_parts, B, H, D+2]  (layout above) plus
 * the new token (k_new, v_new; may both be NULL to skip it) into out [B, H*D] (q_dtype).
 * No counterpart in the reference. */
ATTN_B200_API int attn_b200_lse_combine(const float* parts, int n_parts, const void* q, const void* k_new,
                          const void* v_new, void* out, int B, int H, int n_kv_heads, int D, float scale,
                          int q_dtype, void* stream);

/* Peer-memory exchange for the KV-split path (no counterpart in the reference).  Replaces the NCCL
 * all-gather of the partial rows: attn_b200_peer_push stores `n_bytes` (multiple of 16) from `src`
 * into peer_dst[g] for every g < n_peers (host arrays of device pointers that are valid in this
 * process: peer allocations mapped by CUDA IPC / symmetric memory, or local memory for g = self),
 * then adds 1 per CTA to each *peer_flag[g] (int32, system-scope atomic).  One push adds
 * attn_b200_peer_push_ctas(n_bytes) to each counter; counters are never reset.
 * attn_b200_wait_flags enqueues a kernel that waits until every flags[i] (i < n_flags <= 32, local
 * memory written by the peers) has reached `expected`; the wait is bounded (about one second) and
 * sets ATTN_B200_FLAG_TIMEOUT in *err_flag when it gives up.  Work enqueued after it on the same
 * stream sees the pushed data. */
ATTN_B200_API int attn_b200_peer_push_ctas(size_t n_bytes);
ATTN_B200_API int attn_b200_peer_push(const void* src, size_t n_bytes, void* const* peer_dst,
                                      int32_t* const* peer_flag, int n_peers, void* stream);
ATTN_B200_API int attn_b200_wait_flags(const int32_t* flags, int n_flags, int32_t expected, int32_t* err_flag,
                                       void* stream);
/* The same wait, but every counter that has reached `count` has `count` taken off it again
 * (system-scope atomic; arrivals of a peer's next push that are already there stay).  With
 * count = attn_b200_peer_push_ctas(n_bytes) every step of an exchange uses the same arguments, so
 * the step can be captured in a CUDA graph and replayed.  A peer may run at most one push ahead. */
ATTN_B200_API int attn_b200_wait_flags_consume(int32_t* flags, int n_flags, int32_t count, int32_t* err_flag,
                                               void* stream);

/* The KV-split exchange in three launches instead of five (no counterpart in the reference).
 * attn_b200_paged_decode_partial_push = attn_b200_paged_decode_partial whose second stage stores
 * each (b, h) row [o[D], m, l] straight into peer_dst[g] ([B, H, D+2] float, this rank's slot of
 * peer g's gather buffer, g < n_peers <= 16; host arrays of device pointers valid in this process)
 * with plain stores and then adds 1 per (b, h) to *peer_flag[g] (system-scope): a step adds B*H to
 * each counter.  attn_b200_lse_combine_wait = attn_b200_lse_combine whose CTAs first wait, each by
 * itself and bounded (about a second, then ATTN_B200_FLAG_TIMEOUT in *err_flag and the kernel goes
 * on and ends), until flags[i] >= B*H for every i < n_parts; the last CTA past the wait takes B*H
 * off every counter again (arrivals of a peer already one step ahead stay) using *done_counter
 * (an int32 of the caller's, zero before the first call, left zero), so every step has the same
 * arguments and can be replayed from a CUDA graph.  16-bit q only. */
ATTN_B200_API int attn_b200_paged_decode_partial_push(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* slots, const int32_t* offsets,
    void* workspace, size_t workspace_bytes, int B, int H, int n_kv_heads, int D, int64_t n_tokens, int64_t n_slots,
    int block_size, int max_blocks, int chunk, float scale, const float* k_scale, const float* v_scale, int q_dtype,
    int kv_dtype, float* const* peer_dst, int32_t* const* peer_flag, int n_peers, int32_t* err_flag, void* stream);
ATTN_B200_API int attn_b200_lse_combine_wait(const float* parts, int n_parts, const void* q, const void* k_new,
                                             const void* v_new, void* out, int B, int H, int n_kv_heads, int D,
                                             float scale, int q_dtype, int32_t* flags, int32_t* done_counter,
                                             int32_t* err_flag, void* stream);

/* Paged decode that allocates nothing and needs no scratch from the caller.
 * (No counterpart in the reference: its launcher allocates S, P and O itself with torch::zeros.)
 * For hosts that cannot call cudaMalloc — an engine that gave all free HBM to its own KV pool, or
 * a decode loop that cannot take the device-wide synchronisation an allocation implies.  Same
 * arguments and result as attn_b200_paged_decode without workspace/S/P/uniform_ctx/stages and for
 * multi-head attention with a per-token slot table only (it passes n_kv_heads = H, block_size = 1:
 * no grouped-query pools, no block tables); the split-KV partial rows go to a fixed
 * ATTN_B200_STATIC_SCRATCH_BYTES array inside the library's device image (every device that loads
 * the library holds it until the process exits).
 *  - Returns ATTN_B200_ETOOLARGE when attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens,
 *    chunk) exceeds ATTN_B200_STATIC_SCRATCH_BYTES; a larger `chunk` (up to 2048) lowers the need.
 *  - The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 *    that device current) and keeps it; make that first call outside any stream capture.  With
 *    CUDA's lazy module loading that look-up is also the moment the 16 MiB array is materialised on
 *    the device: a host that is about to hand all free HBM to its own pool must make this first
 *    call BEFORE it does so, or the look-up fails for lack of memory.
 *  - The address is kept per CURRENT device: the device that is current at the call must be the one
 *    that owns `stream` and the pointers.
 *  - All calls on a device share the one array.  Nothing in it has to be cleared between calls (a
 *    call only reads rows it wrote itself), but two calls that overlap on the GPU — different
 *    streams, no ordering between them — race on it: serialise them.
 *  - Calls no cudaMalloc/cudaFree and no allocating library routine. */
#define ATTN_B200_STATIC_SCRATCH_BYTES (16u << 20)
ATTN_B200_API int attn_b200_paged_decode_static_scratch(
    const void* q, const void* k_new, const void* v_new, const void* k_cache, const void* v_cache,
    const int32_t* slots, const int32_t* offsets, void* out, int B, int H, int D, int64_t n_tokens,
    int64_t n_slots, int chunk, float scale, const float* k_scale, const float* v_scale, int q_dtype,
    int kv_dtype, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------------------------------
 * Packed (non-contiguous) causal prefill.
 * Replaces paged_attention_forward (paged_attention_kernel.cu:189-235, kernel :15-98).
 *   q, k, v, out [n_tokens, H*D] (dtype); offsets int32 [B] inclusive cumulative lengths;
 *   max_len >= longest sequence (sizes the grid; rows beyond a sequence's end are skipped).
 *   S, P optional [B, H, max_len, max_len] (dtype) — both or neither; only the generic path
 *   writes them.  Key j is visible to query i of the same sequence iff j <= i.
 * dtype F16/BF16 with D == 128 and S == NULL runs the tcgen05 tensor-core kernel; everything else
 * runs the generic kernel.  `out_flags` (tensor-core kernel only): ATTN_B200_PREFILL_OUT_F32 stores
 * fp32 output instead of dtype; ATTN_B200_PREFILL_PRECISE_P carries the probabilities into P*V as two
 * terms of the input type on EVERY row instead of only on a sequence's first 256 rows: bf16 inputs
 * then stay within 2e-3 max-abs of exact arithmetic everywhere (3.4e-3 without it, from the 2^-9
 * rounding of one dominant probability), for about a quarter more time.
 * A sequence longer than max_len raises ATTN_B200_FLAG_BAD_OFFSETS; rows that no tile covers (past
 * offsets[B-1], or beyond max_len rounded up to 256) are written as zeros by the tensor-core path.
 */
enum { ATTN_B200_PREFILL_OUT_F32 = 1, ATTN_B200_PREFILL_PRECISE_P = 2 };
ATTN_B200_API int attn_b200_varlen_prefill(const void* q, const void* k, const void* v, const int32_t* offsets, void* out,
                             void* S, void* P, int B, int64_t n_tokens, int max_len, int H, int D,
                             float scale, int dtype, int out_flags, int force_generic, int32_t* err_flag,
                             void* stream);

/* Chunked / prefix-cached prefill through the slot table (no counterpart in the reference: it is
 * its packed prefill and its paged single-query operator unified).  Sequence b contributes the
 * query rows [q_offsets[b-1], q_offsets[b]) of q [n_q_tokens, H*D] — the LAST tokens of the sequence —
 * and the keys slots[kv_offsets[b-1] .. kv_offsets[b]) (all of its tokens, the chunk's own included,
 * already in the pools k_cache, v_cache [n_slots, n_kv_heads*D]).  Query i of a chunk of q_len rows
 * over kv_len keys sees key j iff j <= kv_len - q_len + i.  max_q_len / max_kv_len bound the
 * per-sequence lengths (grid and shared-memory sizing; max_kv_len <= 12288 on the generic path).
 * dtype F16 / BF16 / F32; out [n_q_tokens, H*D] in dtype. */
ATTN_B200_API int attn_b200_paged_prefill(const void* q, const void* k_cache, const void* v_cache,
                                          const int32_t* slots, const int32_t* kv_offsets, const int32_t* q_offsets,
                                          void* out, int B, int64_t n_q_tokens, int64_t n_kv_tokens, int max_q_len,
                                          int max_kv_len, int H, int n_kv_heads, int D, int64_t n_slots, float scale,
                                          int dtype, int force_generic, int32_t* err_flag, void* stream);

/* Dense masked attention.  Replaces naive_attention_forward (attention_kernel.cu:187-229,
 * kernel :15-94).  q, k, v, out [B, L, H*D]; mask [B, L, L] (dtype) or NULL; scores are
 * scale*<q,k> + (mask-1)*fill;  S, P optional [B, H, L, L] (dtype). */
ATTN_B200_API int attn_b200_dense_attention(const void* q, const void* k, const void* v, const void* mask, void* out,
                              void* S, void* P, int B, int L, int H, int D, float scale, float fill,
                              int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATTN_B200_H */
