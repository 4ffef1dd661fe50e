// Paged decode for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a serving engine that reserved every
// free byte of HBM for its own KV pool at start-up (an allocation would simply fail), or a
// latency-critical decode loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply.  The regular entry point needs the caller to hand it a split-KV scratch buffer;
// this one carries its own, a fixed array that lives in the library's device image.
#include <mutex>

#include "common.cuh"

namespace {

// Scratch for the (unit, head) partial rows [o[D], m, l].  One copy exists on every device that
// loads the library, from load until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[ATTN_B200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can
// use; the real device address differs per device and has to be asked for with that device current.
int scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ATTN_B200_ETOOLARGE;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return (int)cudaErrorInvalidSymbol;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int attn_b200_paged_decode_static_scratch(
    const void* q, const void* k_new, const void* v_new, const void* k_cache, const void* v_cache,
    const int32_t* slots, const int32_t* offsets, void* out, int B, int H, int D, int64_t n_tokens,
    int64_t n_slots, int chunk, float scale, const float* k_scale, const float* v_scale, int q_dtype,
    int kv_dtype, int32_t* err_flag, void* stream) {
    const size_t need = attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens, chunk);
    if (need == 0) return ATTN_B200_EINVAL;
    if (need > (size_t)ATTN_B200_STATIC_SCRATCH_BYTES) return ATTN_B200_ETOOLARGE;
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    return attn_b200_paged_decode(q, k_new, v_new, k_cache, v_cache, slots, offsets, out, scratch,
                                  (size_t)ATTN_B200_STATIC_SCRATCH_BYTES, nullptr, nullptr, 0, B, H, /*n_kv_heads=*/H,
                                  D, n_tokens, n_slots, 0, /*block_size=*/1, /*max_blocks=*/0, chunk, scale, k_scale,
                                  v_scale, q_dtype, kv_dtype, 3, err_flag, stream);
}
