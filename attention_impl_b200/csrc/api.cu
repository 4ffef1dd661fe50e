// Status strings and ABI version of libattn_b200.
#include <cuda_runtime.h>

#include "../../include/attn_b200.h"

extern "C" const char* attn_b200_strerror(int status) {
    switch (status) {
        case 0: return "ok";
        case ATTN_B200_EINVAL: return "invalid argument (null pointer or non-positive size)";
        case ATTN_B200_EDTYPE: return "unsupported element type for this entry point";
        case ATTN_B200_ESHAPE: return "unsupported head_dim / rot_half / chunk";
        case ATTN_B200_EWORKSPACE: return "workspace too small or misaligned";
        case ATTN_B200_ETOOLARGE: return "size beyond a documented limit";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

extern "C" int attn_b200_abi_version(void) { return 4; }
