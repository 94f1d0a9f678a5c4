// Small host-only entry points of the C ABI.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/biloco_b200.h"

extern "C" const char* biloco_b200_error_string(int code) {
    switch (code) {
        case BILOCO_OK: return "ok";
        case BILOCO_ERR_NULL: return "a required pointer is null";
        case BILOCO_ERR_SHAPE: return "shape not supported";
        case BILOCO_ERR_ALIGN: return "pointer not aligned as required";
        case BILOCO_ERR_SCRATCH: return "scratch buffer too small";
        case BILOCO_ERR_CUDA: return "CUDA runtime or driver call failed";
        case BILOCO_ERR_MODE: return "unknown mode or quantisation rule";
        case BILOCO_ERR_EPOCH: return "epoch must be >= 1";
        case BILOCO_ERR_LIMIT: return "size beyond the stated maximum";
        case BILOCO_ERR_WAIT: return "a bounded wait on the device ran out";
        default: return "unknown error code";
    }
}

extern "C" int biloco_b200_abi_version(void) { return 1; }

extern "C" size_t biloco_b200_sf_bytes(int rows, int k) {
    if (rows < 0 || k < 0) return 0;
    return (size_t)((rows + 127) / 128 * 128) * (size_t)(((k / 16) + 3) / 4 * 4);
}
