// Version and error-string entry points of the C ABI.
#include "common.cuh"

extern "C" int rwkv_b200_version(void) { return 1000; }

extern "C" const char* rwkv_b200_error_string(int code) {
    switch (code) {
    case RWKV_OK: return "ok";
    case RWKV_ERR_INVALID_ARG: return "invalid argument (size, NULL pointer, dtype or epilogue)";
    case RWKV_ERR_ALIGNMENT: return "pointer or stride alignment not supported by the kernel";
    case RWKV_ERR_WORKSPACE: return "workspace missing or too small";
    case RWKV_ERR_LAUNCH: return "CUDA runtime rejected the kernel launch";
    case RWKV_ERR_UNSUPPORTED: return "no kernel for this configuration";
    case RWKV_ERR_STATIC_LIMIT: return "M exceeds the fixed scratch of rwkv_mm8_one_static (M <= 32768)";
    default: return "unknown error code";
    }
}
