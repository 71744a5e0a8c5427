// Shared helpers for the sm_100a kernels behind the C ABI declared in include/rwkv_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/rwkv_b200.h"

#define RWKV_CHECK_ARG(cond) do { if (!(cond)) return RWKV_ERR_INVALID_ARG; } while (0)
#define RWKV_CHECK_ALIGN(p, a) do { if ((reinterpret_cast<uintptr_t>(p) % (a)) != 0) return RWKV_ERR_ALIGNMENT; } while (0)

static inline int rwkv_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? RWKV_OK : RWKV_ERR_LAUNCH;
}

// Launch with programmatic stream serialization: the kernel may begin while its predecessor
// in the stream drains; kernels order themselves with griddepcontrol.wait.  RWKV_B200_PDL=0
// in the environment turns the attribute off.
template <typename... KArgs, typename... Args>
static inline int rwkv_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args... args) {
    static int use_pdl = -1;
    if (use_pdl < 0) {
        const char* e = getenv("RWKV_B200_PDL");
        use_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

static inline int rwkv_sm_count() {       // of the current device
    static int sms_by_device[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
    if (sms_by_device[dev] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        sms_by_device[dev] = sms;
    }
    return sms_by_device[dev];
}

template <typename F> __device__ __forceinline__ float to_f32(F v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename F> __device__ __forceinline__ F from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Round-to-fp16-and-back: the reference rounds every torch op on fp16 tensors once.
__device__ __forceinline__ float r16(float v) { return __half2float(__float2half_rn(v)); }
