// Device helpers of the stand-alone fp8_flow_moe kernels (sm_100a): export macro, bf16 pack / unpack, warp
// reductions. Kept separate from the training framework's kernel header so that this package builds on its own.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#ifndef NP_API
#define NP_API extern "C" __attribute__((visibility("default")))
#endif

// "Done once" guard for settings CUDA keeps per device (cudaFuncSetAttribute).
#ifndef NP_PER_DEVICE_ONCE_DEFINED
#define NP_PER_DEVICE_ONCE_DEFINED
struct NpPerDeviceOnce {
  bool done[64] = {};
  bool* slot() {
    int dev = 0;
    cudaGetDevice(&dev);
    return &done[dev & 63];
  }
};
#endif

namespace np {
#ifndef NP_FP8_COMMON_HELPERS
#define NP_FP8_COMMON_HELPERS
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(h);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
#endif
}  // namespace np
