// FP8 (e4m3) block-scaling kernels for sm_100a, the data-movement half of FP8-Flow-MoE:
//   quant_1x128      bf16 [rows, cols] -> e4m3 + fp32 scale per 1x128 block (amax / 448)
//   dequant_1x128    the inverse, to bf16
//   quant_128x128    weight quantisation, one scale per 128x128 tile
//   transpose_1x128  scaling-aware transpose: [M, N] quantised along N -> [N, M] quantised along M,
//                    tile by tile through shared memory, never materialising bf16 in HBM
//   swiglu_quant     silu(gate) * up quantised in the same pass
// Reference names: quantize_to_fp8 / dequantize_from_fp8 / scaling_aware_transpose /
// fused_silu_multiply_quantize of the fp8_flow_moe package (fp8/__init__.py:8-22 of the reference).
#include "fp8_common.cuh"

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint32_t to_e4m3(float v) {
  return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint32_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(b & 0xffu), __NV_E4M3);
  return __half2float(__half(h));
}
__device__ __forceinline__ uint2 quant8(const float* f, float inv) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= to_e4m3(f[j] * inv) << (8 * j);
    hi |= to_e4m3(f[4 + j] * inv) << (8 * j);
  }
  return make_uint2(lo, hi);
}

// One half-warp (16 lanes x 8 elements) per 128-element block. mode 0: x; mode 1: silu(x) * y.
__global__ void __launch_bounds__(256) quant_1x128_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ q,
                                                          float* __restrict__ scales, long long nblocks, int mode,
                                                          int bpr, long long x_ld, long long y_ld) {
  const int lane16 = threadIdx.x & 15;
  const long long hw = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 4;
  const long long nhw = ((long long)gridDim.x * blockDim.x) >> 4;
  const long long iters = (nblocks + nhw - 1) / nhw;  // uniform trip count keeps the shuffles converged
  for (long long it = 0; it < iters; ++it) {
    const long long b = hw + it * nhw;
    const bool ok = b < nblocks;
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (ok) {
      const long long row = b / bpr;
      const int kb = (int)(b - row * bpr);  // inputs may be strided rows (views into a wider buffer)
      load8(x + row * x_ld + kb * 128 + lane16 * 8, f);
      if (mode == 1) {
        float g[8];
        load8(y + row * y_ld + kb * 128 + lane16 * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = np::silu_f(f[j]) * g[j];
      }
    }
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[j]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float scale = fmaxf(am, 1e-12f) / 448.f;
    if (ok) {
      *reinterpret_cast<uint2*>(q + b * 128 + lane16 * 8) = quant8(f, 1.f / scale);
      if (lane16 == 0) scales[b] = scale;
    }
  }
}

__global__ void __launch_bounds__(256) dequant_1x128_kernel(const uint8_t* __restrict__ q,
                                                            const float* __restrict__ scales,
                                                            __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint2 u = reinterpret_cast<const uint2*>(q)[i];
    const float s = scales[i >> 4];
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[j] = from_e4m3(u.x >> (8 * j)) * s;
      f[4 + j] = from_e4m3(u.y >> (8 * j)) * s;
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                                  np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
  }
}

// One CTA (256 threads) per 128x128 tile: thread t covers row t/2, columns (t%2)*64 .. +63.
__global__ void __launch_bounds__(256) quant_128x128_kernel(const __nv_bfloat16* __restrict__ w,
                                                            uint8_t* __restrict__ q, float* __restrict__ scales, int R,
                                                            int C) {
  __shared__ float red[8];
  const int tr = blockIdx.y, tc = blockIdx.x;
  const int r = tr * 128 + (threadIdx.x >> 1), c0 = tc * 128 + (threadIdx.x & 1) * 64;
  float f[64];
  float am = 0.f;
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    load8(w + (size_t)r * C + c0 + v * 8, f + v * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[v * 8 + j]));
  }
  am = np::warp_max(am);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
  __syncthreads();
  am = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) am = fmaxf(am, red[i]);
  const float scale = fmaxf(am, 1e-12f) / 448.f, inv = 1.f / scale;
#pragma unroll
  for (int v = 0; v < 8; ++v)
    *reinterpret_cast<uint2*>(q + (size_t)r * C + c0 + v * 8) = quant8(f + v * 8, inv);
  if (threadIdx.x == 0) scales[(size_t)tr * (C >> 7) + tc] = scale;
}

// One CTA (128 threads) per 128x128 tile. Input rows are dequantised into shared memory; thread j then
// owns input column j = output row j: amax over its 128 values, new scale, quantise, 128 contiguous bytes out.
__global__ void __launch_bounds__(128) transpose_1x128_kernel(const uint8_t* __restrict__ q,
                                                              const float* __restrict__ s, uint8_t* __restrict__ qt,
                                                              float* __restrict__ st, int M, int N) {
  extern __shared__ float tile_raw[];
  float (*tile)[129] = reinterpret_cast<float (*)[129]>(tile_raw);
  const int tm = blockIdx.y, tn = blockIdx.x;
  const int t = threadIdx.x;
  {
    const int row = tm * 128 + t;
    const float sc = s[(size_t)row * (N >> 7) + tn];
    const uint8_t* src = q + (size_t)row * N + tn * 128;
#pragma unroll 4
    for (int v = 0; v < 16; ++v) {
      const uint2 u = reinterpret_cast<const uint2*>(src)[v];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        tile[t][v * 8 + j] = from_e4m3(u.x >> (8 * j)) * sc;
        tile[t][v * 8 + 4 + j] = from_e4m3(u.y >> (8 * j)) * sc;
      }
    }
  }
  __syncthreads();
  float am = 0.f;
  for (int i = 0; i < 128; ++i) am = fmaxf(am, fabsf(tile[i][t]));
  const float scale = fmaxf(am, 1e-12f) / 448.f, inv = 1.f / scale;
  uint8_t* dst = qt + (size_t)(tn * 128 + t) * M + tm * 128;
  for (int v = 0; v < 16; ++v) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = tile[v * 8 + j][t];
    reinterpret_cast<uint2*>(dst)[v] = quant8(f, inv);
  }
  st[(size_t)(tn * 128 + t) * (M >> 7) + tm] = scale;
}

}  // namespace

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 500 + (int)e_; } while (0)

static int grid_for_blocks(long long nblocks) {
  long long g = (nblocks * 16 + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

NP_API int np_quant_1x128(const void* x, void* q, float* scales, long long rows, long long cols, void* stream) {
  if (cols % 128) return 1;
  const long long nb = rows * (cols / 128);
  if (nb <= 0) return 0;
  quant_1x128_kernel<<<grid_for_blocks(nb), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, nullptr,
                                                                           (uint8_t*)q, scales, nb, 0,
                                                                           (int)(cols / 128), cols, cols);
  CHECK_LAUNCH();
}
// gate / up: [rows, cols] views with row strides gate_ld / up_ld (elements; 0 = contiguous)
NP_API int np_swiglu_quant(const void* gate, const void* up, void* q, float* scales, long long rows, long long cols,
                           long long gate_ld, long long up_ld, void* stream) {
  if (cols % 128 || gate_ld % 8 || up_ld % 8) return 1;
  const long long nb = rows * (cols / 128);
  if (nb <= 0) return 0;
  quant_1x128_kernel<<<grid_for_blocks(nb), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (uint8_t*)q, scales, nb, 1, (int)(cols / 128),
      gate_ld ? gate_ld : cols, up_ld ? up_ld : cols);
  CHECK_LAUNCH();
}
NP_API int np_dequant_1x128(const void* q, const float* scales, void* out, long long rows, long long cols,
                            void* stream) {
  if (cols % 128) return 1;
  const long long nvec = rows * cols / 8;
  if (nvec <= 0) return 0;
  long long g = (nvec + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  dequant_1x128_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, scales, (__nv_bfloat16*)out, nvec);
  CHECK_LAUNCH();
}
NP_API int np_quant_128x128(const void* w, void* q, float* scales, int R, int C, void* stream) {
  if (R % 128 || C % 128) return 1;
  if (R <= 0 || C <= 0) return 0;
  quant_128x128_kernel<<<dim3(C / 128, R / 128), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q,
                                                                                scales, R, C);
  CHECK_LAUNCH();
}
NP_API int np_transpose_1x128(const void* q, const float* s, void* qt, float* st, int M, int N, void* stream) {
  if (M % 128 || N % 128) return 1;
  if (M <= 0 || N <= 0) return 0;
  constexpr int SMEM = 128 * 129 * 4;
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(transpose_1x128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  transpose_1x128_kernel<<<dim3(N / 128, M / 128), 128, SMEM, (cudaStream_t)stream>>>((const uint8_t*)q, s, (uint8_t*)qt,
                                                                                  st, M, N);
  CHECK_LAUNCH();
}
