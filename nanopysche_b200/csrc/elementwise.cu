// Bandwidth-bound training kernels for sm_100a: RMSNorm fwd/bwd (with fused residual add),
// SwiGLU / GeGLU fwd/bwd, RoPE fwd/bwd over strided head views, RoPE table generation
// (piecewise and YaRN scaling), cross-entropy fwd/bwd, fused AdamW on fp32 masters writing bf16
// weights, and sum-of-squares partials for gradient clipping.
//
// Each one replaces a chain of ATen pointwise/reduce launches in the reference
// (model/norm.py:38-47, model/feed_forward.py:64-75, model/rope.py:98-170,
//  model/transformer.py:451-458, optim/adamw.py:74-121, train/trainer.py:280-284).
// All are single-pass over HBM with 16-byte vector accesses.
#include "common.cuh"
#include "noalloc.h"

namespace {

constexpr int NT = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = np::warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (int)(blockDim.x >> 5)) ? red[l] : 0.f;
  t = np::warp_sum(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = np::warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (int)(blockDim.x >> 5)) ? red[l] : -INFINITY;
  t = np::warp_max(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void ld8f(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  *reinterpret_cast<uint4*>(p) = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                            np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
}

// ------------------------------------------------------------------ RMSNorm
// y = (x [+ res]) * rsqrt(mean((x+res)^2) + eps) * w ; optionally writes h = x + res.
// cols must be a multiple of 8 and <= NT*8*MAXV.
template <int MAXV>
__global__ void __launch_bounds__(NT) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ res,
                                                         const float* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ y,
                                                         __nv_bfloat16* __restrict__ h_out,
                                                         float* __restrict__ rstd, int rows, int cols,
                                                         float eps) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)r * cols;
    float v[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
        if (res) {
          float t[8];
          load8(res + (size_t)r * cols + c * 8, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += t[j];
        }
        if (h_out) {
          // round to bf16 first so the normalised value matches what later readers of h see
          store8(h_out + (size_t)r * cols + c * 8, v[i]);
          if (res) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)cols + eps);
    if (threadIdx.x == 0 && rstd) rstd[r] = rs;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
        const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
        o[0] = v[i][0] * rs * w0.x; o[1] = v[i][1] * rs * w0.y; o[2] = v[i][2] * rs * w0.z; o[3] = v[i][3] * rs * w0.w;
        o[4] = v[i][4] * rs * w1.x; o[5] = v[i][5] * rs * w1.y; o[6] = v[i][6] * rs * w1.z; o[7] = v[i][7] * rs * w1.w;
        store8(y + (size_t)r * cols + c * 8, o);
      }
    }
  }
}

// RMSNorm forward with an e4m3 output for an fp8 GEMM that follows: the normalised row (rounded to bf16 first, so the
// result equals quantising the bf16 output of the plain kernel) is quantised per 1x128 block with an fp32 scale
// amax / 448; y (bf16) is optional. cols must be a multiple of 128: a block is the 16 consecutive threads of a
// half-warp, 8 elements each.
template <int MAXV>
__global__ void __launch_bounds__(NT) rmsnorm_quant_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ res,
                                                               const float* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y,
                                                               __nv_bfloat16* __restrict__ h_out,
                                                               float* __restrict__ rstd, uint8_t* __restrict__ q,
                                                               float* __restrict__ scales, int rows, int cols,
                                                               float eps) {
  __shared__ float red[32];
  const int nvec = cols >> 3, bpr = cols >> 7;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)r * cols;
    float v[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
        if (res) {
          float t[8];
          load8(res + (size_t)r * cols + c * 8, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += t[j];
        }
        if (h_out) {
          store8(h_out + (size_t)r * cols + c * 8, v[i]);
          if (res) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)cols + eps);
    if (threadIdx.x == 0 && rstd) rstd[r] = rs;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      const bool ok = c < nvec;       // whole half-warps are in or out (cols % 128 == 0): the shuffles stay converged
      float o[8];
      float am = 0.f;
      const int cc = ok ? c : 0;
      const float4 w0 = *reinterpret_cast<const float4*>(w + cc * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(w + cc * 8 + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = __bfloat162float(__float2bfloat16(v[i][j] * rs * wv[j]));
        am = fmaxf(am, fabsf(o[j]));
      }
#pragma unroll
      for (int d = 8; d > 0; d >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, d));
      const float scale = fmaxf(am, 1e-12f) / 448.f, inv = 1.f / scale;
      if (ok) {
        if (y) store8(y + (size_t)r * cols + c * 8, o);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo |= (uint32_t)__nv_cvt_float_to_fp8(o[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
          hi |= (uint32_t)__nv_cvt_float_to_fp8(o[4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        }
        *reinterpret_cast<uint2*>(q + (size_t)r * cols + c * 8) = make_uint2(lo, hi);
        if ((threadIdx.x & 15) == 0) scales[(size_t)r * bpr + (c >> 4)] = scale;
      }
    }
  }
}

// dx = rs * (w*dy - xhat * mean(w*dy*xhat)) [+ dres]; per-CTA partial dw into scratch[grid, cols].
template <int MAXV>
__global__ void __launch_bounds__(NT) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                         const __nv_bfloat16* __restrict__ x,
                                                         const float* __restrict__ w,
                                                         const float* __restrict__ rstd,
                                                         const __nv_bfloat16* __restrict__ dres,
                                                         __nv_bfloat16* __restrict__ dx,
                                                         float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  float dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  // The next row's loads are issued before this row's block-wide reduction, so their latency overlaps it.
  uint4 gq[MAXV], xq[MAXV];
  auto fetch = [&](int r) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (r < rows && c < nvec) {
        gq[i] = *reinterpret_cast<const uint4*>(dy + (size_t)r * cols + c * 8);
        xq[i] = *reinterpret_cast<const uint4*>(x + (size_t)r * cols + c * 8);
      }
    }
  };
  fetch(blockIdx.x);
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float rs = rstd[r];
    float g[MAXV][8], xh[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        unpack8(gq[i], g[i]);
        unpack8(xq[i], xh[i]);
      }
    }
    fetch(r + gridDim.x);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          dwacc[i][j] += g[i][j] * xh[i][j];
          g[i][j] *= ww[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    uint4 rq[MAXV];   // residual gradient of this row, in flight during the reduction
    if (dres) {
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int c = threadIdx.x + i * NT;
        if (c < nvec) rq[i] = *reinterpret_cast<const uint4*>(dres + (size_t)r * cols + c * 8);
      }
    }
    dot = block_sum(dot, red) / (float)cols;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float t[8];
          unpack8(rq[i], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        }
        store8(dx + (size_t)r * cols + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) {
      float* dst = dw_partial + (size_t)blockIdx.x * cols + c * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// out[c] (+)= sum_p partial[p, c] with 8 row lanes per 32-column strip (block 32 x 8) and four loads in flight per
// thread: the partial matrix is a few hundred rows tall, so one thread per column would be a serial chain of
// dependent loads.
__global__ void __launch_bounds__(256) colsum_tall_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                          int parts, int cols, int accumulate) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a4[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < cols) {
    int p = ty;
    for (; p + 24 < parts; p += 32) {
#pragma unroll
      for (int u = 0; u < 4; ++u) a4[u] += partial[(size_t)(p + 8 * u) * cols + c];
    }
    for (; p < parts; p += 8) a4[0] += partial[(size_t)p * cols + c];
  }
  red[ty][tx] = (a4[0] + a4[1]) + (a4[2] + a4[3]);
  __syncthreads();
  if (ty == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][tx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// RMSNorm backward with one warp per row (cols == 256 * VPL <= 2048): no block-wide reduction per row, so all rows
// of the grid are in flight at once. Every warp adds its dw contributions into a private shared-memory row
// (deterministic: no atomics); the eight rows are summed into one partial per CTA at the end. The row is read
// twice, the second time from L1, to keep the register count low enough for three CTAs per SM.
template <int VPL>
__global__ void __launch_bounds__(NT) rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy,
                                                              const __nv_bfloat16* __restrict__ x,
                                                              const float* __restrict__ w,
                                                              const float* __restrict__ rstd,
                                                              const __nv_bfloat16* __restrict__ dres,
                                                              __nv_bfloat16* __restrict__ dx,
                                                              float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float s_dw[];   // [8 warps][cols]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* mine = s_dw + (size_t)warp * cols;
  for (int i = lane; i < cols; i += 32) mine[i] = 0.f;
  __syncwarp();
  for (int r = blockIdx.x * 8 + warp; r < rows; r += gridDim.x * 8) {
    const float rs = rstd[r];
    const __nv_bfloat16* gy = dy + (size_t)r * cols;
    const __nv_bfloat16* xr = x + (size_t)r * cols;
    float dot = 0.f;
#pragma unroll 2
    for (int i = 0; i < VPL; ++i) {
      const int c = (lane + 32 * i) * 8;
      float g[8], xv[8], ww[8];
      load8(gy + c, g);
      load8(xr + c, xv);
      ld8f(w + c, ww);
      float4 a0 = *reinterpret_cast<float4*>(mine + c), a1 = *reinterpret_cast<float4*>(mine + c + 4);
      float acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = xv[j] * rs;
        acc[j] += g[j] * xh;
        dot += g[j] * ww[j] * xh;
      }
      *reinterpret_cast<float4*>(mine + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(mine + c + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    dot = np::warp_sum(dot) / (float)cols;
#pragma unroll 2
    for (int i = 0; i < VPL; ++i) {
      const int c = (lane + 32 * i) * 8;
      float g[8], xv[8], ww[8], o[8];
      load8(gy + c, g);
      load8(xr + c, xv);
      ld8f(w + c, ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (g[j] * ww[j] - xv[j] * rs * dot);
      if (dres) {
        float t[8];
        load8(dres + (size_t)r * cols + c, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += t[j];
      }
      store8(dx + (size_t)r * cols + c, o);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += NT) {
    float t = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) t += s_dw[(size_t)ww * cols + c];
    dw_partial[(size_t)blockIdx.x * cols + c] = t;
  }
}

// ------------------------------------------------------------------ SwiGLU / GeGLU
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}

// gu = [gate | up] rows of 2F; h = act(gate) * up
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                               long long rows, int F, int act) {
  const long long nvec = rows * (F >> 3);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (F >> 3);
    const int c = (int)(i - r * (F >> 3)) * 8;
    float g[8], u[8], o[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = (act == 0 ? np::silu_f(g[j]) : gelu_tanh_f(g[j])) * u[j];
    store8(h + r * F + c, o);
  }
}

__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                               __nv_bfloat16* __restrict__ dgu, long long rows, int F, int act) {
  const long long nvec = rows * (F >> 3);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (F >> 3);
    const int c = (int)(i - r * (F >> 3)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
    load8(dh + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a, da;
      if (act == 0) {
        const float s = 1.f / (1.f + __expf(-g[j]));
        a = g[j] * s;
        da = s * (1.f + g[j] * (1.f - s));
      } else {
        a = gelu_tanh_f(g[j]);
        da = gelu_tanh_grad(g[j]);
      }
      dg[j] = d[j] * u[j] * da;
      du[j] = d[j] * a;
    }
    store8(dgu + r * 2 * F + c, dg);
    store8(dgu + r * 2 * F + F + c, du);
  }
}

// ------------------------------------------------------------------ RoPE
// x: [T, H, hd] viewed with row stride ld (elements) and head stride hd; half-split rotation on
// the first rot dims: out[i] = x[i]*cos - x[i+rot/2]*sin ; out[i+rot/2] = x[i+rot/2]*cos + x[i]*sin.
// sign = -1 gives the inverse rotation (the backward pass). pos = pos_ids ? pos_ids[t] : t % S + off.
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const int* __restrict__ pos_ids, long long T, int S, int pos_off, int H, int hd,
                            int rot, long long ld_in, long long ld_out, float sign) {
  const int half = rot >> 1;
  const int vec_per_head = hd >> 3;
  const long long total = T * H * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int hh = (int)(th % H);
    const long long t = th / H;
    const int d0 = v * 8;
    const __nv_bfloat16* src = x + t * ld_in + (size_t)hh * hd;
    __nv_bfloat16* dst = out + t * ld_out + (size_t)hh * hd;
    float a[8];
    load8(src + d0, a);
    if (d0 < rot) {
      const int pos = pos_ids ? pos_ids[t] : (int)(t % S) + pos_off;
      const bool lo = d0 < half;
      const int pd = lo ? d0 + half : d0 - half;
      float b[8], o[8];
      load8(src + pd, b);
      const int f0 = lo ? d0 : d0 - half;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cos_t[(size_t)pos * half + f0 + j];
        const float s = sin_t[(size_t)pos * half + f0 + j] * sign;
        o[j] = lo ? (a[j] * c - b[j] * s) : (a[j] * c + b[j] * s);
      }
      store8(dst + d0, o);
    } else if (dst != src) {
      store8(dst + d0, a);
    }
  }
}

// Fused "split QKV + RoPE": one pass over the [T, H, hd] output of the QKV GEMM (H = hq + 2*hkv heads).
// Forward (sign=+1): heads [0, rot_heads) are rotated, the rest (V) copied, into one contiguous [T, H, hd]
// buffer whose q / k / v slices are then used as strided views. Backward (sign=-1): the three gradient
// tensors (separate row / head strides) are gathered into one contiguous dqkv with the inverse rotation.
struct HeadSrc {
  const __nv_bfloat16* p;
  long long row_stride, head_stride;
  int heads;
};
// One CTA per token; a thread takes a (head, 8-wide slice of the lower half) pair and produces both halves of the
// rotation from two 16-byte loads, so every input element is read once. Slices outside the rotated range and the
// V heads are copied.
__global__ void __launch_bounds__(256) qkv_rope_kernel(HeadSrc s0, HeadSrc s1, HeadSrc s2,
                                                       __nv_bfloat16* __restrict__ out,
                                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                       const int* __restrict__ pos_ids, long long T, int S, int pos_off,
                                                       int hd, int rot, int rot_heads, float sign) {
  const int H = s0.heads + s1.heads + s2.heads;
  const int half = rot >> 1;
  const int hv = half >> 3;                    // 8-wide slices in one half of the rotated range
  const int cv = (hd - rot) >> 3;              // slices of a rotated head that are only copied
  const int per_rot = hv + cv, per_plain = hd >> 3;
  const int items = rot_heads * per_rot + (H - rot_heads) * per_plain;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const int pos = pos_ids ? pos_ids[t] : (int)(t % S) + pos_off;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      int hh, v;
      bool rotate;
      if (it < rot_heads * per_rot) {
        hh = it / per_rot;
        v = it - hh * per_rot;
        rotate = v < hv;
      } else {
        const int r = it - rot_heads * per_rot;
        hh = rot_heads + r / per_plain;
        v = r % per_plain;
        rotate = false;
      }
      const __nv_bfloat16* src;
      if (hh < s0.heads) src = s0.p + t * s0.row_stride + (long long)hh * s0.head_stride;
      else if (hh < s0.heads + s1.heads) src = s1.p + t * s1.row_stride + (long long)(hh - s0.heads) * s1.head_stride;
      else src = s2.p + t * s2.row_stride + (long long)(hh - s0.heads - s1.heads) * s2.head_stride;
      __nv_bfloat16* dst = out + (t * H + hh) * (long long)hd;
      if (rotate) {
        const int d0 = v * 8;
        float a[8], b[8], lo[8], hi[8];
        load8(src + d0, a);
        load8(src + d0 + half, b);
        const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + d0);
        const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + d0 + 4);
        const float4 n0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + d0);
        const float4 n1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + d0 + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sj = sn[j] * sign;
          lo[j] = a[j] * c[j] - b[j] * sj;
          hi[j] = b[j] * c[j] + a[j] * sj;
        }
        store8(dst + d0, lo);
        store8(dst + d0 + half, hi);
      } else {
        const int d0 = (it < rot_heads * per_rot) ? rot + (v - hv) * 8 : v * 8;
        *reinterpret_cast<uint4*>(dst + d0) = *reinterpret_cast<const uint4*>(src + d0);
      }
    }
  }
}

// Fused "split QKV + per-head LayerNorm(q), LayerNorm(k) + RoPE" for head_dim 128 with full rotary. A head is
// handled by 8 neighbouring threads (16 elements each: an 8-wide slice of the lower half and its partner in the
// upper half), which share the LayerNorm statistics through shuffles inside their 8-lane group.
// Replaces q_norm / k_norm (nn.LayerNorm over head_dim) + apply_rotary_emb in the reference
// (model/attention.py:152-164, model/rope.py:139-170).
__device__ __forceinline__ float group8_sum(float v, unsigned mask) {
  v += __shfl_xor_sync(mask, v, 1);
  v += __shfl_xor_sync(mask, v, 2);
  v += __shfl_xor_sync(mask, v, 4);
  return v;
}

__global__ void __launch_bounds__(256) qkv_norm_rope_fwd_kernel(
    const __nv_bfloat16* __restrict__ qkv, long long row_stride, int hq, int hkv, const float* __restrict__ gq,
    const float* __restrict__ bq, const float* __restrict__ gk, const float* __restrict__ bk, float eps,
    __nv_bfloat16* __restrict__ out, float2* __restrict__ stats, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ pos_ids, long long T, int S, int pos_off) {
  constexpr int HD = 128, HALF = 64;
  const int nrot = hq + hkv, H = hq + 2 * hkv;
  const int items = nrot * 8 + hkv * 16;
  const unsigned mask = 0xffu << (threadIdx.x & 24);
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const int pos = pos_ids ? pos_ids[t] : (int)(t % S) + pos_off;
    const __nv_bfloat16* row = qkv + t * row_stride;
    __nv_bfloat16* orow = out + t * (long long)H * HD;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      if (it < nrot * 8) {
        const int hh = it >> 3, d0 = (it & 7) * 8;
        float a[8], b[8];
        load8(row + hh * HD + d0, a);
        load8(row + hh * HD + d0 + HALF, b);
        float sm = 0.f, sq = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { sm += a[j] + b[j]; sq += a[j] * a[j] + b[j] * b[j]; }
        sm = group8_sum(sm, mask);
        sq = group8_sum(sq, mask);
        const float mean = sm * (1.f / HD);
        const float rstd = rsqrtf(fmaxf(sq * (1.f / HD) - mean * mean, 0.f) + eps);
        const float* g = hh < hq ? gq : gk;
        const float* be = hh < hq ? bq : bk;
        float gl[8], gh[8], bl[8], bh[8], c[8], sn[8], lo[8], hi[8];
        ld8f(g + d0, gl); ld8f(g + d0 + HALF, gh); ld8f(be + d0, bl); ld8f(be + d0 + HALF, bh);
        ld8f(cos_t + (size_t)pos * HALF + d0, c);
        ld8f(sin_t + (size_t)pos * HALF + d0, sn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // the normalised value passes through bf16 like the output of the unfused LayerNorm
          const float na = __bfloat162float(__float2bfloat16((a[j] - mean) * rstd * gl[j] + bl[j]));
          const float nb = __bfloat162float(__float2bfloat16((b[j] - mean) * rstd * gh[j] + bh[j]));
          lo[j] = na * c[j] - nb * sn[j];
          hi[j] = nb * c[j] + na * sn[j];
        }
        store8(orow + hh * HD + d0, lo);
        store8(orow + hh * HD + d0 + HALF, hi);
        if ((it & 7) == 0) stats[t * nrot + hh] = make_float2(mean, rstd);
      } else {
        const int r = it - nrot * 8;
        const int off = (nrot + (r >> 4)) * HD + (r & 15) * 8;
        *reinterpret_cast<uint4*>(orow + off) = *reinterpret_cast<const uint4*>(row + off);
      }
    }
  }
}

// Backward: inverse rotation of dq / dk, LayerNorm backward against the saved pre-norm values and statistics,
// dv copied; the three results form one contiguous dqkv. The gamma / beta gradients are accumulated per thread
// (a thread keeps its (head, slice) across tokens), summed over the heads of a kind in shared memory and written as
// one partial row [4 x 128] per CTA (dgamma_q, dbeta_q, dgamma_k, dbeta_k).
__global__ void __launch_bounds__(256) qkv_norm_rope_bwd_kernel(
    HeadSrc s0, HeadSrc s1, HeadSrc s2, const __nv_bfloat16* __restrict__ qkv, long long row_stride, int hq, int hkv,
    const float* __restrict__ gq, const float* __restrict__ gk, const float2* __restrict__ stats,
    __nv_bfloat16* __restrict__ dqkv, float* __restrict__ partial, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ pos_ids, long long T, int S, int pos_off) {
  constexpr int HD = 128, HALF = 64;
  __shared__ float s_acc[4][HD];
  const int nrot = hq + hkv, H = hq + 2 * hkv;
  const int items = nrot * 8 + hkv * 16;
  const unsigned mask = 0xffu << (threadIdx.x & 24);
  for (int i = threadIdx.x; i < 4 * HD; i += blockDim.x) (&s_acc[0][0])[i] = 0.f;
  float dg[2][16], db[2][16];   // up to two rotated items per thread (nrot * 8 <= 512)
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int j = 0; j < 16; ++j) { dg[u][j] = 0.f; db[u][j] = 0.f; }
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const int pos = pos_ids ? pos_ids[t] : (int)(t % S) + pos_off;
    const __nv_bfloat16* row = qkv + t * row_stride;
    __nv_bfloat16* orow = dqkv + t * (long long)H * HD;
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int it = threadIdx.x + u * 256;
      if (it >= items) break;
      if (it < nrot * 8) {
        const int hh = it >> 3, d0 = (it & 7) * 8;
        const __nv_bfloat16* gsrc = hh < hq ? s0.p + t * s0.row_stride + (long long)hh * s0.head_stride
                                            : s1.p + t * s1.row_stride + (long long)(hh - hq) * s1.head_stride;
        float dl[8], dh[8], a[8], b[8], c[8], sn[8], gl[8], gh[8];
        load8(gsrc + d0, dl);
        load8(gsrc + d0 + HALF, dh);
        load8(row + hh * HD + d0, a);
        load8(row + hh * HD + d0 + HALF, b);
        ld8f(cos_t + (size_t)pos * HALF + d0, c);
        ld8f(sin_t + (size_t)pos * HALF + d0, sn);
        const float* g = hh < hq ? gq : gk;
        ld8f(g + d0, gl); ld8f(g + d0 + HALF, gh);
        const float2 st = stats[t * nrot + hh];
        float ya[8], yb[8], xa[8], xb[8];
        float m1 = 0.f, m2 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ya[j] = dl[j] * c[j] + dh[j] * sn[j];   // gradient at the LayerNorm output
          yb[j] = dh[j] * c[j] - dl[j] * sn[j];
          xa[j] = (a[j] - st.x) * st.y;
          xb[j] = (b[j] - st.x) * st.y;
          if (u < 2) {
            dg[u][j] += ya[j] * xa[j]; dg[u][8 + j] += yb[j] * xb[j];
            db[u][j] += ya[j]; db[u][8 + j] += yb[j];
          }
          ya[j] *= gl[j];
          yb[j] *= gh[j];
          m1 += ya[j] + yb[j];
          m2 += ya[j] * xa[j] + yb[j] * xb[j];
        }
        m1 = group8_sum(m1, mask) * (1.f / HD);
        m2 = group8_sum(m2, mask) * (1.f / HD);
        float oa[8], ob[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          oa[j] = st.y * (ya[j] - m1 - xa[j] * m2);
          ob[j] = st.y * (yb[j] - m1 - xb[j] * m2);
        }
        store8(orow + hh * HD + d0, oa);
        store8(orow + hh * HD + d0 + HALF, ob);
      } else {
        const int r = it - nrot * 8;
        const int hv = r >> 4, d0 = (r & 15) * 8;
        *reinterpret_cast<uint4*>(orow + (nrot + hv) * HD + d0) =
            *reinterpret_cast<const uint4*>(s2.p + t * s2.row_stride + (long long)hv * s2.head_stride + d0);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int it = threadIdx.x + u * 256;
    if (it < nrot * 8) {
      const int kind = (it >> 3) < hq ? 0 : 2, d0 = (it & 7) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&s_acc[kind][d0 + j], dg[u][j]);
        atomicAdd(&s_acc[kind][d0 + HALF + j], dg[u][8 + j]);
        atomicAdd(&s_acc[kind + 1][d0 + j], db[u][j]);
        atomicAdd(&s_acc[kind + 1][d0 + HALF + j], db[u][8 + j]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 4 * HD; i += blockDim.x) partial[(size_t)blockIdx.x * 4 * HD + i] = (&s_acc[0][0])[i];
}

// cos/sin tables [S, rot/2] in fp32.
// scaling: 0 none; 1 piecewise (wavelen < orig/high_freq keeps, wavelen > orig/low_freq divides by
// factor, the band between keeps: the reference's rule, model/rope.py:64-80); 2 YaRN (NTK-by-parts
// linear ramp between beta_fast/beta_slow rotations, cos/sin multiplied by mscale).
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int S, int rot,
                                  float base, int scaling, float factor, float orig_len, float low_f,
                                  float high_f, float mscale) {
  const int half = rot >> 1;
  const long long total = (long long)S * half;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int f = (int)(i % half);
    const int pos = (int)(i / half);
    float inv = powf(base, -2.f * (float)f / (float)rot);
    float ms = 1.f;
    if (scaling == 1) {
      const float wavelen = 6.283185307179586f / inv;
      if (!(wavelen < orig_len / high_f) && wavelen > orig_len / low_f) inv = inv / factor;
    } else if (scaling == 2) {
      // low_f = beta_slow (default 1), high_f = beta_fast (default 32)
      const float lnb = logf(base);
      const float d_lo = (float)rot * logf(orig_len / (high_f * 6.283185307179586f)) / (2.f * lnb);
      const float d_hi = (float)rot * logf(orig_len / (low_f * 6.283185307179586f)) / (2.f * lnb);
      const float lo = fmaxf(floorf(d_lo), 0.f), hi = fminf(ceilf(d_hi), (float)(half - 1));
      float ramp = ((float)f - lo) / fmaxf(hi - lo, 1e-3f);
      ramp = fminf(fmaxf(ramp, 0.f), 1.f);
      const float extrap = 1.f - ramp;  // 1 = keep original frequency
      inv = (inv / factor) * (1.f - extrap) + inv * extrap;
      ms = mscale;
    }
    const float ang = (float)pos * inv;
    cos_t[i] = cosf(ang) * ms;
    sin_t[i] = sinf(ang) * ms;
  }
}

// ------------------------------------------------------------------ cross-entropy
// Row-wise: lse[r] = logsumexp(logits[r]), loss[r] = lse - logits[r, label] (0 if label == ignore).
__global__ void __launch_bounds__(NT) xent_fwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                      const long long* __restrict__ labels,
                                                      float* __restrict__ loss, float* __restrict__ lse,
                                                      int rows, int V, long long ld, long long ignore) {
  __shared__ float red[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* lr = logits + (size_t)r * ld;
    const int nvec = V >> 3;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < nvec; c += NT) {
      float f[8];
      load8(lr + c * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += NT) mx = fmaxf(mx, __bfloat162float(lr[c]));
    mx = block_max(mx, red);
    float se = 0.f;
    for (int c = threadIdx.x; c < nvec; c += NT) {
      float f[8];
      load8(lr + c * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += NT) se += __expf(__bfloat162float(lr[c]) - mx);
    se = block_sum(se, red);
    if (threadIdx.x == 0) {
      const float l = mx + logf(se);
      lse[r] = l;
      const long long lab = labels[r];
      loss[r] = (lab == ignore || lab < 0 || lab >= V) ? 0.f : l - __bfloat162float(lr[lab]);
    }
  }
}

// dlogits[r, c] = (exp(logits - lse) - [c == label]) * gscale[0] * inv_count[0]; ignored rows -> 0.
__global__ void __launch_bounds__(NT) xent_bwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                      const long long* __restrict__ labels,
                                                      const float* __restrict__ lse,
                                                      const float* __restrict__ gscale,
                                                      const float* __restrict__ inv_count,
                                                      __nv_bfloat16* __restrict__ dlogits, int rows, int V,
                                                      long long ld, long long ignore) {
  const float sc = gscale[0] * inv_count[0];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* lr = logits + (size_t)r * ld;
    __nv_bfloat16* dr = dlogits + (size_t)r * ld;
    const long long lab = labels[r];
    const bool ign = (lab == ignore || lab < 0 || lab >= V);
    const float l = lse[r];
    const int nvec = V >> 3;
    for (int c = threadIdx.x; c < nvec; c += NT) {
      float f[8], o[8];
      load8(lr + c * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float pr = __expf(f[j] - l);
        o[j] = ign ? 0.f : (pr - ((long long)(c * 8 + j) == lab ? 1.f : 0.f)) * sc;
      }
      store8(dr + c * 8, o);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += NT) {
      const float pr = __expf(__bfloat162float(lr[c]) - l);
      dr[c] = __float2bfloat16(ign ? 0.f : (pr - ((long long)c == lab ? 1.f : 0.f)) * sc);
    }
  }
}

// ------------------------------------------------------------------ AdamW + norms
// Decoupled weight decay on fp32 masters; writes the bf16 compute copy in the same pass.
// gscale (device scalar, may be null) multiplies the gradient (gradient clipping coefficient).
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ w16, long long n, float lr,
                             float b1, float b2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ gscale, const float* __restrict__ hyper) {
  const float gs = gscale ? gscale[0] : 1.f;
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }  // device-resident schedule (graph replay)
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* P = &pp.x; const float* G = &gg.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = G[j] * gs;
      M[j] = b1 * M[j] + (1.f - b1) * gr;
      V[j] = b2 * V[j] + (1.f - b2) * gr * gr;
      const float den = sqrtf(V[j] / bc2) + eps;
      P[j] = P[j] * (1.f - lr * wd) - lr * (M[j] / bc1) / den;
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (w16) reinterpret_cast<uint2*>(w16)[i] = make_uint2(np::pack_bf16(pp.x, pp.y), np::pack_bf16(pp.z, pp.w));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = nvec * 4; i < n; ++i) {
      const float gr = g[i] * gs;
      m[i] = b1 * m[i] + (1.f - b1) * gr;
      v[i] = b2 * v[i] + (1.f - b2) * gr * gr;
      p[i] = p[i] * (1.f - lr * wd) - lr * (m[i] / bc1) / (sqrtf(v[i] / bc2) + eps);
      if (w16) w16[i] = __float2bfloat16(p[i]);
    }
  }
}

// partial[b] = sum over this CTA's grid-stride slice of x^2 (fp32 input)
__global__ void __launch_bounds__(NT) sumsq_kernel(const float* __restrict__ x, long long n,
                                                   float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec * 4; i < n; ++i) s += x[i] * x[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// out[0] = min(1, max_norm / (sqrt(sum(partial) + extra_sq[0]) + 1e-6)); out[1] = the norm.
__global__ void clip_coef_kernel(const float* __restrict__ partial, int parts, const float* __restrict__ extra_sq,
                                 float max_norm, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    if (extra_sq) s += extra_sq[0];
    const float nrm = sqrtf(s);
    out[1] = nrm;
    out[0] = max_norm > 0.f ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<uint2*>(y)[i] = make_uint2(np::pack_bf16(a.x, a.y), np::pack_bf16(a.z, a.w));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec * 4; i < n; ++i) y[i] = __float2bfloat16(x[i]);
}

inline int grid_for(long long work_items, int threads, int cap) {
  long long g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}
constexpr int GRID_CAP = 148 * 8;

}  // namespace

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 500 + (int)e_; } while (0)

NP_API int np_rmsnorm_fwd(const void* x, const void* res, const float* w, void* y, void* h_out, float* rstd,
                          int rows, int cols, float eps, void* stream) {
  if (cols % 8 || cols > NT * 8 * 4) return 1;
  const int grid = rows < GRID_CAP ? rows : GRID_CAP;
  if (grid <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (cols <= NT * 8)
    rmsnorm_fwd_kernel<1><<<grid, NT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w,
                                              (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, cols, eps);
  else if (cols <= NT * 16)
    rmsnorm_fwd_kernel<2><<<grid, NT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w,
                                              (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, cols, eps);
  else
    rmsnorm_fwd_kernel<4><<<grid, NT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w,
                                              (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, cols, eps);
  CHECK_LAUNCH();
}

// RMSNorm (+ residual) with an e4m3 + 1x128-scale output (q [rows, cols] bytes, scales [rows, cols / 128] fp32);
// y may be null when only the quantised output is wanted. cols a multiple of 128.
NP_API int np_rmsnorm_quant_fwd(const void* x, const void* res, const float* w, void* y, void* h_out, float* rstd,
                                void* q, float* scales, int rows, int cols, float eps, void* stream) {
  if (cols % 128 || cols > NT * 8 * 4) return 1;
  const int grid = rows < GRID_CAP ? rows : GRID_CAP;
  if (grid <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
#define RQ(V) rmsnorm_quant_fwd_kernel<V><<<grid, NT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w, \
      (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, (uint8_t*)q, scales, rows, cols, eps)
  if (cols <= NT * 8) RQ(1);
  else if (cols <= NT * 16) RQ(2);
  else RQ(4);
#undef RQ
  CHECK_LAUNCH();
}

// The backward kernel followed by the column sum of its partials. Returns 0, or 400 + the CUDA error of the
// shared-memory attribute call (made once per device).
static int launch_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                               void* dx, float* dw, float* scratch, int rows, int cols, int accumulate_dw, int grid,
                               cudaStream_t s) {
#define RB(V) rmsnorm_bwd_kernel<V><<<grid, NT, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, rstd, \
                                                       (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, rows, cols)
#define RBW(V) rmsnorm_bwd_warp_kernel<V><<<grid, NT, 8 * cols * sizeof(float), s>>>( \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, \
      rows, cols)
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {   // the warp-per-row kernels keep 8 x cols floats in shared memory (64 KB at 2048 columns)
    cudaError_t ea = cudaFuncSetAttribute(rmsnorm_bwd_warp_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2048 * 4);
    if (ea == cudaSuccess)
      ea = cudaFuncSetAttribute(rmsnorm_bwd_warp_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 1024 * 4);
    if (ea != cudaSuccess) return 400 + (int)ea;
    attr_set = true;
  }
  if (cols == 2048) RBW(8);
  else if (cols == 1024) RBW(4);
  else if (cols <= NT * 8) RB(1);
  else if (cols <= NT * 16) RB(2);
  else RB(4);
#undef RB
#undef RBW
  colsum_tall_kernel<<<(cols + 31) / 32, 256, 0, s>>>(scratch, dw, grid, cols, accumulate_dw);
  return 0;
}

// Number of partial rows np_rmsnorm_bwd writes into its scratch for a given row count.
NP_API int np_rmsnorm_bwd_parts(int rows) {
  const int cap = 148 * 2;
  return rows < cap ? (rows > 0 ? rows : 1) : cap;
}

// scratch: fp32 [np_rmsnorm_bwd_parts(rows), cols]. dw (+)= column sums of dy * xhat.
NP_API int np_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                          void* dx, float* dw, float* scratch, int rows, int cols, int accumulate_dw,
                          void* stream) {
  if (cols % 8 || cols > NT * 8 * 4) return 1;
  if (rows <= 0) return 0;
  const int grid = np_rmsnorm_bwd_parts(rows);
  const int rc_attr = launch_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw, scratch, rows, cols, accumulate_dw, grid,
                                         (cudaStream_t)stream);
  if (rc_attr) return rc_attr;
  CHECK_LAUNCH();
}

NP_API int np_glu_fwd(const void* gu, void* h, long long rows, int F, int act, void* stream) {
  if (F % 8) return 1;
  if (rows <= 0) return 0;
  glu_fwd_kernel<<<grid_for(rows * (F / 8), 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, rows, F, act);
  CHECK_LAUNCH();
}
NP_API int np_glu_bwd(const void* gu, const void* dh, void* dgu, long long rows, int F, int act, void* stream) {
  if (F % 8) return 1;
  if (rows <= 0) return 0;
  glu_bwd_kernel<<<grid_for(rows * (F / 8), 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dh, (__nv_bfloat16*)dgu, rows, F, act);
  CHECK_LAUNCH();
}

NP_API int np_rope(const void* x, void* out, const float* cos_t, const float* sin_t, const int* pos_ids,
                   long long T, int S, int pos_off, int H, int hd, int rot, long long ld_in, long long ld_out,
                   float sign, void* stream) {
  if (hd % 8 || rot % 16 || rot > hd || ld_in % 8 || ld_out % 8) return 1;
  if (T <= 0) return 0;
  rope_kernel<<<grid_for(T * H * (hd / 8), 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)out, cos_t, sin_t, pos_ids, T, S, pos_off, H, hd, rot, ld_in,
      ld_out, sign);
  CHECK_LAUNCH();
}

// Sources i = 0..2: pointer, row stride and head stride (elements), head count; out: contiguous [T, H, hd].
NP_API int np_qkv_rope(const void* p0, long long rs0, long long hs0, int h0, const void* p1, long long rs1,
                       long long hs1, int h1, const void* p2, long long rs2, long long hs2, int h2, void* out,
                       const float* cos_t, const float* sin_t, const int* pos_ids, long long T, int S, int pos_off,
                       int hd, int rot, int rot_heads, float sign, void* stream) {
  if (hd % 8 || rot % 16 || rot > hd || (rs0 | hs0 | rs1 | hs1 | rs2 | hs2) % 8) return 1;
  if (T <= 0) return 0;
  HeadSrc s0{(const __nv_bfloat16*)p0, rs0, hs0, h0}, s1{(const __nv_bfloat16*)p1, rs1, hs1, h1},
      s2{(const __nv_bfloat16*)p2, rs2, hs2, h2};
  qkv_rope_kernel<<<(unsigned)(T < GRID_CAP ? T : GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      s0, s1, s2, (__nv_bfloat16*)out, cos_t, sin_t, pos_ids, T, S, pos_off, hd, rot, rot_heads, sign);
  CHECK_LAUNCH();
}

// Fused split + LayerNorm(q), LayerNorm(k) + RoPE (head_dim 128, full rotary). qkv: rows of (hq + 2 hkv) * 128 with
// row stride `row_stride`; out: contiguous [T, hq + 2 hkv, 128]; stats: (mean, rstd) per (token, q or k head).
NP_API int np_qkv_norm_rope_fwd(const void* qkv, long long row_stride, int hq, int hkv, const float* gq,
                                const float* bq, const float* gk, const float* bk, float eps, void* out, void* stats,
                                const float* cos_t, const float* sin_t, const int* pos_ids, long long T, int S,
                                int pos_off, void* stream) {
  if (row_stride % 8 || (hq + hkv) * 8 > 512 || (hq + hkv) * 8 + hkv * 16 > 768) return 1;
  if (T <= 0) return 0;
  qkv_norm_rope_fwd_kernel<<<(unsigned)(T < GRID_CAP ? T : GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, row_stride, hq, hkv, gq, bq, gk, bk, eps, (__nv_bfloat16*)out, (float2*)stats, cos_t,
      sin_t, pos_ids, T, S, pos_off);
  CHECK_LAUNCH();
}
NP_API int np_qkv_norm_rope_parts(long long T) { return (int)(T < 296 ? (T > 0 ? T : 1) : 296); }
// dparams[4 * 128] (+)= (dgamma_q, dbeta_q, dgamma_k, dbeta_k); scratch: fp32 [np_qkv_norm_rope_parts(T), 4 * 128].
NP_API int np_qkv_norm_rope_bwd(const void* dq, long long rs0, long long hs0, const void* dk, long long rs1,
                                long long hs1, const void* dv, long long rs2, long long hs2, const void* qkv,
                                long long row_stride, int hq, int hkv, const float* gq, const float* gk,
                                const void* stats, void* dqkv, float* dparams, float* scratch, const float* cos_t,
                                const float* sin_t, const int* pos_ids, long long T, int S, int pos_off,
                                int accumulate, void* stream) {
  if ((row_stride | rs0 | hs0 | rs1 | hs1 | rs2 | hs2) % 8 || (hq + hkv) * 8 > 512 || (hq + hkv) * 8 + hkv * 16 > 768)
    return 1;
  if (T <= 0) return 0;
  HeadSrc s0{(const __nv_bfloat16*)dq, rs0, hs0, hq}, s1{(const __nv_bfloat16*)dk, rs1, hs1, hkv},
      s2{(const __nv_bfloat16*)dv, rs2, hs2, hkv};
  const int grid = np_qkv_norm_rope_parts(T);
  cudaStream_t s = (cudaStream_t)stream;
  qkv_norm_rope_bwd_kernel<<<grid, 256, 0, s>>>(s0, s1, s2, (const __nv_bfloat16*)qkv, row_stride, hq, hkv, gq, gk,
                                                (const float2*)stats, (__nv_bfloat16*)dqkv, scratch, cos_t, sin_t,
                                                pos_ids, T, S, pos_off);
  colsum_tall_kernel<<<(4 * 128 + 31) / 32, 256, 0, s>>>(scratch, dparams, grid, 4 * 128, accumulate);
  CHECK_LAUNCH();
}

NP_API int np_rope_table(float* cos_t, float* sin_t, int S, int rot, float base, int scaling, float factor,
                         float orig_len, float low_f, float high_f, float mscale, void* stream) {
  if (S <= 0) return 0;
  rope_table_kernel<<<grid_for((long long)S * (rot / 2), 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      cos_t, sin_t, S, rot, base, scaling, factor, orig_len, low_f, high_f, mscale);
  CHECK_LAUNCH();
}

NP_API int np_xent_fwd(const void* logits, const long long* labels, float* loss, float* lse, int rows, int V,
                       long long ld, long long ignore, void* stream) {
  if (ld % 8) return 1;
  if (rows <= 0) return 0;
  xent_fwd_kernel<<<rows < GRID_CAP ? rows : GRID_CAP, NT, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, labels, loss, lse, rows, V, ld, ignore);
  CHECK_LAUNCH();
}
NP_API int np_xent_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
                       const float* inv_count, void* dlogits, int rows, int V, long long ld, long long ignore,
                       void* stream) {
  if (ld % 8) return 1;
  if (rows <= 0) return 0;
  xent_bwd_kernel<<<rows < GRID_CAP ? rows : GRID_CAP, NT, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, labels, lse, gscale, inv_count, (__nv_bfloat16*)dlogits, rows, V, ld, ignore);
  CHECK_LAUNCH();
}

NP_API int np_adamw(float* p, const float* g, float* m, float* v, void* w16, long long n, float lr, float b1,
                    float b2, float eps, float wd, int step, const float* gscale, const float* hyper, void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<grid_for(n / 4 + 1, 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      p, g, m, v, (__nv_bfloat16*)w16, n, lr, b1, b2, eps, wd, bc1, bc2, gscale, hyper);
  CHECK_LAUNCH();
}

NP_API int np_sumsq_parts() { return 148 * 4; }
// partial: fp32 [np_sumsq_parts()]
NP_API int np_sumsq(const float* x, long long n, float* partial, void* stream) {
  sumsq_kernel<<<np_sumsq_parts(), NT, 0, (cudaStream_t)stream>>>(x, n, partial);
  CHECK_LAUNCH();
}
// Embedding backward straight into the fp32 gradient arena: grad[ids[t], :] += dy[t, :]. One thread per four
// columns of a token row, one 16-byte vector reduction each; rows of ids outside [0, V) are skipped.
namespace {
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const long long* __restrict__ ids, float* __restrict__ grad,
                                                            long long T, int D, long long V) {
  const int vec_per_row = D >> 2;
  const long long total = T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int d = (int)(i - t * vec_per_row) * 4;
    const long long row = ids[t];
    NP_DBG_SKIP_UNLESS(row >= 0 && row < V, 40, row)   // a token id outside the vocabulary (debug build: reported)
    if (row < 0 || row >= V) continue;
    const uint2 u = *reinterpret_cast<const uint2*>(dy + t * D + d);
    const float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y);
    atomicAdd(reinterpret_cast<float4*>(grad + row * D + d), make_float4(a.x, a.y, b.x, b.y));
  }
}
}  // namespace

NP_API int np_embedding_bwd(const void* dy, const long long* ids, float* grad, long long T, int D, long long V,
                            int zero_first, void* stream) {
  if (T <= 0) return 0;
  if (D % 4 || (((uintptr_t)dy) & 7) || (((uintptr_t)grad) & 15)) return 1;
  cudaStream_t s = (cudaStream_t)stream;
  if (zero_first) {
    cudaError_t e = cudaMemsetAsync(grad, 0, (size_t)V * D * sizeof(float), s);
    if (e != cudaSuccess) return 400 + (int)e;
  }
  long long blocks = (T * (D / 4) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  embedding_bwd_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)dy, ids, grad, T, D, V);
  CHECK_LAUNCH();
}

NP_API int np_clip_coef(const float* partial, int parts, const float* extra_sq, float max_norm, float* out2,
                        void* stream) {
  clip_coef_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(partial, parts, extra_sq, max_norm, out2);
  CHECK_LAUNCH();
}
NP_API int np_cast_f32_bf16(const float* x, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n / 4 + 1, 256, GRID_CAP), 256, 0, (cudaStream_t)stream>>>(
      x, (__nv_bfloat16*)y, n);
  CHECK_LAUNCH();
}

// ------------------------------------------------------------------ allocation-free variant
// Scratch for np_rmsnorm_bwd_noalloc: per-CTA partial sums of the weight gradient, [parts, cols].
// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address each device uses is resolved once with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[NP_NOALLOC_MAX_PARTS * NP_NOALLOC_MAX_COLS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

NP_API int np_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                                  void* dx, float* dw, int rows, int cols, int accumulate_dw, void* stream) {
  if (cols % 8) return 1;
  if (cols > NP_NOALLOC_MAX_COLS) return 3;  // beyond the static scratch: use np_rmsnorm_bwd with your own buffer
  if (rows <= 0) return 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return 400 + (int)e;
  if (dev < 0 || dev >= kMaxDevices) return 3;
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up for this device (it is the current one): device address of the static array
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return 400 + (int)e;
    g_noalloc_ptr[dev] = p;
  }
  float* scratch = g_noalloc_ptr[dev];
  const int grid = np_rmsnorm_bwd_parts(rows);  // <= NP_NOALLOC_MAX_PARTS
  // every partial row [0, grid) x [0, cols) is written by the first kernel, so the column sum reads nothing stale
  const int rc_attr = launch_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw, scratch, rows, cols, accumulate_dw, grid,
                                         (cudaStream_t)stream);
  if (rc_attr) return rc_attr;
  CHECK_LAUNCH();
}
