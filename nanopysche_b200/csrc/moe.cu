// MoE routing and expert-parallel token movement for sm_100a.
//
//  router_logits / router_topk / router_bwd : fp32 gate, DeepSeek-V3 score bias, top-k with softmax-
//      over-top-k or sigmoid+renorm gating, per-expert histogram, sum of full-softmax probabilities
//      and sum of logsumexp^2 (aux / z loss) in one pass; analytic backward to the logits.
//  capacity_scan : position of every token inside each expert it picked (index order), whole-token
//      drop beyond the capacity, positions among the kept tokens - no host sync.
//  ep_dispatch   : the all-to-all dispatch as peer stores: every kept (token, k) row is written
//      straight into the owning rank's expert-major receive buffer (region [local expert][source
//      rank], fixed size), optionally scaled (backward) or quantised to e4m3 with 1x128 scales
//      (FP8-Flow-MoE), together with the per-block row counts and per-row return addresses the
//      consuming grouped GEMM needs; the last CTA releases an epoch flag on every peer.
//  ep_combine    : waits (bounded) for the peers' epoch flags and reduces the K returned rows of each
//      token with the router weights, adding optional dense/shared/router-gradient terms.
//
// Replaces model/moe.py:133-321 (router), :1395-1448 (capacity), :360-498 (NCCL dispatcher: 4
// collectives + 3 host syncs per layer) and :1386-1390,1691-1714 (scatter-back) of the reference.
#include "common.cuh"

namespace {

constexpr int KID_DISPATCH = 10;
constexpr int KID_COMBINE = 11;
constexpr int MAX_E = 64;
constexpr int MAX_K = 8;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]), np::pack_bf16(f[4], f[5]),
                    np::pack_bf16(f[6], f[7]));
}

// ------------------------------------------------------------------ router
// logits[t, e] = <x[t], Wg[e]> + bias[e]  (fp32 accumulate, fp32 gate weights). One warp per token; the register
// cap keeps four CTAs per SM resident so that enough row loads are in flight; the gate weights come from L1.
template <int EB>
__global__ void __launch_bounds__(256, 4) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const float* __restrict__ wg,
                                                               const float* __restrict__ bias,
                                                               float* __restrict__ logits, int T, int D, int E) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nwarps) {
    for (int e0 = 0; e0 < E; e0 += EB) {
      float acc[EB];
#pragma unroll
      for (int e = 0; e < EB; ++e) acc[e] = 0.f;
      for (int d = lane * 8; d < D; d += 512) {
        const bool two = d + 256 < D;
        const uint4 q0 = *reinterpret_cast<const uint4*>(x + (size_t)t * D + d);
        const uint4 q1 = two ? *reinterpret_cast<const uint4*>(x + (size_t)t * D + d + 256) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !two) break;
          float xv[8];
          const uint4 q = h ? q1 : q0;
          float2 a = np::unpack_bf16(q.x), b = np::unpack_bf16(q.y), c = np::unpack_bf16(q.z), dd = np::unpack_bf16(q.w);
          xv[0] = a.x; xv[1] = a.y; xv[2] = b.x; xv[3] = b.y; xv[4] = c.x; xv[5] = c.y; xv[6] = dd.x; xv[7] = dd.y;
#pragma unroll
          for (int e = 0; e < EB; ++e) {
            if (e0 + e < E) {
              const float* wp = wg + (size_t)(e0 + e) * D + d + h * 256;
              const float4 w0 = __ldg(reinterpret_cast<const float4*>(wp));
              const float4 w1 = __ldg(reinterpret_cast<const float4*>(wp + 4));
              acc[e] += xv[0] * w0.x + xv[1] * w0.y + xv[2] * w0.z + xv[3] * w0.w + xv[4] * w1.x + xv[5] * w1.y +
                        xv[6] * w1.z + xv[7] * w1.w;
            }
          }
        }
      }
#pragma unroll
      for (int e = 0; e < EB; ++e) {
        const float sm = np::warp_sum(acc[e]);
        if (lane == 0 && e0 + e < E) logits[(size_t)t * E + e0 + e] = sm + (bias ? bias[e0 + e] : 0.f);
      }
    }
  }
}

// One thread per token. gating: 0 softmax over the selected logits, 1 sigmoid + renormalise.
// stats: counts[E] (int), psum[E] (sum of full-softmax probabilities), zsum[1] (sum of lse^2).
template <int EMAX>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits,
                                                          const float* __restrict__ score_bias,
                                                          float* __restrict__ weights, int* __restrict__ indices,
                                                          int* __restrict__ counts, float* __restrict__ psum,
                                                          float* __restrict__ zsum, int T, int E, int K,
                                                          int gating) {
  __shared__ int s_cnt[MAX_E];
  __shared__ float s_p[MAX_E];
  __shared__ float s_z;
  for (int i = threadIdx.x; i < E; i += blockDim.x) { s_cnt[i] = 0; s_p[i] = 0.f; }
  if (threadIdx.x == 0) s_z = 0.f;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  // per-thread contributions to the statistics; reduced over the warp before they touch shared memory
  float pe[EMAX];
  float pz = 0.f;
  unsigned long long picked = 0ull;
#pragma unroll
  for (int e = 0; e < EMAX; ++e) pe[e] = 0.f;
  if (t < T) {
    float l[EMAX];  // EMAX is a compile-time bound so the logits stay in registers
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      if (e >= E) { l[e] = -INFINITY; continue; }
      l[e] = logits[(size_t)t * E + e] + (score_bias ? score_bias[e] : 0.f);
      mx = fmaxf(mx, l[e]);
    }
    float se = 0.f;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) se += (e < E) ? __expf(l[e] - mx) : 0.f;
    const float lse = mx + logf(se);
    pz = lse * lse;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) pe[e] = (e < E) ? __expf(l[e] - lse) : 0.f;
    // top-k by repeated argmax (ties -> lowest index, as torch.topk on distinct values)
    int sel[MAX_K];
    float sv[MAX_K];
    unsigned long long used = 0ull;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      float bv = -INFINITY;
#pragma unroll
      for (int e = 0; e < EMAX; ++e) {
        if (e >= E) continue;
        const float v = gating == 1 ? 1.f / (1.f + __expf(-l[e])) : l[e];
        if (!((used >> e) & 1ull) && (best < 0 || v > bv)) { best = e; bv = v; }
      }
      used |= 1ull << best;
      sel[k] = best;
      sv[k] = bv;
    }
    picked = used;
    float den = 0.f;
    if (gating == 1) {
      for (int k = 0; k < K; ++k) den += sv[k];
      den += 1e-8f;
      for (int k = 0; k < K; ++k) sv[k] /= den;
    } else {
      const float m0 = sv[0];  // the first pick is the largest selected logit
      for (int k = 0; k < K; ++k) { sv[k] = __expf(sv[k] - m0); den += sv[k]; }
      for (int k = 0; k < K; ++k) sv[k] /= den;
    }
    for (int k = 0; k < K; ++k) {
      weights[(size_t)t * K + k] = sv[k];
      indices[(size_t)t * K + k] = sel[k];
    }
  }
  {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      if (e >= E) break;
      const float ps = np::warp_sum(pe[e]);
      const int c = __popc(__ballot_sync(0xffffffffu, (picked >> e) & 1ull));
      if (lane == 0) {
        atomicAdd(&s_p[e], ps);
        if (c) atomicAdd(&s_cnt[e], c);
      }
    }
    pz = np::warp_sum(pz);
    if (lane == 0) atomicAdd(&s_z, pz);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    if (s_cnt[i]) atomicAdd(&counts[i], s_cnt[i]);
    atomicAdd(&psum[i], s_p[i]);
  }
  if (threadIdx.x == 0) atomicAdd(zsum, s_z);
}

// dlogits[t, :] from d(weights) and d(aux): aux = coef_lb * E * sum_i f_i * mean_t p[t,i]
//                                                + coef_z * mean_t lse_t^2
// f (fractions, [E]) is treated as a constant, as autograd does for the reference's one_hot count.
__global__ void __launch_bounds__(256) router_bwd_kernel(const float* __restrict__ logits,
                                                         const float* __restrict__ score_bias,
                                                         const float* __restrict__ weights,
                                                         const int* __restrict__ indices,
                                                         const float* __restrict__ dweights,
                                                         const float* __restrict__ f,
                                                         const float* __restrict__ daux, float coef_lb,
                                                         float coef_z, float* __restrict__ dlogits, int T, int E,
                                                         int K, int gating) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float l[MAX_E], dl[MAX_E];
  float mx = -INFINITY;
#pragma unroll 1
  for (int e = 0; e < E; ++e) {
    l[e] = logits[(size_t)t * E + e] + (score_bias ? score_bias[e] : 0.f);
    mx = fmaxf(mx, l[e]);
    dl[e] = 0.f;
  }
  float se = 0.f;
#pragma unroll 1
  for (int e = 0; e < E; ++e) se += __expf(l[e] - mx);
  const float lse = mx + logf(se);
  const float da = daux ? daux[0] : 0.f;
  if (da != 0.f) {
    float fp = 0.f;
#pragma unroll 1
    for (int e = 0; e < E; ++e) fp += f[e] * __expf(l[e] - lse);
#pragma unroll 1
    for (int e = 0; e < E; ++e) {
      const float p = __expf(l[e] - lse);
      dl[e] += da * (coef_lb * (float)E / (float)T * p * (f[e] - fp) + coef_z * 2.f * lse / (float)T * p);
    }
  }
  if (dweights) {
    float wsum = 0.f;
    for (int k = 0; k < K; ++k) wsum += weights[(size_t)t * K + k] * dweights[(size_t)t * K + k];
    for (int k = 0; k < K; ++k) {
      const int e = indices[(size_t)t * K + k];
      const float w = weights[(size_t)t * K + k], dw = dweights[(size_t)t * K + k];
      if (gating == 0) {
        dl[e] += w * (dw - wsum);
      } else {
        // w_k = s_k / (sum s + eps); ds_k = (dw_k - sum_j w_j dw_j) / (sum s + eps); dl = ds * s(1-s)
        const float s = 1.f / (1.f + __expf(-l[e]));
        float ssum = 1e-8f;
        for (int j = 0; j < K; ++j) ssum += 1.f / (1.f + __expf(-l[indices[(size_t)t * K + j]]));
        dl[e] += (dw - wsum) / ssum * s * (1.f - s);
      }
    }
  }
#pragma unroll 1
  for (int e = 0; e < E; ++e) dlogits[(size_t)t * E + e] = dl[e];
}

// partial[c, e, d] = sum over the chunk's tokens of dl[t, e] * x[t, d]. CTA = 64 column threads (8 columns each) x 4
// token lanes; a lane walks every fourth token of the chunk with four row loads in flight, the lanes are summed
// through shared memory.
template <int EB>
__global__ void __launch_bounds__(256) router_dgate_kernel(const float* __restrict__ dl,
                                                           const __nv_bfloat16* __restrict__ x,
                                                           float* __restrict__ partial, int T, int D, int E,
                                                           int chunk) {
  __shared__ float red[2][64][EB * 8 + 1];
  const int c = blockIdx.y;
  const int t0 = c * chunk, t1 = min(T, t0 + chunk);
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int d = (blockIdx.x * 64 + tx) * 8;
  const bool col_ok = d < D;
  for (int e0 = 0; e0 < E; e0 += EB) {
    float acc[EB][8];
#pragma unroll
    for (int e = 0; e < EB; ++e)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[e][j] = 0.f;
    if (col_ok) {
      for (int tb = t0 + ty; tb < t1; tb += 16) {   // tokens tb, tb+4, tb+8, tb+12
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          q[u] = (tb + 4 * u < t1) ? *reinterpret_cast<const uint4*>(x + (size_t)(tb + 4 * u) * D + d)
                                   : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (tb + 4 * u >= t1) break;
          float2 a = np::unpack_bf16(q[u].x), b = np::unpack_bf16(q[u].y), cc = np::unpack_bf16(q[u].z),
                 dd = np::unpack_bf16(q[u].w);
          const float xv[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, dd.x, dd.y};
#pragma unroll
          for (int e = 0; e < EB; ++e) {
            if (e0 + e < E) {
              const float g = __ldg(dl + (size_t)(tb + 4 * u) * E + e0 + e);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[e][j] += g * xv[j];
            }
          }
        }
      }
    }
    if (ty >= 2) {   // lanes 2, 3 -> lanes 0, 1
#pragma unroll
      for (int e = 0; e < EB; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j) red[ty - 2][tx][e * 8 + j] = acc[e][j];
    }
    __syncthreads();
    if (ty < 2) {
#pragma unroll
      for (int e = 0; e < EB; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[e][j] += red[ty][tx][e * 8 + j];
    }
    __syncthreads();
    if (ty == 1) {   // lane 1 -> lane 0
#pragma unroll
      for (int e = 0; e < EB; ++e)
#pragma unroll
        for (int j = 0; j < 8; ++j) red[0][tx][e * 8 + j] = acc[e][j];
    }
    __syncthreads();
    if (ty == 0 && col_ok) {
#pragma unroll
      for (int e = 0; e < EB; ++e) {
        if (e0 + e < E) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[e][j] += red[0][tx][e * 8 + j];
          float* dst = partial + ((size_t)c * E + e0 + e) * D + d;
          *reinterpret_cast<float4*>(dst) = make_float4(acc[e][0], acc[e][1], acc[e][2], acc[e][3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[e][4], acc[e][5], acc[e][6], acc[e][7]);
        }
      }
    }
    __syncthreads();
  }
}

// dx[t, :] = sum_e dl[t, e] * Wg[e, :] in bf16: the router's contribution to the gradient of its input (a
// [T, E] x [E, D] product with E of 8 to 64: one thread per 8 output columns, the gate rows come from L1).
__global__ void __launch_bounds__(256) router_dx_kernel(const float* __restrict__ dl, const float* __restrict__ wg,
                                                        __nv_bfloat16* __restrict__ dx, int T, int D, int E) {
  const int vec_per_row = D >> 3;
  const long long total = (long long)T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row), d = (int)(i % vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < E; ++e) {
      const float g = __ldg(dl + (size_t)t * E + e);
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(wg + (size_t)e * D + d));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(wg + (size_t)e * D + d + 4));
      acc[0] += g * w0.x; acc[1] += g * w0.y; acc[2] += g * w0.z; acc[3] += g * w0.w;
      acc[4] += g * w1.x; acc[5] += g * w1.y; acc[6] += g * w1.z; acc[7] += g * w1.w;
    }
    *reinterpret_cast<uint4*>(dx + (size_t)t * D + d) = pack8(acc);
  }
}

// Same product for E <= 8 with D = 8 * blockDim.x: a thread keeps its 8 columns of all gate rows in registers and
// walks TOK tokens, so the only memory traffic per token is the [E] gradient row (broadcast) and one 16-byte store.
template <int TOK>
__global__ void __launch_bounds__(256) router_dx_reg_kernel(const float* __restrict__ dl, const float* __restrict__ wg,
                                                            __nv_bfloat16* __restrict__ dx, int T, int D, int E) {
  const int d = threadIdx.x * 8;
  float w[8][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
    if (e < E) {
      w0 = __ldg(reinterpret_cast<const float4*>(wg + (size_t)e * D + d));
      w1 = __ldg(reinterpret_cast<const float4*>(wg + (size_t)e * D + d + 4));
    }
    w[e][0] = w0.x; w[e][1] = w0.y; w[e][2] = w0.z; w[e][3] = w0.w;
    w[e][4] = w1.x; w[e][5] = w1.y; w[e][6] = w1.z; w[e][7] = w1.w;
  }
  const int t0 = blockIdx.x * TOK;
#pragma unroll 4
  for (int i = 0; i < TOK; ++i) {
    const int t = t0 + i;
    if (t >= T) break;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = e < E ? __ldg(dl + (size_t)t * E + e) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += g * w[e][j];
    }
    *reinterpret_cast<uint4*>(dx + (size_t)t * D + d) = pack8(acc);
  }
}

__global__ void colsum2_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts,
                               long long cols, int accumulate) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int p = 0;
  for (; p + 7 < parts; p += 8) {   // eight independent loads in flight
#pragma unroll
    for (int u = 0; u < 8; ++u) a8[u] += partial[(size_t)(p + u) * cols + c];
  }
  for (; p < parts; ++p) a8[0] += partial[(size_t)p * cols + c];
  const float s = ((a8[0] + a8[1]) + (a8[2] + a8[3])) + ((a8[4] + a8[5]) + (a8[6] + a8[7]));
  out[c] = accumulate ? out[c] + s : s;
}

// out[c] (+)= sum over rows of a[r, c] for a narrow matrix (cols <= 64): 1024 threads, thread -> (row group, col)
__global__ void __launch_bounds__(1024) colsum_narrow_kernel(const float* __restrict__ a, float* __restrict__ out,
                                                             int rows, int cols, int accumulate) {
  __shared__ float red[1024];
  const int c = threadIdx.x % cols, g = threadIdx.x / cols, ng = 1024 / cols;
  float s = 0.f;
  if (g < ng) {
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
    int r = g;
    for (; r + 3 * ng < rows; r += 4 * ng) {
#pragma unroll
      for (int u = 0; u < 4; ++u) a4[u] += a[(size_t)(r + u * ng) * cols + c];
    }
    for (; r < rows; r += ng) a4[0] += a[(size_t)r * cols + c];
    s = (a4[0] + a4[1]) + (a4[2] + a4[3]);
  }
  red[threadIdx.x] = (g < ng) ? s : 0.f;
  __syncthreads();
  if (threadIdx.x < cols) {
    float t = 0.f;
    for (int i = 0; i < ng; ++i) t += red[i * cols + threadIdx.x];
    out[threadIdx.x] = accumulate ? out[threadIdx.x] + t : t;
  }
}

// ------------------------------------------------------------------ capacity / positions
// One CTA of 1024 threads; thread i owns a contiguous run of tokens, so a block-wide exclusive scan of
// per-thread pick counts gives positions in token order. The counters of a group of experts are packed into up to
// four 64-bit words (16-bit fields while T < 65536, else 32-bit) and scanned together. Phase 0 ranks every pick
// among all tokens that picked the expert and clears keep[t] when any pick of t lies at or beyond `capacity`
// (capacity < 0: keep all); phase 1 ranks among the kept tokens.
// Outputs: slot_pos[t,k] (position among kept for expert idx[t,k], -1 if dropped), keep[T],
// counts_kept[E], drops[E] (tokens beyond capacity per expert), n_dropped[1].
struct U64x4 {
  unsigned long long w[4];
};
__device__ __forceinline__ U64x4 block_excl_scan4(const U64x4& v, int nw_used, U64x4* s_warp, U64x4* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  U64x4 inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q < nw_used) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, inc.w[q], o);
        if (lane >= o) inc.w[q] += n;
      }
    }
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    U64x4 wv = lane < nwarps ? s_warp[lane] : U64x4{{0ull, 0ull, 0ull, 0ull}};
    U64x4 winc = wv;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (q < nw_used) {
          const unsigned long long n = __shfl_up_sync(0xffffffffu, winc.w[q], o);
          if (lane >= o) winc.w[q] += n;
        }
      }
    }
    U64x4 ex;
#pragma unroll
    for (int q = 0; q < 4; ++q) ex.w[q] = winc.w[q] - wv.w[q];
    s_warp[lane] = ex;                 // exclusive offset of each warp
    if (lane == 31) s_warp[32] = winc;  // grand total
  }
  __syncthreads();
  U64x4 res;
#pragma unroll
  for (int q = 0; q < 4; ++q) res.w[q] = s_warp[warp].w[q] + inc.w[q] - v.w[q];
  *total = s_warp[32];
  __syncthreads();                     // s_warp is reused by the next scan
  return res;
}

template <int FB>   // bits per counter: 16 or 32
__global__ void __launch_bounds__(1024) capacity_scan_kernel(const int* __restrict__ indices, int T, int E, int K,
                                                             int capacity, int* __restrict__ slot_pos,
                                                             int* __restrict__ keep, int* __restrict__ counts_kept,
                                                             int* __restrict__ drops, int* __restrict__ n_dropped,
                                                             int use_smem) {
  constexpr int EPW = 64 / FB;          // experts per 64-bit word
  constexpr int GROUP = 4 * EPW;        // experts per pass
  constexpr unsigned long long FMASK = (FB == 16) ? 0xffffull : 0xffffffffull;
  extern __shared__ int s_dyn[];        // routing table staged once, then one keep byte per token
  __shared__ U64x4 s_warp[33];
  int* s_idx = s_dyn;
  unsigned char* s_keep = reinterpret_cast<unsigned char*>(s_dyn + (use_smem ? T * K : 0));
  const int* idx = indices;
  if (use_smem) {
    for (int i = threadIdx.x; i < T * K; i += blockDim.x) s_idx[i] = indices[i];
    for (int t = threadIdx.x; t < T; t += blockDim.x) s_keep[t] = 1;
    idx = s_idx;
  } else {
    for (int t = threadIdx.x; t < T; t += blockDim.x) keep[t] = 1;
  }
  __syncthreads();
  const int per = (T + blockDim.x - 1) / blockDim.x;
  const int t_lo = min(T, (int)threadIdx.x * per), t_hi = min(T, t_lo + per);
  for (int phase = (capacity < 0 ? 1 : 0); phase < 2; ++phase) {
    for (int e0 = 0; e0 < E; e0 += GROUP) {
      const int n_e = min(GROUP, E - e0);
      const int nw_used = (n_e + EPW - 1) / EPW;
      U64x4 loc{{0ull, 0ull, 0ull, 0ull}};
      for (int t = t_lo; t < t_hi; ++t) {
        if (phase == 1 && !(use_smem ? s_keep[t] : keep[t])) continue;
        for (int k = 0; k < K; ++k) {
          const int e = idx[(size_t)t * K + k] - e0;
          if (e >= 0 && e < n_e) loc.w[e / EPW] += 1ull << (FB * (e % EPW));
        }
      }
      U64x4 total;
      U64x4 run = block_excl_scan4(loc, nw_used, s_warp, &total);
      for (int t = t_lo; t < t_hi; ++t) {
        const bool kept = phase == 0 || (use_smem ? s_keep[t] : keep[t]);
        for (int k = 0; k < K; ++k) {
          const int e = idx[(size_t)t * K + k] - e0;
          if (e < 0 || e >= n_e) continue;
          if (!kept) {
            slot_pos[(size_t)t * K + k] = -1;
            continue;
          }
          const int q = e / EPW, sh = FB * (e % EPW);
          const int pos = (int)((run.w[q] >> sh) & FMASK);
          run.w[q] += 1ull << sh;
          if (phase == 0) {
            if (pos >= capacity) {   // only ever written to 0, by the thread that owns the token
              if (use_smem) s_keep[t] = 0; else keep[t] = 0;
            }
          } else {
            slot_pos[(size_t)t * K + k] = pos;
          }
        }
      }
      if ((int)threadIdx.x < n_e) {
        const int e = threadIdx.x;
        const int c = (int)((total.w[e / EPW] >> (FB * (e % EPW))) & FMASK);
        if (phase == 0) {
          drops[e0 + e] = c > capacity ? c - capacity : 0;
        } else {
          counts_kept[e0 + e] = c;
          if (capacity < 0) drops[e0 + e] = 0;
        }
      }
    }
    __syncthreads();   // keep flags of phase 0 are complete before phase 1 reads them
  }
  int nd = 0;
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const int kp = use_smem ? (int)s_keep[t] : keep[t];
    if (use_smem) keep[t] = kp;
    nd += kp ? 0 : 1;
  }
  U64x4 ndv{{(unsigned long long)nd, 0ull, 0ull, 0ull}}, total;
  block_excl_scan4(ndv, 1, s_warp, &total);
  if (threadIdx.x == 0) n_dropped[0] = (int)total.w[0];
}

// ------------------------------------------------------------------ EP dispatch (peer stores)
struct DispatchParams {
  const __nv_bfloat16* x;      // [T, D] source rows
  const int* indices;          // [T, K] expert of each slot
  const int* slot_pos;         // [T, K] position inside (expert, this source) region, -1 = dropped
  const int* counts_kept;      // [E]
  const float* slot_scale;     // [T, K] optional multiplier (backward: router weight), nullptr = 1
  int T, K, D, E, E_local, n_ranks, my_rank;
  int region_rows;             // rows reserved per (local expert, source) region, multiple of 128
  int quant;                   // 0: bf16 rows, 1: e4m3 rows + fp32 1x128 scales
  void* const* peer_rows;      // [n_ranks] receive buffer (bf16 [rows, D] or uint8 [rows, D])
  float* const* peer_scales;   // [n_ranks] fp32 [rows, D/128] (quant only)
  long long* const* peer_row_dst;   // [n_ranks] per-row return address (source << 40 | slot), -1 = padding
  int* const* peer_mblk_rows;  // [n_ranks] valid rows of every 128-row block of the receive buffer
  int* const* peer_src_blocks; // [n_ranks] [n_ranks] number of non-empty blocks sent by each source
  int* const* peer_flags;      // [n_ranks] [n_ranks] arrival epoch per source
  int* done_ctr;               // local CTA counter (zero between launches)
  int epoch;
  int write_meta;              // 1: also write row_dst / mblk_rows / src_blocks (forward); 0: rows only
  const int* epoch_base;       // optional device counter added to `epoch`
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const DispatchParams p) {
  np::CommSpan span(p.n_ranks > 1);
  const int lane = threadIdx.x & 31;
  const int warp_g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int slots = p.T * p.K;
  const int pad_items = p.E * 128;
  for (int it = warp_g; it < slots + pad_items; it += nwarps) {
    int e, pos;
    bool is_pad = it >= slots;
    float sc = 1.f;
    const __nv_bfloat16* src = nullptr;
    long long ret = -1;
    if (!is_pad) {
      pos = p.slot_pos[it];
      if (pos < 0) continue;
      e = p.indices[it];
      NP_DBG_SKIP_UNLESS(e >= 0 && e < p.E, KID_DISPATCH, e)
      src = p.x + (size_t)(it / p.K) * p.D;
      if (p.slot_scale) sc = p.slot_scale[it];
      ret = ((long long)p.my_rank << 40) | (long long)it;
    } else {
      e = (it - slots) >> 7;
      const int cnt = p.counts_kept[e];
      pos = cnt + ((it - slots) & 127);
      if (pos >= ((cnt + 127) & ~127)) continue;
    }
    if (pos >= p.region_rows) {  // cannot happen when region_rows >= capacity; recorded, not stored
      if (lane == 0) np::report(NP_ERR_BOUNDS, KID_DISPATCH, pos);
      continue;
    }
    const int peer = e / p.E_local, le = e - peer * p.E_local;
    const size_t row = ((size_t)le * p.n_ranks + p.my_rank) * p.region_rows + pos;
    if (!p.quant) {
      uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)p.peer_rows[peer] + row * p.D);
      for (int v = lane; v < (p.D >> 3); v += 32) {
        uint4 u = make_uint4(0, 0, 0, 0);
        if (!is_pad) {
          u = *reinterpret_cast<const uint4*>(src + v * 8);
          if (p.slot_scale) {
            float f[8];
            float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
            f[0] = a.x * sc; f[1] = a.y * sc; f[2] = b.x * sc; f[3] = b.y * sc;
            f[4] = c.x * sc; f[5] = c.y * sc; f[6] = d.x * sc; f[7] = d.y * sc;
            u = pack8(f);
          }
        }
        dst[v] = u;
      }
    } else {
      // 16 lanes x 8 elements = one 128-element scale block; two blocks per warp iteration
      uint2* dst = reinterpret_cast<uint2*>((uint8_t*)p.peer_rows[peer] + row * p.D);
      float* sdst = p.peer_scales[peer] + row * (p.D >> 7);
      for (int v = lane; v < (p.D >> 3); v += 32) {
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (!is_pad) {
          load8(src + v * 8, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] *= sc;
        }
        float am = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[j]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        float scale, inv;
        int e2 = -127;
        if (p.quant == 2) {   // power-of-two scale (UE8M0): ceil(log2(am / 448))
          if (am > 0.f) {
            int ex;
            const float mant = frexpf(__fdiv_rn(am, 448.f), &ex);
            e2 = (mant == 0.5f) ? ex - 1 : ex;
            e2 = max(-127, min(127, e2));
          }
          inv = exp2f((float)-e2);
          scale = 0.f;
        } else {
          scale = fmaxf(am, 1e-12f) / 448.f;
          inv = 1.f / scale;
        }
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo |= (uint32_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
          hi |= (uint32_t)__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        }
        dst[v] = make_uint2(lo, hi);
        if ((lane & 15) == 0) {
          if (p.quant == 2) {
            // exponent byte, four times, in the 512-byte chunk layout the block-scaled MMA reads (gemm_mxfp8_sm100.cu)
            const int r = (int)(row & 127), kb = v >> 4, nkb = p.D >> 7;
            uint8_t* sfb = reinterpret_cast<uint8_t*>(p.peer_scales[peer]);
            *reinterpret_cast<uint32_t*>(sfb + ((row >> 7) * nkb + kb) * 512 + (r & 31) * 16 + (r >> 5) * 4) =
                (uint32_t)(e2 + 127) * 0x01010101u;
          } else {
            sdst[v >> 4] = scale;
          }
        }
      }
    }
    if (p.write_meta && lane == 0) p.peer_row_dst[peer][row] = ret;
  }
  // ---- completion: last CTA publishes the block table and releases the epoch flags
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.done_ctr, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  const int bpr = p.region_rows >> 7;  // blocks per region
  if (p.write_meta) {
    for (int i = threadIdx.x; i < p.E * bpr; i += blockDim.x) {
      const int e = i / bpr, b = i - e * bpr;
      const int peer = e / p.E_local, le = e - peer * p.E_local;
      int r = p.counts_kept[e] - b * 128;
      r = r < 0 ? 0 : (r > 128 ? 128 : r);
      // a block with any row is processed whole (its padding rows are zero)
      p.peer_mblk_rows[peer][((size_t)le * p.n_ranks + p.my_rank) * bpr + b] = r > 0 ? 128 : 0;
    }
    for (int peer = threadIdx.x; peer < p.n_ranks; peer += blockDim.x) {
      int nb = 0;
      for (int le = 0; le < p.E_local; ++le) nb += (p.counts_kept[peer * p.E_local + le] + 127) >> 7;
      p.peer_src_blocks[peer][p.my_rank] = nb;
    }
  }
  __threadfence_system();
  __syncthreads();
  for (int peer = threadIdx.x; peer < p.n_ranks; peer += blockDim.x)
    np::st_release_sys(p.peer_flags[peer] + p.my_rank, p.epoch + (p.epoch_base ? *p.epoch_base : 0));
  if (threadIdx.x == 0) *p.done_ctr = 0;
}

// ------------------------------------------------------------------ EP combine (reduce at the source)
struct CombineParams {
  const __nv_bfloat16* rows;   // [T*K, D] rows returned by the experts (slot-major)
  const int* slot_pos;         // [T, K], -1 = dropped slot (contributes zero)
  const float* weights;        // [T, K] router weights, nullptr = 1 (backward)
  const __nv_bfloat16* add1;   // optional [T, D] term added to every token
  const __nv_bfloat16* add2;   // optional second [T, D] term
  const float* dl;             // optional router term: out += dl[t, :] @ wg   (dl [T, E], wg [E, D])
  const float* wg;
  __nv_bfloat16* out;          // [T, D]
  int T, K, D, E;
  const int* flags;            // [n_ranks] completion epoch written by each peer, nullptr = no wait
  const int* sent_to_peer;     // [n_ranks] rows this rank sent to each peer (0 = nothing to wait for)
  int n_ranks, epoch;
  unsigned long long limit_ns;
  const int* epoch_base;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const CombineParams p) {
  __shared__ int s_ok;
  if (p.flags) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < p.n_ranks && p.sent_to_peer[threadIdx.x] > 0) {
      if (!np::wait_flag_ge(p.flags + threadIdx.x, p.epoch + (p.epoch_base ? *p.epoch_base : 0), p.limit_ns, KID_COMBINE,
                            threadIdx.x)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;
  }
  const int vec_per_row = p.D >> 3;
  const long long total = (long long)p.T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row);
    const int d = (int)(i - (long long)t * vec_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < p.K; ++k) {
      if (p.slot_pos[(size_t)t * p.K + k] < 0) continue;
      NP_DBG_SKIP_UNLESS(p.slot_pos[(size_t)t * p.K + k] < (1 << 24), KID_COMBINE, p.slot_pos[(size_t)t * p.K + k])
      float f[8];
      load8(p.rows + ((size_t)t * p.K + k) * p.D + d, f);
      const float w = p.weights ? p.weights[(size_t)t * p.K + k] : 1.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
    }
    if (p.add1) {
      float f[8];
      load8(p.add1 + (size_t)t * p.D + d, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (p.add2) {
      float f[8];
      load8(p.add2 + (size_t)t * p.D + d, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (p.dl) {
      for (int e = 0; e < p.E; ++e) {
        const float g = p.dl[(size_t)t * p.E + e];
        const float4 w0 = *reinterpret_cast<const float4*>(p.wg + (size_t)e * p.D + d);
        const float4 w1 = *reinterpret_cast<const float4*>(p.wg + (size_t)e * p.D + d + 4);
        acc[0] += g * w0.x; acc[1] += g * w0.y; acc[2] += g * w0.z; acc[3] += g * w0.w;
        acc[4] += g * w1.x; acc[5] += g * w1.y; acc[6] += g * w1.z; acc[7] += g * w1.w;
      }
    }
    *reinterpret_cast<uint4*>(p.out + (size_t)t * p.D + d) = pack8(acc);
  }
}

// dots[t, k] = <a[t, :], rows[t*K + k, :]>  (0 for dropped slots); one warp per slot.
__global__ void __launch_bounds__(256) slot_dot_kernel(const __nv_bfloat16* __restrict__ a,
                                                       const __nv_bfloat16* __restrict__ rows,
                                                       const int* __restrict__ slot_pos, float* __restrict__ dots,
                                                       int T, int K, int D) {
  const int lane = threadIdx.x & 31;
  const int warp_g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int s = warp_g; s < T * K; s += nwarps) {
    float acc = 0.f;
    if (slot_pos[s] >= 0) {
      const int t = s / K;
      for (int d = lane * 8; d < D; d += 256) {
        float f[8], g[8];
        load8(a + (size_t)t * D + d, f);
        load8(rows + (size_t)s * D + d, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += f[j] * g[j];
      }
    }
    acc = np::warp_sum(acc);
    if (lane == 0) dots[s] = acc;
  }
}

}  // namespace

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 500 + (int)e_; } while (0)

NP_API int np_router_logits(const void* x, const float* wg, const float* bias, float* logits, int T, int D, int E,
                            void* stream) {
  if (D % 8 || T <= 0) return T <= 0 ? 0 : 1;
  const int grid = (T * 32 + 255) / 256 < 148 * 8 ? (T * 32 + 255) / 256 : 148 * 8;
  router_logits_kernel<8><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, wg, bias, logits, T, D, E);
  CHECK_LAUNCH();
}

// counts/psum/zsum must be zeroed by the caller before the launch.
NP_API int np_router_topk(const float* logits, const float* score_bias, float* weights, int* indices, int* counts,
                          float* psum, float* zsum, int T, int E, int K, int gating, void* stream) {
  if (E > MAX_E || K > MAX_K || K > E) return 1;
  if (T <= 0) return 0;
#define TOPK(EM) router_topk_kernel<EM><<<(T + 127) / 128, 128, 0, (cudaStream_t)stream>>>( \
      logits, score_bias, weights, indices, counts, psum, zsum, T, E, K, gating)
  if (E <= 8) TOPK(8);
  else if (E <= 16) TOPK(16);
  else if (E <= 32) TOPK(32);
  else TOPK(64);
#undef TOPK
  CHECK_LAUNCH();
}

NP_API int np_router_bwd(const float* logits, const float* score_bias, const float* weights, const int* indices,
                         const float* dweights, const float* f, const float* daux, float coef_lb, float coef_z,
                         float* dlogits, int T, int E, int K, int gating, void* stream) {
  if (E > MAX_E || K > MAX_K) return 1;
  if (T <= 0) return 0;
  router_bwd_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)stream>>>(logits, score_bias, weights, indices, dweights,
                                                                       f, daux, coef_lb, coef_z, dlogits, T, E, K,
                                                                       gating);
  CHECK_LAUNCH();
}

NP_API int np_router_dgate_parts(int T) { return (T + 63) / 64; }
// scratch: fp32 [np_router_dgate_parts(T), E, D]; dwg[E, D] (+)= dl^T x ; dbias[E] (+)= column sums of dl.
NP_API int np_router_dgate(const float* dl, const void* x, float* dwg, float* dbias, float* scratch, int T, int D,
                           int E, int accumulate, void* stream) {
  if (D % 8) return 1;
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int parts = np_router_dgate_parts(T);
  dim3 grid((D / 8 + 63) / 64, parts);
  router_dgate_kernel<8><<<grid, 256, 0, s>>>(dl, (const __nv_bfloat16*)x, scratch, T, D, E, 64);
  const long long cols = (long long)E * D;
  colsum2_kernel<<<(int)((cols + 63) / 64), 64, 0, s>>>(scratch, dwg, parts, cols, accumulate);
  if (dbias) colsum_narrow_kernel<<<1, 1024, 0, s>>>(dl, dbias, T, E, accumulate);
  CHECK_LAUNCH();
}

NP_API int np_router_dx(const float* dl, const float* wg, void* dx, int T, int D, int E, void* stream) {
  if (D % 8) return 1;
  if (T <= 0) return 0;
  if (E <= 8 && D % 8 == 0 && D / 8 <= 256 && D / 8 >= 32) {
    constexpr int TOK = 8;
    router_dx_reg_kernel<TOK><<<(unsigned)((T + TOK - 1) / TOK), D / 8, 0, (cudaStream_t)stream>>>(
        dl, wg, (__nv_bfloat16*)dx, T, D, E);
    CHECK_LAUNCH();
  }
  const long long blocks = ((long long)T * (D / 8) + 255) / 256;
  router_dx_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dl, wg, (__nv_bfloat16*)dx, T, D, E);
  CHECK_LAUNCH();
}

NP_API int np_capacity_scan(const int* indices, int T, int E, int K, int capacity, int* slot_pos, int* keep,
                            int* counts_kept, int* drops, int* n_dropped, void* stream) {
  if (K > MAX_K) return 1;
  if (T <= 0) return 0;
  const size_t smem = (size_t)T * K * 4 + (size_t)((T + 3) / 4) * 4;
  const int use_smem = smem <= 200 * 1024;
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (use_smem && !attr_set) {
    cudaError_t e = cudaFuncSetAttribute(capacity_scan_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(capacity_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  if (T < 65536)   // a 16-bit counter holds any per-expert count
    capacity_scan_kernel<16><<<1, 1024, use_smem ? smem : 0, (cudaStream_t)stream>>>(
        indices, T, E, K, capacity, slot_pos, keep, counts_kept, drops, n_dropped, use_smem);
  else
    capacity_scan_kernel<32><<<1, 1024, use_smem ? smem : 0, (cudaStream_t)stream>>>(
        indices, T, E, K, capacity, slot_pos, keep, counts_kept, drops, n_dropped, use_smem);
  CHECK_LAUNCH();
}

struct NpDispatchArgs {
  const void* x; const int* indices; const int* slot_pos; const int* counts_kept; const float* slot_scale;
  int T, K, D, E, E_local, n_ranks, my_rank, region_rows, quant;
  void* const* peer_rows; float* const* peer_scales; long long* const* peer_row_dst;
  int* const* peer_mblk_rows; int* const* peer_src_blocks; int* const* peer_flags;
  int* done_ctr; int epoch; int write_meta; int max_ctas; const int* epoch_base;
};
NP_API int np_ep_dispatch(const NpDispatchArgs* a, void* stream) {
  if (a->D % 128 || a->region_rows % 128 || a->E % a->E_local || (a->quant && a->D % 256)) return 1;
  DispatchParams p;
  p.x = (const __nv_bfloat16*)a->x; p.indices = a->indices; p.slot_pos = a->slot_pos; p.counts_kept = a->counts_kept;
  p.slot_scale = a->slot_scale; p.T = a->T; p.K = a->K; p.D = a->D; p.E = a->E; p.E_local = a->E_local;
  p.n_ranks = a->n_ranks; p.my_rank = a->my_rank; p.region_rows = a->region_rows; p.quant = a->quant;
  p.peer_rows = a->peer_rows; p.peer_scales = a->peer_scales; p.peer_row_dst = a->peer_row_dst;
  p.peer_mblk_rows = a->peer_mblk_rows; p.peer_src_blocks = a->peer_src_blocks; p.peer_flags = a->peer_flags;
  p.done_ctr = a->done_ctr; p.epoch = a->epoch; p.write_meta = a->write_meta;
  p.epoch_base = a->epoch_base;
  const int items = a->T * a->K + a->E * 128;
  int grid = (items + 7) / 8;
  const int cap = a->max_ctas > 0 ? a->max_ctas : 148 * 4;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  ep_dispatch_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  CHECK_LAUNCH();
}

struct NpCombineArgs {
  const void* rows; const int* slot_pos; const float* weights; const void* add1; const void* add2;
  const float* dl; const float* wg; void* out; int T, K, D, E;
  const int* flags; const int* sent_to_peer; int n_ranks, epoch; unsigned long long limit_ns;
  const int* epoch_base;
};
NP_API int np_ep_combine(const NpCombineArgs* a, void* stream) {
  if (a->D % 8 || a->n_ranks > 256) return 1;
  if (a->T <= 0) return 0;
  CombineParams p;
  p.rows = (const __nv_bfloat16*)a->rows; p.slot_pos = a->slot_pos; p.weights = a->weights;
  p.add1 = (const __nv_bfloat16*)a->add1; p.add2 = (const __nv_bfloat16*)a->add2; p.dl = a->dl; p.wg = a->wg;
  p.out = (__nv_bfloat16*)a->out; p.T = a->T; p.K = a->K; p.D = a->D; p.E = a->E; p.flags = a->flags;
  p.sent_to_peer = a->sent_to_peer; p.n_ranks = a->n_ranks; p.epoch = a->epoch;
  p.limit_ns = a->limit_ns ? a->limit_ns : NP_WAIT_LIMIT_NS;
  p.epoch_base = a->epoch_base;
  long long work = (long long)a->T * (a->D / 8);
  int grid = (int)((work + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  ep_combine_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  CHECK_LAUNCH();
}

NP_API int np_slot_dot(const void* a, const void* rows, const int* slot_pos, float* dots, int T, int K, int D,
                       void* stream) {
  if (D % 8) return 1;
  if (T <= 0) return 0;
  int grid = (T * K + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  slot_dot_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)rows, slot_pos,
                                                          dots, T, K, D);
  CHECK_LAUNCH();
}
