// Symmetric-memory runtime and the fused data-parallel optimizer step for sm_100a.
//
//  np_symm_*        : one cudaMalloc'd arena per rank, shared with the other ranks of the node through
//                     CUDA IPC handles; every kernel then gets a table of peer base pointers.
//  symm_barrier     : device-side barrier over epoch flags in peer memory (bounded wait).
//  zero_reduce      : gradient reduce-scatter as peer loads: each rank sums its shard of the flat fp32
//                     gradient over all ranks' buffers, scales it, and produces sum-of-squares partials.
//  zero_adamw_bcast : AdamW on the shard (fp32 master, m, v) and all-gather as peer stores: the bf16
//                     compute weights are written straight into every rank's parameter arena.
//
// Together the last two replace FSDP2's reduce_scatter_tensor + per-parameter AdamW + all_gather
// (reference: model/transformer.py:570-627, optim/adamw.py:74-121) with two launches per step.
// All peer access is plain ld/st.global on IPC-mapped pointers; waits are bounded.
#include "common.cuh"

namespace {

constexpr int KID_BARRIER = 20;
constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__global__ void symm_barrier_kernel(PeerPtrs flags, int my_rank, int n, int epoch, unsigned long long limit_ns) {
  const int t = threadIdx.x;
  if (t < n) {
    __threadfence_system();
    np::st_release_sys(reinterpret_cast<int*>(flags.p[t]) + my_rank, epoch);
    np::wait_flag_ge(reinterpret_cast<int*>(flags.p[my_rank]) + t, epoch, limit_ns, KID_BARRIER, t);
  }
}

// gshard[i] = scale * sum_r grads_r[lo + i]; partial[b] = sum of gshard^2 over this CTA's slice.
__global__ void __launch_bounds__(256) zero_reduce_kernel(PeerPtrs grads, int n, long long lo, long long cnt,
                                                          float scale, float* __restrict__ gshard,
                                                          float* __restrict__ partial) {
  __shared__ float red[32];
  float ss = 0.f;
  const long long nvec = cnt >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < n; ++r) {
      const float4 g = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(gshard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = np::warp_sum(ss);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = ss;
  __syncthreads();
  if (w == 0) {
    float t = l < 8 ? red[l] : 0.f;
    t = np::warp_sum(t);
    if (l == 0) partial[blockIdx.x] = t;
  }
}

// AdamW on this rank's shard, bf16 result stored into every rank's weight arena at [lo, lo+cnt).
__global__ void __launch_bounds__(256) zero_adamw_bcast_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                               float* __restrict__ m, float* __restrict__ v,
                                                               PeerPtrs w16, int n, long long lo, long long cnt,
                                                               float lr, float b1, float b2, float eps, float wd,
                                                               float bc1, float bc2, const float* __restrict__ gscale) {
  const float gs = gscale ? gscale[0] : 1.f;
  const long long nvec = cnt >> 2;
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
      P[j] = P[j] * (1.f - lr * wd) - lr * (M[j] / bc1) / (sqrtf(V[j] / bc2) + eps);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    const uint2 packed = make_uint2(np::pack_bf16(pp.x, pp.y), np::pack_bf16(pp.z, pp.w));
    for (int r = 0; r < n; ++r)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(w16.p[r]) + lo)[i] = packed;
  }
}

}  // namespace

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 500 + (int)e_; } while (0)

// Allocate `bytes` of device memory (zeroed) and export its IPC handle (64 bytes).
NP_API int np_symm_alloc(unsigned long long bytes, void** ptr, unsigned char* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return 100 + (int)e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return 200 + (int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return 300 + (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
NP_API int np_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : 100 + (int)e;
}
NP_API int np_symm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
NP_API int np_symm_free(void* ptr) { return (int)cudaFree(ptr); }

// flag_ptrs[r] = base of rank r's flag array (n ints per barrier slot).
NP_API int np_symm_barrier(void* const* flag_ptrs, int my_rank, int n, int epoch, unsigned long long limit_ns,
                           void* stream) {
  if (n > MAX_PEERS) return 1;
  PeerPtrs f;
  for (int i = 0; i < n; ++i) f.p[i] = flag_ptrs[i];
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, my_rank, n, epoch,
                                                          limit_ns ? limit_ns : NP_WAIT_LIMIT_NS);
  CHECK_LAUNCH();
}

NP_API int np_zero_parts() { return 148 * 4; }

// partial: fp32 [np_zero_parts()]. lo/cnt in elements; lo and cnt must be multiples of 4.
NP_API int np_zero_reduce(void* const* grad_ptrs, int n, long long lo, long long cnt, float scale, float* gshard,
                          float* partial, void* stream) {
  if (n > MAX_PEERS || (lo & 3) || (cnt & 3)) return 1;
  PeerPtrs g;
  for (int i = 0; i < n; ++i) g.p[i] = grad_ptrs[i];
  zero_reduce_kernel<<<np_zero_parts(), 256, 0, (cudaStream_t)stream>>>(g, n, lo, cnt, scale, gshard, partial);
  CHECK_LAUNCH();
}

NP_API int np_zero_adamw_bcast(float* p, const float* g, float* m, float* v, void* const* w16_ptrs, int n,
                               long long lo, long long cnt, float lr, float b1, float b2, float eps, float wd,
                               int step, const float* gscale, void* stream) {
  if (n > MAX_PEERS || (lo & 3) || (cnt & 3)) return 1;
  if (cnt <= 0) return 0;
  PeerPtrs w;
  for (int i = 0; i < n; ++i) w.p[i] = w16_ptrs[i];
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  zero_adamw_bcast_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, w, n, lo, cnt, lr, b1, b2, eps, wd,
                                                                    bc1, bc2, gscale);
  CHECK_LAUNCH();
}
