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

__global__ void symm_barrier_kernel(PeerPtrs flags, int my_rank, int n, int epoch, const int* epoch_base,
                                    unsigned long long limit_ns) {
  const int t = threadIdx.x;
  const int ep = epoch + (epoch_base ? *epoch_base : 0);
  if (t < n) {
    __threadfence_system();
    np::st_release_sys(reinterpret_cast<int*>(flags.p[t]) + my_rank, ep);
    np::wait_flag_ge(reinterpret_cast<int*>(flags.p[my_rank]) + t, ep, limit_ns, KID_BARRIER, t);
  }
}

// Small all-reduce (sum) over peer memory: every rank stores its vector into slot [my_rank] of every
// peer's staging buffer, releases an epoch flag, waits for all peers' flags and sums the n slots.
// staging: [n ranks][count] floats per rank; one CTA per 1024 elements would be overkill - the vectors
// this is used for (gradient-norm partials, fp32 norm / router gradients) are a few MB at most.
__global__ void __launch_bounds__(256) symm_allreduce_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                             PeerPtrs staging, PeerPtrs flags, int* __restrict__ ctr,
                                                             long long half_elems, long long count, int my_rank, int n,
                                                             int epoch,
                                                             const int* epoch_base, float scale,
                                                             unsigned long long limit_ns) {
  const int ep = epoch + (epoch_base ? *epoch_base : 0);
  // ctr[1] counts the calls: its parity picks one of two staging halves, so a fast rank that is already
  // in the next call never overwrites a slot a slow rank is still summing
  const size_t half = (size_t)(ctr[1] & 1) * (size_t)half_elems;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < count; i += nth) {
    const float v = src[i];
    for (int r = 0; r < n; ++r) reinterpret_cast<float*>(staging.p[r])[half + (size_t)my_rank * count + i] = v;
  }
  // grid-wide: last CTA to finish its stores releases the flags (threadfence-reduction pattern)
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < n) np::st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + my_rank, ep);
    if (threadIdx.x == 0) { ctr[0] = 0; ctr[1] += 1; }
  }
  // every CTA waits for all ranks' contributions, then reduces its slice
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    if (!np::wait_flag_ge(reinterpret_cast<int*>(flags.p[my_rank]) + threadIdx.x, ep, limit_ns, KID_BARRIER,
                          100 + threadIdx.x))
      s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const float* mine = reinterpret_cast<const float*>(staging.p[my_rank]) + half;
  for (long long i = tid; i < count; i += nth) {
    float acc = 0.f;
    for (int r = 0; r < n; ++r) acc += mine[(size_t)r * count + i];
    dst[i] = acc * scale;
  }
}

// All-gather as peer stores: this rank's shard (vecs x 16 bytes) is written into every rank's gather
// buffer at the shard's offset, then flag [my_rank] is released on every rank. The consumer (a GEMM
// with a per-M-block flag wait) can start on a shard as soon as that shard's flag arrives.
__global__ void __launch_bounds__(256) allgather_push_kernel(const uint4* __restrict__ src, PeerPtrs dst,
                                                             long long vecs, long long dst_off_vecs, PeerPtrs flags,
                                                             int* __restrict__ ctr, int my_rank, int n, int epoch,
                                                             const int* epoch_base) {
  np::CommSpan span(n > 1);
  const int ep = epoch + (epoch_base ? *epoch_base : 0);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int r = 0; r < n; ++r) reinterpret_cast<uint4*>(dst.p[r])[dst_off_vecs + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < n) np::st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + my_rank, ep);
    if (threadIdx.x == 0) *ctr = 0;
  }
}

// All-to-all as peer stores: every row of `src` (row_vecs x 16 bytes) is cut into n equal slices and slice r of
// every row is stored into rank r's buffer at [my_rank][row][slice]; with `set_flag` the last CTA releases
// flag [my_rank] on every rank (several tensors can share one flag: only the last push sets it, stream order
// makes the earlier ones complete first).
__global__ void __launch_bounds__(256) a2a_push_kernel(const uint4* __restrict__ src, long long rows,
                                                       long long row_vecs, PeerPtrs dst, PeerPtrs flags,
                                                       int* __restrict__ ctr, int my_rank, int n, int epoch,
                                                       const int* epoch_base, int set_flag) {
  np::CommSpan span(n > 1);
  const long long slice_vecs = row_vecs / n;
  const long long total = rows * row_vecs;
  const long long base = (long long)my_rank * rows * slice_vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / row_vecs, c = i - row * row_vecs;
    const int r = (int)(c / slice_vecs);
    reinterpret_cast<uint4*>(dst.p[r])[base + row * slice_vecs + (c - r * slice_vecs)] = src[i];
  }
  if (!set_flag) return;
  const int ep = epoch + (epoch_base ? *epoch_base : 0);
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < n) np::st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + my_rank, ep);
    if (threadIdx.x == 0) *ctr = 0;
  }
}

// out[i] = sum_r src_r[off + i] over bf16 buffers that live on the n ranks (peer loads, fp32 accumulation): the
// reduction half of a reduce-scatter whose partial results were written locally by each rank's GEMM.
__global__ void __launch_bounds__(256) rs_reduce_bf16_kernel(PeerPtrs src, int n, long long off_vecs, long long vecs,
                                                             uint4* __restrict__ out) {
  np::CommSpan span(n > 1);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < n; ++r) {
      const uint4 u = reinterpret_cast<const uint4*>(src.p[r])[off_vecs + i];
      const float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    out[i] = make_uint4(np::pack_bf16(acc[0], acc[1]), np::pack_bf16(acc[2], acc[3]), np::pack_bf16(acc[4], acc[5]),
                        np::pack_bf16(acc[6], acc[7]));
  }
}

// gshard[i] = scale * sum_r grads_r[lo + i]; partial[b] = sum of gshard^2 over this CTA's slice.
__global__ void __launch_bounds__(256) zero_reduce_kernel(PeerPtrs grads, int n, long long lo, long long cnt,
                                                          float scale, float* __restrict__ gshard,
                                                          float* __restrict__ partial) {
  __shared__ float red[32];
  np::CommSpan span(n > 1);
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
                                                               float bc1, float bc2, const float* __restrict__ gscale,
                                                               const float* __restrict__ hyper, long long slice,
                                                               long long bstride) {
  np::CommSpan span(n > 1);
  const float gs = gscale ? gscale[0] : 1.f;
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }
  const long long nvec = cnt >> 2;
  const long long svec = slice >> 2;   // bucketed layout: shard element 4i lives at flat (4i / slice) * bstride + lo + 4i % slice
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
    const long long fv = svec > 0 ? (i / svec) * (bstride >> 2) + (i % svec) : i;   // position in float4 units after lo
    for (int r = 0; r < n; ++r)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(w16.p[r]) + lo)[fv] = packed;
  }
}

// Copy-engine form of the overlapped reduce-scatter. bucket_sync_kernel (one warp) announces "bucket b is final on
// this rank" to every rank and waits for everyone's announcement; the host then queues one cudaMemcpyAsync per peer
// (peer gradient slice -> local staging), which the copy engines move over NVLink without occupying an SM, so the
// tensor-core kernels of the backward pass keep all SMs to themselves. After the backward pass
// zero_reduce_staged_kernel sums the local slice and the staged peer slices at HBM speed.
__global__ void bucket_sync_kernel(PeerPtrs flags, int flag_off, int my_rank, int n, int epoch,
                                   const int* __restrict__ epoch_base, unsigned long long limit_ns) {
  const int t = threadIdx.x;
  const int ep = epoch + (epoch_base ? *epoch_base : 0);
  if (t < n) {
    __threadfence_system();
    np::st_release_sys(reinterpret_cast<int*>(flags.p[t]) + flag_off + my_rank, ep);
    np::wait_flag_ge(reinterpret_cast<int*>(flags.p[my_rank]) + flag_off + t, ep, limit_ns, KID_BARRIER, 300 + t);
  }
}

// gshard[i] = scale * (local[flat(i)] + sum over the staged peer copies of element i), i over this rank's compact
// shard (slices of `slice` elements, slice k at flat offset lo + k * bstride in the local gradient buffer; the staged
// copies already use the compact order, `cnt` elements per peer). partial[block] = sum of squares of the CTA's part.
__global__ void __launch_bounds__(256) zero_reduce_staged_kernel(const float* __restrict__ local, long long lo,
                                                                 long long slice, long long bstride,
                                                                 const float* __restrict__ staged, int n_staged,
                                                                 long long cnt, float scale, float* __restrict__ gshard,
                                                                 float* __restrict__ partial) {
  __shared__ float red[32];
  float ss = 0.f;
  const long long nvec = cnt >> 2, svec = slice >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long fv = (i / svec) * (bstride >> 2) + (i % svec);
    float4 acc = reinterpret_cast<const float4*>(local + lo)[fv];
    for (int k = 0; k < n_staged; ++k) {
      const float4 g = reinterpret_cast<const float4*>(staged + (size_t)k * cnt)[i];
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

// The same two kernels through an NVLink multicast mapping of the gradient / weight arenas (NVLS): one
// multimem.ld_reduce returns the sum over all ranks, formed inside the switch, so a rank receives its shard once
// instead of once per peer; one multimem.st delivers the updated bf16 weights to every rank.
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_bf16x4(void* mc, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(mc), "r"(a), "r"(b) : "memory");
}

__global__ void __launch_bounds__(256) zero_reduce_mc_kernel(const float* __restrict__ mc_grads, long long lo,
                                                             long long cnt, float scale, float* __restrict__ gshard,
                                                             float* __restrict__ partial) {
  __shared__ float red[32];
  np::CommSpan span(true);
  float ss = 0.f;
  const long long nvec = cnt >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = mc_ld_reduce_f32x4(mc_grads + lo + 4 * i);
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

__global__ void __launch_bounds__(256) zero_adamw_bcast_mc_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                                  float* __restrict__ m, float* __restrict__ v,
                                                                  __nv_bfloat16* __restrict__ mc_w16, long long lo,
                                                                  long long cnt, float lr, float b1, float b2, float eps,
                                                                  float wd, float bc1, float bc2,
                                                                  const float* __restrict__ gscale,
                                                                  const float* __restrict__ hyper) {
  np::CommSpan span(true);
  const float gs = gscale ? gscale[0] : 1.f;
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }
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
    mc_st_bf16x4(mc_w16 + lo + 4 * i, np::pack_bf16(pp.x, pp.y), np::pack_bf16(pp.z, pp.w));
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
NP_API int np_symm_barrier(void* const* flag_ptrs, int my_rank, int n, int epoch, const int* epoch_base,
                           unsigned long long limit_ns, void* stream) {
  if (n > MAX_PEERS) return 1;
  PeerPtrs f;
  for (int i = 0; i < n; ++i) f.p[i] = flag_ptrs[i];
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, my_rank, n, epoch, epoch_base,
                                                          limit_ns ? limit_ns : NP_WAIT_LIMIT_NS);
  CHECK_LAUNCH();
}

// dst[i] = scale * sum over ranks of src[i]; staging_ptrs[r] = rank r's staging buffer of 2 * half_elems floats
// (half_elems >= n * count), flag_ptrs[r] = rank r's n-int flag array, ctr = two zeroed local ints.
// src/dst may alias.
NP_API int np_symm_allreduce(const float* src, float* dst, void* const* staging_ptrs, void* const* flag_ptrs,
                             int* ctr, long long half_elems, long long count, int my_rank, int n, int epoch,
                             const int* epoch_base,
                             float scale, unsigned long long limit_ns, void* stream) {
  if (n > MAX_PEERS || n > 256 || (long long)n * count > half_elems) return 1;
  if (count <= 0) return 0;
  PeerPtrs st, fl;
  for (int i = 0; i < n; ++i) { st.p[i] = staging_ptrs[i]; fl.p[i] = flag_ptrs[i]; }
  long long g = (count + 255) / 256;
  if (g > 148) g = 148;  // all CTAs are co-resident (they wait on one another through the counter)
  symm_allreduce_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(src, dst, st, fl, ctr, half_elems, count, my_rank, n,
                                                                  epoch, epoch_base, scale,
                                                                  limit_ns ? limit_ns : NP_WAIT_LIMIT_NS);
  CHECK_LAUNCH();
}

// src: this rank's shard (bytes, multiple of 16); gather_ptrs[r]: rank r's gather buffer; the shard lands at
// byte offset my_rank * bytes; flag_ptrs[r]: rank r's n-int flag array; ctr: a zeroed local int.
NP_API int np_allgather_push(const void* src, void* const* gather_ptrs, long long bytes, void* const* flag_ptrs,
                             int* ctr, int my_rank, int n, int epoch, const int* epoch_base, int max_ctas,
                             void* stream) {
  if (n > MAX_PEERS || (bytes & 15) || (((uintptr_t)src) & 15)) return 1;
  if (bytes <= 0) return 0;
  PeerPtrs d, f;
  for (int i = 0; i < n; ++i) { d.p[i] = gather_ptrs[i]; f.p[i] = flag_ptrs[i]; }
  const long long vecs = bytes >> 4;
  long long g = (vecs + 255) / 256;
  const int cap = max_ctas > 0 ? max_ctas : 148 * 2;
  if (g > cap) g = cap;
  allgather_push_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, d, vecs, (long long)my_rank * vecs,
                                                                  f, ctr, my_rank, n, epoch, epoch_base);
  CHECK_LAUNCH();
}

// src: [rows, row_bytes] contiguous; dst_ptrs[r]: rank r's buffer of n x rows x (row_bytes / n) bytes; the slice of
// this rank's rows lands at index my_rank. flag_ptrs / ctr as in np_allgather_push (used when set_flag != 0).
NP_API int np_a2a_push(const void* src, long long rows, long long row_bytes, void* const* dst_ptrs,
                       void* const* flag_ptrs, int* ctr, int my_rank, int n, int epoch, const int* epoch_base,
                       int set_flag, int max_ctas, void* stream) {
  if (n > MAX_PEERS || (row_bytes % (16 * n)) || (((uintptr_t)src) & 15)) return 1;
  if (rows <= 0) return 0;
  PeerPtrs d, f;
  for (int i = 0; i < n; ++i) { d.p[i] = dst_ptrs[i]; f.p[i] = flag_ptrs ? flag_ptrs[i] : nullptr; }
  const long long vecs = rows * (row_bytes >> 4);
  long long g = (vecs + 255) / 256;
  const int cap = max_ctas > 0 ? max_ctas : 148 * 2;
  if (g > cap) g = cap;
  a2a_push_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, rows, row_bytes >> 4, d, f, ctr, my_rank, n,
                                                            epoch, epoch_base, set_flag);
  CHECK_LAUNCH();
}

// out[count] (bf16) = sum over the n ranks of their bf16 buffer at element offset `off` (off, count multiples of 8).
NP_API int np_rs_reduce_bf16(void* const* src_ptrs, int n, long long off, long long count, void* out, void* stream) {
  if (n > MAX_PEERS || (off & 7) || (count & 7)) return 1;
  if (count <= 0) return 0;
  PeerPtrs s;
  for (int i = 0; i < n; ++i) s.p[i] = src_ptrs[i];
  long long g = ((count >> 3) + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  rs_reduce_bf16_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(s, n, off >> 3, count >> 3, (uint4*)out);
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

NP_API int np_bucket_sync(void* const* flag_ptrs, int bucket, int my_rank, int n, int epoch, const int* epoch_base,
                          unsigned long long limit_ns, void* stream) {
  if (n > MAX_PEERS || n > 32) return 1;
  PeerPtrs f;
  for (int i = 0; i < n; ++i) f.p[i] = flag_ptrs[i];
  bucket_sync_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, bucket * n, my_rank, n, epoch, epoch_base,
                                                         limit_ns ? limit_ns : NP_WAIT_LIMIT_NS);
  CHECK_LAUNCH();
}

// Stream-ordered copy between any two device addresses of the unified address space (a peer's buffer mapped through
// CUDA IPC included): one plain cudaMemcpyAsync, executed by a copy engine.
NP_API int np_memcpy_async(void* dst, const void* src, unsigned long long bytes, void* stream) {
  if (bytes == 0) return 0;
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream);
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// partial: fp32 [np_zero_parts()]; see zero_reduce_staged_kernel.
NP_API int np_zero_reduce_staged(const float* local, long long lo, long long slice, long long bstride,
                                 const float* staged, int n_staged, long long cnt, float scale, float* gshard,
                                 float* partial, void* stream) {
  if ((lo & 3) || (cnt & 3) || (slice & 3) || (bstride & 3) || slice <= 0) return 1;
  zero_reduce_staged_kernel<<<np_zero_parts(), 256, 0, (cudaStream_t)stream>>>(local, lo, slice, bstride, staged,
                                                                              n_staged, cnt, scale, gshard, partial);
  CHECK_LAUNCH();
}

// slice > 0: the shard is `cnt / slice` slices of `slice` elements, slice k at flat offset lo + k * bstride (the
// bucketed layout of the overlapped reduce-scatter); slice == 0: one contiguous range [lo, lo + cnt).
NP_API int np_zero_adamw_bcast(float* p, const float* g, float* m, float* v, void* const* w16_ptrs, int n,
                               long long lo, long long cnt, float lr, float b1, float b2, float eps, float wd,
                               int step, const float* gscale, const float* hyper, long long slice, long long bstride,
                               void* stream) {
  if (n > MAX_PEERS || (lo & 3) || (cnt & 3) || (slice & 3) || (bstride & 3)) return 1;
  if (cnt <= 0) return 0;
  PeerPtrs w;
  for (int i = 0; i < n; ++i) w.p[i] = w16_ptrs[i];
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  zero_adamw_bcast_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, w, n, lo, cnt, lr, b1, b2, eps, wd,
                                                                    bc1, bc2, gscale, hyper, slice, bstride);
  CHECK_LAUNCH();
}

// NVLS forms of np_zero_reduce / np_zero_adamw_bcast: mc_grads / mc_w16 are the multicast addresses of the
// gradient / weight arenas (memory of every rank bound to one NVLink multicast object at the same offsets).
NP_API int np_zero_reduce_mc(const float* mc_grads, long long lo, long long cnt, float scale, float* gshard,
                             float* partial, void* stream) {
  if ((lo & 3) || (cnt & 3) || (((uintptr_t)mc_grads) & 15)) return 1;
  zero_reduce_mc_kernel<<<np_zero_parts(), 256, 0, (cudaStream_t)stream>>>(mc_grads, lo, cnt, scale, gshard, partial);
  CHECK_LAUNCH();
}

NP_API int np_zero_adamw_bcast_mc(float* p, const float* g, float* m, float* v, void* mc_w16, long long lo,
                                  long long cnt, float lr, float b1, float b2, float eps, float wd, int step,
                                  const float* gscale, const float* hyper, void* stream) {
  if ((lo & 3) || (cnt & 3) || (((uintptr_t)mc_w16) & 15)) return 1;
  if (cnt <= 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  zero_adamw_bcast_mc_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, (__nv_bfloat16*)mc_w16, lo, cnt, lr,
                                                                       b1, b2, eps, wd, bc1, bc2, gscale, hyper);
  CHECK_LAUNCH();
}
