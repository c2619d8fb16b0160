// Row permutation for grouped expert GEMMs (sm_100a), the index half of FP8-Flow-MoE:
//   expert_rank     stable position of every row inside its expert's padded segment (counting sort, no argsort),
//                   plus the padded segment sizes
//   permute_rows    out[row_map[i]] = x[i]            (padding rows stay zero)
//   unpermute_rows  out[i] = y[row_map[i]] (* w[i])
// Reference names: fused_permute_pad / fused_unpermute_unpad of the fp8_flow_moe package (fp8/__init__.py:8-22 of
// the reference; its implementation is not in that tree, only the call sites at model/moe.py:1313-1332).
#include "fp8_common.cuh"

namespace {

// One CTA of 1024 threads. counts -> padded sizes and segment starts -> for every expert a pass over the rows with a
// block-wide ballot scan, so equal-expert rows keep their input order (the stable order argsort would give).
__global__ void __launch_bounds__(1024) expert_rank_kernel(const long long* __restrict__ indices, int n, int E,
                                                           int pad_multiple, long long* __restrict__ row_map,
                                                           long long* __restrict__ padded_out) {
  extern __shared__ int sm[];          // counts[E], starts[E], warp_sums[32], running
  int* counts = sm;
  int* starts = sm + E;
  int* wsum = sm + 2 * E;
  int* running = wsum + 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const long long e = indices[i];
    if (e >= 0 && e < E) atomicAdd(&counts[(int)e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      const int p = (counts[e] + pad_multiple - 1) / pad_multiple * pad_multiple;
      starts[e] = acc;
      padded_out[e] = p;
      acc += p;
    }
  }
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    if (counts[e] == 0) continue;               // uniform across the CTA
    if (tid == 0) *running = starts[e];
    __syncthreads();
    for (int base = 0; base < n; base += blockDim.x) {
      const int i = base + tid;
      const bool hit = i < n && indices[i] == e;
      const unsigned bal = __ballot_sync(0xffffffffu, hit);
      if (lane == 0) wsum[warp] = __popc(bal);
      __syncthreads();
      int before = 0, total = 0;
      for (int w = 0; w < 32; ++w) {
        const int c = wsum[w];
        before += (w < warp) ? c : 0;
        total += c;
      }
      if (hit) row_map[i] = *running + before + __popc(bal & ((1u << lane) - 1u));
      __syncthreads();
      if (tid == 0) *running += total;
      __syncthreads();
    }
  }
}

// One warp per row, 16-byte vectors. scatter = 1: out[map[i]] = x[i]; scatter = 0: out[i] = x[map[i]] * w[i].
__global__ void __launch_bounds__(256) move_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                                        const long long* __restrict__ map,
                                                        const float* __restrict__ w, long long n, int vecs,
                                                        int scatter) {
  const long long warp_g = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long i = warp_g; i < n; i += nwarps) {
    const long long m = map[i];
    const uint4* src = x + (scatter ? i : m) * vecs;
    uint4* dst = out + (scatter ? m : i) * vecs;
    const float sc = (!scatter && w) ? w[i] : 1.f;
    for (int v = lane; v < vecs; v += 32) {
      uint4 u = src[v];
      if (sc != 1.f) {
        const float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
        u = make_uint4(np::pack_bf16(a.x * sc, a.y * sc), np::pack_bf16(b.x * sc, b.y * sc),
                       np::pack_bf16(c.x * sc, c.y * sc), np::pack_bf16(d.x * sc, d.y * sc));
      }
      dst[v] = u;
    }
  }
}

}  // namespace

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 500 + (int)e_; } while (0)

// indices: int64 [n] expert of every row; row_map: int64 [n] (out), padded: int64 [E] (out).
NP_API int np_expert_rank(const long long* indices, int n, int E, int pad_multiple, long long* row_map,
                          long long* padded, void* stream) {
  if (n < 0 || E <= 0 || E > 4096 || pad_multiple <= 0) return 1;
  const size_t smem = (2 * (size_t)E + 33) * sizeof(int);
  expert_rank_kernel<<<1, 1024, smem, (cudaStream_t)stream>>>(indices, n, E, pad_multiple, row_map, padded);
  CHECK_LAUNCH();
}

// Rows of `row_bytes` bytes (a multiple of 16, 16-byte aligned buffers). scatter: out[map[i]] = x[i] for i < n;
// gather: out[i] = x[map[i]] times w[i] when w is given (bf16 rows only).
NP_API int np_move_rows(const void* x, void* out, const long long* map, const float* w, long long n,
                        long long row_bytes, int scatter, void* stream) {
  if (n <= 0) return 0;
  if ((row_bytes & 15) || (((uintptr_t)x) & 15) || (((uintptr_t)out) & 15)) return 1;
  long long blocks = (n + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  move_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)out, map, w, n,
                                                                   (int)(row_bytes >> 4), scatter);
  CHECK_LAUNCH();
}
