// Shared device helpers for the sm_100a kernels of this library: inline-PTX wrappers for
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05 (TMEM alloc,
// MMA, commit, ld), bounded spin-waits and the status word every kernel reports through.
//
// Every wait in this library is bounded: after NP_WAIT_LIMIT_NS of polling the waiting thread
// records a code in the status buffer, raises the CTA-wide abort flag and returns false, so a
// kernel never hangs the GPU; the host reads the status after the launch (np_status_read).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#define NP_API extern "C" __attribute__((visibility("default")))

// Status codes written by kernels (0 = ok).
enum NpStatus : int {
  NP_OK = 0,
  NP_ERR_MBAR_TIMEOUT = 1,     // an mbarrier wait ran out
  NP_ERR_FLAG_TIMEOUT = 2,     // a wait on a global/peer flag ran out
  NP_ERR_BAD_ARG = 3,          // a kernel-side argument check failed
  NP_ERR_BOUNDS = 4,           // a bounds check recorded an index and skipped the access
};

// Global status buffer: [0]=code, [1]=kernel id, [2]=block, [3]=detail, [4..7]=extra.
// One per library instance; kernels only ever write a non-zero code (first writer wins).
extern __device__ int g_np_status[8];

// Communication-time accounting, per SM: the total length of the union of the intervals during which a thread
// on that SM was polling a flag that had not been raised yet, or a CTA of a kernel that only moves data between
// GPUs was running. The host reads the mean over the SMs per step as "exposed communication time": SM time that
// no tensor-core or elementwise work could use. Two arrays of NP_MAX_SMS entries (np_wait_stats_read).
#define NP_MAX_SMS 192
extern __device__ unsigned long long g_np_wait_end[NP_MAX_SMS];  // end (globaltimer) of the last counted interval
extern __device__ unsigned long long g_np_wait_ns[NP_MAX_SMS];   // accumulated union length in ns

#ifndef NP_WAIT_LIMIT_NS
#define NP_WAIT_LIMIT_NS 2000000000ull  // 2 s
#endif

namespace np {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Add [t0, t1) to this SM's communication time, counting only the part not already covered by an earlier
// interval (several CTAs of one SM usually wait at the same time).
__device__ __forceinline__ void account_interval(uint64_t t0, uint64_t t1) {
  unsigned sm;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  if (sm >= NP_MAX_SMS || t1 <= t0) return;
  const unsigned long long old = atomicMax(&g_np_wait_end[sm], (unsigned long long)t1);
  const unsigned long long from = old > t0 ? old : (unsigned long long)t0;
  if (t1 > from) atomicAdd(&g_np_wait_ns[sm], (unsigned long long)t1 - from);
}
// Counts the lifetime of thread 0 of a CTA as communication time (kernels whose only job is a transfer).
struct CommSpan {
  uint64_t t0;
  bool on;
  __device__ __forceinline__ explicit CommSpan(bool enable) : t0(0), on(enable && threadIdx.x == 0) {
    if (on) t0 = globaltimer_ns();
  }
  __device__ __forceinline__ ~CommSpan() {
    if (on) account_interval(t0, globaltimer_ns());
  }
};

__device__ __forceinline__ void report(int code, int kernel_id, int detail) {
  if (atomicCAS(&g_np_status[0], 0, code) == 0) {
    g_np_status[1] = kernel_id;
    g_np_status[2] = (int)blockIdx.x;
    g_np_status[3] = detail;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. `abort_flag` lives in shared memory; once any thread of the CTA gives up,
// every later wait in the CTA returns false at once so the CTA drains and exits.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int kernel_id, int detail) {
  if (mbar_try(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > NP_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        report(NP_ERR_MBAR_TIMEOUT, kernel_id, detail);
        return false;
      }
    }
  }
}

}  // namespace np
// Debug-bounds build: compile with -DNP_DEBUG (NPB200_NVCC_EXTRA=-DNP_DEBUG python -m nanopysche_b200.build --force).
// compute-sanitizer is not always available; these index predicates record (code 4, kernel id, block, offending
// value) in the status word and skip the access instead of trapping, so that a wrong index shows up as a readable
// status after the launch. In a normal build they compile to nothing.
#ifdef NP_DEBUG
#define NP_DBG_SKIP_UNLESS(cond, kid, detail) \
  if (!(cond)) {                              \
    np::report(NP_ERR_BOUNDS, kid, (int)(detail)); \
    continue;                                 \
  }
#else
#define NP_DBG_SKIP_UNLESS(cond, kid, detail)
#endif
namespace np {
// ------------------------------------------------------------------ global flags
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= want (flags are monotone epoch counters). Bounded; `limit_ns` lets tests
// use a short budget. Returns false (and reports) on timeout.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int want, uint64_t limit_ns,
                                             int kernel_id, int detail) {
  if (ld_acquire_sys(flag) >= want) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_sys(flag) >= want) {
      account_interval(t0, globaltimer_ns());
      return true;
    }
    if ((it & 63u) == 0u) {
      if (globaltimer_ns() - t0 > limit_ns) {
        report(NP_ERR_FLAG_TIMEOUT, kernel_id, detail);
        return false;
      }
      __nanosleep(200);
    }
  }
}

// ------------------------------------------------------------------ TMA (no multicast)
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16/f16 inputs, fp32 accumulate.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// e4m3/e5m2 inputs, fp32 accumulate (K = 32 per instruction).
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (warp%4)*32+t.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   K-major  operand: rows of 128 B along K, 8-row atoms of 1024 B; SBO = 1024, LBO unused.
//   MN-major operand: rows of 128 B along M/N (64 bf16), 8 K-rows per 1024 B atom;
//                     LBO = byte stride between 64-element M/N chunks, SBO = 1024.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp32 accumulate, M x N tile, operand formats and majors.
// fmt: kind::f16 -> 0 f16, 1 bf16 ; kind::f8f6f4 -> 0 e4m3, 1 e5m2.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_fmt, int b_fmt, int a_mn,
                                                  int b_mn) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------ small math helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
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

}  // namespace np

// ------------------------------------------------------------------ host helpers
// "Done once" guard for settings CUDA keeps per device (cudaFuncSetAttribute): a process that drives several
// GPUs has to repeat them on each one, so the flag is per device ordinal, not per process.
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
typedef CUresult (*NpEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
NpEncodeTiledFn np_get_encode_tiled();
// 2-D row-major tensor [rows, cols] of `elt_bytes` elements, row stride `ld` elements;
// box = box_cols x box_rows, 128-byte swizzle. Returns 0 on success.
int np_make_tmap_2d(CUtensorMap* out, const void* base, int elt_bytes, uint64_t rows, uint64_t cols,
                    uint64_t ld, uint32_t box_cols, uint32_t box_rows);
