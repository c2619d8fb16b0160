// Block-scaled fp8 (e4m3) GEMM for sm_100a - the FP8-Flow-MoE expert GEMM.
//
//   C[M, N] = sum over 128-wide K blocks kb of  sa[m, kb] * sb[n / 128, kb] * (Aq[m, kb] . Bq[n, kb])
//
// Aq: e4m3 [M, K] with 1x128 scales sa [M, K/128];  Bq: e4m3 [N, K] with 128x128 scales sb [N/128, K/128]
// (DeepSeek-V3 recipe). tcgen05.mma kind::f8f6f4 computes each 128-deep partial product into a TMEM
// slot (4 slots of 128 columns, so the tensor core runs ahead); four promotion warps read a slot
// (tcgen05.ld), scale it by sa*sb in fp32 and add it to register accumulators (one output row per
// thread). fp32 scaling per K block is what the recipe asks for; hardware block scaling
// (kind::mxf8f6f4) only offers 1x32 power-of-two scales.
//
// Same roles, TMA pipeline, bounded waits, row-grouped mode (per-M-block expert offset, arrival-flag
// wait) and peer-push epilogue as the bf16 kernel in gemm_sm100.cu.
//
// Reference counterpart: fp8_grouped_gemm of the fp8_flow_moe package (torch._scaled_mm per the
// reference README); call sites model/moe.py:1313-1332,1557-1558.
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;  // 128 e4m3 = 128 B = one swizzle row, and one scale block
constexpr int STAGES = 6;
constexpr int SLOTS = 4;
constexpr int KID = 2;

struct Fp8Params {
  void* C;
  const float* sa;            // [M rows of A, K/128]
  const float* sb;            // [rows of B / 128, K/128]
  int M, N, K;
  long long ldc;
  int out_f32;
  int mode;                   // 0 dense, 1 row-grouped
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;  // B rows per group
  const int* ready_flags; const int* mblk_flag; int epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  const long long* row_dst; void* const* peer_base;
  int* done_counters; const int* done_expected; int* const* done_flag_ptr;
};

__global__ void __launch_bounds__(192, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
  constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (np::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto sfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto sempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + SLOTS + a); };
  uint8_t* tail = smem_raw + (bar_base - np::smem_u32(smem_raw)) + 8 * (2 * STAGES + 2 * SLOTS);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0);
  const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int nkb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { np::mbar_init(full_bar(s), 1); np::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < SLOTS; ++a) { np::mbar_init(sfull_bar(a), 1); np::mbar_init(sempty_bar(a), 4); }
    *abort_flag = 0;
    np::mbar_fence_init();
    np::tma_prefetch_desc(&tmA);
    np::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), SLOTS * BN);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  auto tile_rows = [&](int m_blk, int role) -> int {
    if (p.mode != 1) return BM;
    if (p.ready_flags) {
      const int fi = p.mblk_flag ? p.mblk_flag[m_blk] : 0;
      if (!np::wait_flag_ge(p.ready_flags + fi, epoch, p.flag_limit_ns, KID, 100 + role)) {
        *abort_flag = 1;
        return -1;
      }
    }
    return p.mblk_rows ? p.mblk_rows[m_blk] : BM;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const int m_blk = t % m_blocks, n_blk = t / m_blocks;
        const int rows = tile_rows(m_blk, 0);
        if (rows < 0) break;
        if (rows == 0) continue;
        long long brow = (long long)n_blk * BN;
        if (p.mode == 1 && p.mblk_group) brow += (long long)p.mblk_group[m_blk] * p.group_stride_b;
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          ok = np::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, KID, 1);
          if (!ok) break;
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          np::mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          np::tma_load_2d(sA, &tmA, full_bar(stage), kb * BK, m_blk * BM);
          np::tma_load_2d(sB, &tmB, full_bar(stage), kb * BK, (int)brow);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
      }
      if (*abort_flag) __nanosleep(1000000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = np::make_idesc(BM, BN, 0, 0, 0, 0);  // e4m3 x e4m3, fp32 accumulate, both K-major
      int stage = 0, slot = 0;
      uint32_t phase = 0, slot_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const int m_blk = t % m_blocks;
        const int rows = tile_rows(m_blk, 1);
        if (rows < 0) break;
        if (rows == 0) continue;
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          ok = np::mbar_wait(sempty_bar(slot), slot_phase ^ 1u, abort_flag, KID, 2) &&
               np::mbar_wait(full_bar(stage), phase, abort_flag, KID, 3);
          if (!ok) break;
          np::tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          const uint32_t tmem_d = tmem_base + (uint32_t)(slot * BN);
#pragma unroll
          for (int kk = 0; kk < BK / 32; ++kk) {  // K = 32 bytes of e4m3 per instruction
            const uint64_t ad = np::make_smem_desc(sA + kk * 32, 16, 1024);
            const uint64_t bd = np::make_smem_desc(sB + kk * 32, 16, 1024);
            np::tc_mma_f8(tmem_d, ad, bd, idesc, kk > 0 ? 1u : 0u);
          }
          np::tc_commit(empty_bar(stage));
          np::tc_commit(sfull_bar(slot));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++slot == SLOTS) { slot = 0; slot_phase ^= 1u; }
        }
        if (!ok) break;
      }
      if (*abort_flag) __nanosleep(1000000);
    }
  } else {
    const int quarter = warp & 3;
    int slot = 0;
    uint32_t slot_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      const int m_blk = t % m_blocks, n_blk = t / m_blocks;
      const int rows = tile_rows(m_blk, 2);
      if (rows < 0) break;
      if (rows == 0) continue;
      const int row = m_blk * BM + quarter * 32 + lane;
      const int row_c = row < p.M ? row : p.M - 1;
      long long bgrp = 0;
      if (p.mode == 1 && p.mblk_group) bgrp = (long long)p.mblk_group[m_blk] * (p.group_stride_b / 128);
      const float* sa_row = p.sa + (size_t)row_c * nkb;
      const float* sb_row = p.sb + (size_t)(bgrp + n_blk) * nkb;
      float acc[BN];
#pragma unroll
      for (int i = 0; i < BN; ++i) acc[i] = 0.f;
      bool ok = true;
      float sc_next = sa_row[0] * sb_row[0];
      for (int kb = 0; kb < nkb; ++kb) {
        const float sc = sc_next;
        if (kb + 1 < nkb) sc_next = sa_row[kb + 1] * sb_row[kb + 1];
        ok = np::mbar_wait(sfull_bar(slot), slot_phase, abort_flag, KID, 4);
        if (!ok) break;
        np::tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t)(slot * BN) + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          np::tmem_ld32(taddr + c * 32, r);
          np::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), sc, acc[c * 32 + i]);
        }
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(sempty_bar(slot));
        if (++slot == SLOTS) { slot = 0; slot_phase ^= 1u; }
      }
      if (!ok) break;
      // ---- epilogue from registers
      bool row_ok = row < p.M;
      char* crow;
      if (p.row_dst) {
        const long long d = row_ok ? p.row_dst[row] : -1;
        row_ok = row_ok && d >= 0;
        const long long peer = row_ok ? (d >> 40) : 0;
        crow = (char*)p.peer_base[peer] + (size_t)(d & ((1ll << 40) - 1)) * p.ldc * (p.out_f32 ? 4 : 2);
      } else {
        crow = (char*)p.C + (size_t)row * p.ldc * (p.out_f32 ? 4 : 2);
      }
      const int n0 = n_blk * BN;
      if (row_ok) {
        if (p.out_f32) {
          float* dst = (float*)crow + n0;
#pragma unroll
          for (int i = 0; i < BN / 4; ++i)
            if (n0 + 4 * i + 4 <= p.N)
              reinterpret_cast<float4*>(dst)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        } else {
          __nv_bfloat16* dst = (__nv_bfloat16*)crow + n0;
#pragma unroll
          for (int i = 0; i < BN / 8; ++i)
            if (n0 + 8 * i + 8 <= p.N)
              reinterpret_cast<uint4*>(dst)[i] =
                  make_uint4(np::pack_bf16(acc[8 * i], acc[8 * i + 1]), np::pack_bf16(acc[8 * i + 2], acc[8 * i + 3]),
                             np::pack_bf16(acc[8 * i + 4], acc[8 * i + 5]), np::pack_bf16(acc[8 * i + 6], acc[8 * i + 7]));
        }
      }
      if (p.done_counters) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int fi = p.mblk_flag ? p.mblk_flag[m_blk] : 0;
          const int done = atomicAdd(&p.done_counters[fi], 1) + 1;
          if (done == 4 * n_blocks * p.done_expected[fi]) {
            __threadfence_system();
            np::st_release_sys(p.done_flag_ptr[fi], epoch);
          }
        }
      }
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem_base, SLOTS * BN);
  }
}

}  // namespace

struct NpFp8GemmArgs {
  const void* A; const void* B; void* C; const float* sa; const float* sb;
  long long lda, ldb, ldc, a_rows, b_rows;
  int M, N, K, out_f32, mode;
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;
  const int* ready_flags; const int* mblk_flag; int epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  const long long* row_dst; void* const* peer_base;
  int* done_counters; const int* done_expected; int* const* done_flag_ptr;
  int max_ctas;
};

// C = blockwise-scaled A (e4m3, K-major) times B^T (e4m3, K-major). K, N multiples of 128; lda, ldb
// multiples of 16 bytes. Returns 0 or a set-up / launch error; device problems go to np_status_read.
NP_API int np_gemm_fp8_block(const NpFp8GemmArgs* args, void* stream) {
  const NpFp8GemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0) return 0;
  if (a.K % 128 || a.N % 8 || (a.lda % 16) || (a.ldb % 16) || (((uintptr_t)a.A) & 15) || (((uintptr_t)a.B) & 15))
    return 1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)
      return 2;
    ctx_bound = true;
  }
  CUtensorMap tmA, tmB;
  int rc = np_make_tmap_2d(&tmA, a.A, 1, (uint64_t)a.a_rows, (uint64_t)a.K, (uint64_t)a.lda, BK, BM);
  if (rc) return 100 + rc;
  rc = np_make_tmap_2d(&tmB, a.B, 1, (uint64_t)a.b_rows, (uint64_t)a.K, (uint64_t)a.ldb, BK, BN);
  if (rc) return 200 + rc;
  Fp8Params p{};
  p.C = a.C; p.sa = a.sa; p.sb = a.sb; p.M = a.M; p.N = a.N; p.K = a.K; p.ldc = a.ldc; p.out_f32 = a.out_f32;
  p.mode = a.mode; p.mblk_group = a.mblk_group; p.mblk_rows = a.mblk_rows; p.group_stride_b = a.group_stride_b;
  p.ready_flags = a.ready_flags; p.mblk_flag = a.mblk_flag; p.epoch = a.epoch; p.epoch_base = a.epoch_base;
  p.flag_limit_ns = a.flag_limit_ns ? a.flag_limit_ns : NP_WAIT_LIMIT_NS;
  p.row_dst = a.row_dst; p.peer_base = a.peer_base;
  p.done_counters = a.done_counters; p.done_expected = a.done_expected; p.done_flag_ptr = a.done_flag_ptr;
  constexpr int SMEM = STAGES * (BM * BK + BN * BK) + 1024 + 256;
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (long long)((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  const int cap = a.max_ctas > 0 ? a.max_ctas : sms;
  const int grid = (int)(tiles < cap ? tiles : cap);
  gemm_fp8_kernel<<<grid, 192, SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}
