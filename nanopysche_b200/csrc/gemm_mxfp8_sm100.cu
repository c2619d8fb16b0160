// MXFP8 GEMM for sm_100a: e4m3 operands with one power-of-two (UE8M0) scale per 1x32 block along K, scaled by the
// tensor core itself (tcgen05.mma kind::mxf8f6f4.block_scale).
//
//   C[M, N] = sum_k  2^(sa[m, k/32] - 127) * Aq[m, k]  *  2^(sb[n, k/32] - 127) * Bq[n, k]
//
// Aq [M, K], Bq [N, K]: e4m3, K-major. Scales travel in the layout the tensor core reads: for every (128-row block,
// 128-wide K block) one 512-byte chunk in which row r and 32-block j sit at byte (r % 32) * 16 + (r / 32) * 4 + j,
// chunks ordered [row block][K block]. The quantiser (mx_quant_kernel below) writes that layout directly, so a
// chunk is one 512-byte bulk copy into shared memory and one tcgen05.cp (32 lanes x 128 bit, replicated to the four
// lane quarters) into tensor memory.
//
// CTA roles: warp 0 lane 0 issues the copies (TMA tiles of A and B, bulk copies of the scale chunks) into a
// 5-stage ring; warp 1 lane 0 copies the scales of a stage into TMEM and issues four K = 32 MMAs whose instruction
// descriptors select byte 0..3 of the scale words; warps 2-5 drain one of two 192-column accumulators (tcgen05.ld)
// while the next tile accumulates into the other. The tile is 128 x 192: two 192-column fp32 accumulators plus the
// scale columns fit the 512 TMEM columns (two 256-column ones would leave none for the scales), and the operand
// bytes per FLOP that cross from L2 drop by a fifth against a 128 x 128 tile. A 192-row B tile starts at row 0 or
// 64 of a 128-row scale chunk, so both chunks it touches are copied and the MMA's B-scale address is offset by
// (row % 128) / 32 columns. Accumulation over the whole K stays in TMEM - no per-block
// promotion in registers as in the 1x128 / 128x128 kernel of gemm_fp8_sm100.cu. Row-grouped mode (one B row offset
// per 128-row block of A) serves grouped expert GEMMs. Every wait is bounded and reports through the status word.
//
// Reference counterpart: the `mxfp8` recipe of --fp8-recipe (cli.py:28-186 of the reference), which defers to
// torchao's MX linear (torch._scaled_mm with 1x32 e8m0 scales).
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 192;   // 1.5 scale chunks of B per tile: a tile starts at row 0 or 64 of a 128-row chunk
constexpr int BK = 128;   // four MMAs of K = 32; one scale chunk of A and two of B per stage
constexpr int STAGES = 5;
constexpr int KID_MX = 3;
constexpr int SF_BYTES = 512;
constexpr int SF_SMEM = 2048;             // A chunk + two B chunks, padded so that stages stay 1024-byte aligned
constexpr int SF_COLS = 12;               // TMEM columns per stage: 4 for A, 8 for the two B chunks
constexpr int TMEM_COLS = 512;            // 2 x 192 accumulator columns + 12 scale columns per stage
constexpr int SF_COL0 = 2 * BN;

struct MxParams {
  void* C;
  const uint8_t* sfa;          // [ceil(a_rows / 128)][K / 128][512]
  const uint8_t* sfb;          // [b_rows / 128][K / 128][512]
  int M, N, K;
  long long ldc;
  int out_f32;
  int mode;                    // 0 dense, 1 row-grouped
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;
  long long b_chunks;          // 128-row scale chunks of B
};

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Shared-memory descriptor without swizzle: 8-row x 16-byte core matrices, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, the same data in all four lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_taddr, uint32_t sfb_taddr, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_taddr), "r"(sfb_taddr), "r"(accumulate)
      : "memory");
}
// Block-scaled instruction descriptor: e4m3 x e4m3 (formats 0), both K-major, UE8M0 scales (bit 23), N >> 3 at
// bit 17, M >> 4 at bit 24, scale byte selectors for B at bit 4 and for A at bit 29.
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n, int a_sf, int b_sf) {
  return ((uint32_t)b_sf << 4) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24) |
         ((uint32_t)a_sf << 29);
}

__global__ void __launch_bounds__(192, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxParams p) {
  constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES + SF_SMEM;
  constexpr int TX_BYTES = A_BYTES + B_BYTES + 3 * SF_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (np::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto afull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto aempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint8_t* tail = smem_raw + (bar_base - np::smem_u32(smem_raw)) + 8 * (2 * STAGES + 4);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int nkb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { np::mbar_init(full_bar(s), 1); np::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { np::mbar_init(afull_bar(a), 1); np::mbar_init(aempty_bar(a), 4); }
    *abort_flag = 0;
    np::mbar_fence_init();
    np::tma_prefetch_desc(&tmA);
    np::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), TMEM_COLS);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  auto tile_rows = [&](int m_blk) -> int {
    if (p.mode != 1) return BM;
    return p.mblk_rows ? p.mblk_rows[m_blk] : BM;
  };
  auto b_row0 = [&](int m_blk, int n_blk) -> long long {
    long long brow = (long long)n_blk * BN;
    if (p.mode == 1 && p.mblk_group) brow += (long long)p.mblk_group[m_blk] * p.group_stride_b;
    return brow;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const int m_blk = t % m_blocks, n_blk = t / m_blocks;
        if (tile_rows(m_blk) == 0) continue;
        const long long brow = b_row0(m_blk, n_blk);
        const uint8_t* sfa = p.sfa + (size_t)m_blk * nkb * SF_BYTES;
        // the two 128-row scale chunks of B that cover rows [brow, brow + 192); past the last chunk the last one is
        // read again (those output columns lie beyond N and are never stored)
        const long long c0 = brow / 128, c1 = (c0 + 1 < p.b_chunks) ? c0 + 1 : p.b_chunks - 1;
        const uint8_t* sfb0 = p.sfb + (size_t)c0 * nkb * SF_BYTES;
        const uint8_t* sfb1 = p.sfb + (size_t)c1 * nkb * SF_BYTES;
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          ok = np::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, KID_MX, 1);
          if (!ok) break;
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES, sSF = sB + B_BYTES;
          np::mbar_expect_tx(full_bar(stage), TX_BYTES);
          np::tma_load_2d(sA, &tmA, full_bar(stage), kb * BK, m_blk * BM);
          np::tma_load_2d(sB, &tmB, full_bar(stage), kb * BK, (int)brow);
          bulk_load(sSF, sfa + (size_t)kb * SF_BYTES, SF_BYTES, full_bar(stage));
          bulk_load(sSF + SF_BYTES, sfb0 + (size_t)kb * SF_BYTES, SF_BYTES, full_bar(stage));
          bulk_load(sSF + 2 * SF_BYTES, sfb1 + (size_t)kb * SF_BYTES, SF_BYTES, full_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
      }
      if (*abort_flag) __nanosleep(1000000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const int m_blk = t % m_blocks, n_blk = t / m_blocks;
        if (tile_rows(m_blk) == 0) continue;
        // B scales of the tile's first row sit in column (row % 128) / 32 of the first chunk's four columns
        const uint32_t sfb_off = (uint32_t)((b_row0(m_blk, n_blk) % 128) / 32);
        bool ok = np::mbar_wait(aempty_bar(acc), acc_phase ^ 1u, abort_flag, KID_MX, 2);
        if (!ok) break;
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < nkb && ok; ++kb) {
          ok = np::mbar_wait(full_bar(stage), phase, abort_flag, KID_MX, 3);
          if (!ok) break;
          np::tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES, sSF = sB + B_BYTES;
          const uint32_t t_sfa = tmem_base + (uint32_t)(SF_COL0 + stage * SF_COLS), t_sfb = t_sfa + 4;
          tmem_cp_32x128b_x4(t_sfa, desc_noswizzle(sSF, 16, 128));
          tmem_cp_32x128b_x4(t_sfb, desc_noswizzle(sSF + SF_BYTES, 16, 128));
          tmem_cp_32x128b_x4(t_sfb + 4, desc_noswizzle(sSF + 2 * SF_BYTES, 16, 128));
#pragma unroll
          for (int kk = 0; kk < BK / 32; ++kk) {
            const uint64_t ad = np::make_smem_desc(sA + kk * 32, 16, 1024);
            const uint64_t bd = np::make_smem_desc(sB + kk * 32, 16, 1024);
            np::tc_fence_after();
            tc_mma_mxf8(tmem_d, ad, bd, make_idesc_mx(BM, BN, kk, kk), t_sfa, t_sfb + sfb_off, (kb | kk) ? 1u : 0u);
          }
          np::tc_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        np::tc_commit(afull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (*abort_flag) __nanosleep(1000000);
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      const int m_blk = t % m_blocks, n_blk = t / m_blocks;
      const int rows = tile_rows(m_blk);
      if (rows == 0) continue;
      if (!np::mbar_wait(afull_bar(acc), acc_phase, abort_flag, KID_MX, 4)) break;
      np::tc_fence_after();
      const int r_in = quarter * 32 + lane;
      const int row = m_blk * BM + r_in;
      const bool row_ok = row < p.M && r_in < rows;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
      char* crow = (char*)p.C + (size_t)row * p.ldc * (p.out_f32 ? 4 : 2);
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        np::tmem_ld32(taddr + c * 32, r);        // warp-uniform: every lane loads, only stores are guarded
        np::tmem_ld_wait();
        if (row_ok) {
          if (p.out_f32) {
            float* dst = (float*)crow + n0 + c * 32;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (n0 + c * 32 + 4 * i + 4 <= p.N)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          } else {
            __nv_bfloat16* dst = (__nv_bfloat16*)crow + n0 + c * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (n0 + c * 32 + 8 * i + 8 <= p.N)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(
                    np::pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                    np::pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                    np::pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                    np::pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
          }
        }
      }
      np::tc_fence_before();
      __syncwarp();
      if (lane == 0) np::mbar_arrive(aempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------- quantiser
__device__ __forceinline__ uint32_t to_e4m3(float v) {
  return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// One thread per 1x32 block: amax -> power-of-two scale 2^e with amax / 2^e <= 448 (e = ceil(log2(amax / 448))),
// e4m3 values and the biased exponent byte in the tensor core's chunk layout.
__global__ void __launch_bounds__(256) mx_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                       uint8_t* __restrict__ q, long long ldq,
                                                       uint8_t* __restrict__ sf, int rows, int K) {
  const int bpr = K / 32;
  const long long total = (long long)rows * bpr;
  const int nkb = K / 128;
  for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < total;
       b += (long long)gridDim.x * blockDim.x) {
    const long long row = b / bpr;
    const int kb32 = (int)(b - row * bpr);
    const uint4* src = reinterpret_cast<const uint4*>(x + row * ldx + kb32 * 32);
    float f[32];
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = src[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = np::unpack_bf16(w[j]);
        f[i * 8 + 2 * j] = v.x;
        f[i * 8 + 2 * j + 1] = v.y;
        am = fmaxf(am, fmaxf(fabsf(v.x), fabsf(v.y)));
      }
    }
    int e = -127;
    if (am > 0.f) {
      int ex;
      const float mant = frexpf(__fdiv_rn(am, 448.f), &ex);    // am / 448 = mant * 2^ex, mant in [0.5, 1)
      e = (mant == 0.5f) ? ex - 1 : ex;                     // ceil(log2(am / 448))
      e = max(-127, min(127, e));
    }
    const float inv = exp2f((float)-e);
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = to_e4m3(f[4 * i] * inv) | (to_e4m3(f[4 * i + 1] * inv) << 8) | (to_e4m3(f[4 * i + 2] * inv) << 16) |
               (to_e4m3(f[4 * i + 3] * inv) << 24);
    uint4* dst = reinterpret_cast<uint4*>(q + row * ldq + kb32 * 32);
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    const int r = (int)(row & 127);
    const size_t chunk = (size_t)(row >> 7) * nkb + (kb32 >> 2);
    sf[chunk * SF_BYTES + (r & 31) * 16 + (r >> 5) * 4 + (kb32 & 3)] = (uint8_t)(e + 127);
  }
}

}  // namespace

struct NpMxGemmArgs {
  const void* A; const void* B; void* C; const void* sfa; const void* sfb;
  long long lda, ldb, ldc, a_rows, b_rows;
  int M, N, K, out_f32, mode;
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;
  int max_ctas;
};

// C = A (e4m3, K-major, 1x32 e8m0 scales) times B^T (same). K and N multiples of 128, B rows (and the group stride)
// multiples of 128, lda / ldb multiples of 16 bytes. Returns 0 or a set-up / launch error.
NP_API int np_gemm_mxfp8(const NpMxGemmArgs* args, void* stream) {
  const NpMxGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0) return 0;
  if (a.K % 128 || a.N % 8 || a.b_rows % 128 || (a.lda % 16) || (a.ldb % 16) || (((uintptr_t)a.A) & 15) || (((uintptr_t)a.B) & 15) ||
      (((uintptr_t)a.sfa) & 15) || (((uintptr_t)a.sfb) & 15) || (a.group_stride_b % 128))
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
  MxParams p{};
  p.C = a.C; p.sfa = (const uint8_t*)a.sfa; p.sfb = (const uint8_t*)a.sfb;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldc = a.ldc; p.out_f32 = a.out_f32;
  p.mode = a.mode; p.mblk_group = a.mblk_group; p.mblk_rows = a.mblk_rows; p.group_stride_b = a.group_stride_b;
  p.b_chunks = a.b_rows / 128;
  constexpr int SMEM = STAGES * (BM * BK + BN * BK + SF_SMEM) + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (long long)((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  const int cap = a.max_ctas > 0 ? a.max_ctas : sms;
  const int grid = (int)(tiles < cap ? tiles : cap);
  gemm_mxfp8_kernel<<<grid, 192, SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// bf16 [rows, K] (row stride ldx elements) -> e4m3 [rows, K] (row stride ldq bytes) + scale chunks. K a multiple of
// 128; the scale buffer holds ceil(rows / 128) * (K / 128) chunks of 512 bytes (the caller pre-fills it with 127,
// the exponent byte of 1.0, so rows past the end scale by one).
NP_API int np_mx_quant(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows, int K, void* stream) {
  if (rows <= 0) return 0;
  if (K % 128 || (ldx % 8) || (ldq % 16) || (((uintptr_t)x) & 15) || (((uintptr_t)q) & 15)) return 1;
  const long long total = (long long)rows * (K / 32);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  mx_quant_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                                                                 (uint8_t*)sf, rows, K);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}
