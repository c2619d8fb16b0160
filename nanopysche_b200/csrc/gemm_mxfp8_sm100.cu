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
  // expert-parallel form (same protocol as the bf16 kernel of gemm_sm100.cu): wait for the arrival flag of the rank
  // that pushed an M block before touching it; store output rows through a per-row destination table into peer
  // memory and release the destination's flag when all of its blocks are done
  const int* ready_flags; const int* mblk_flag; int epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  const long long* row_dst; void* const* peer_base;
  int* done_counters; const int* done_expected; int* const* done_flag_ptr;
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
  const int epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0);
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

  // rows of an M block (0: skip it); -1 when the wait for its source's arrival flag ran out (status recorded)
  auto tile_rows = [&](int m_blk, int role) -> int {
    if (p.mode != 1) return BM;
    if (p.ready_flags) {
      const int fi = p.mblk_flag ? p.mblk_flag[m_blk] : 0;
      if (!np::wait_flag_ge(p.ready_flags + fi, epoch, p.flag_limit_ns, KID_MX, 100 + role)) {
        *abort_flag = 1;
        return -1;
      }
    }
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
        const int trows = tile_rows(m_blk, 0);
        if (trows < 0) break;
        if (trows == 0) continue;
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
        const int trows = tile_rows(m_blk, 1);
        if (trows < 0) break;
        if (trows == 0) continue;
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
      const int rows = tile_rows(m_blk, 2);
      if (rows < 0) break;
      if (rows == 0) continue;
      if (!np::mbar_wait(afull_bar(acc), acc_phase, abort_flag, KID_MX, 4)) break;
      np::tc_fence_after();
      const int r_in = quarter * 32 + lane;
      const int row = m_blk * BM + r_in;
      bool row_ok = row < p.M && r_in < rows;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
      char* crow;
      if (p.row_dst) {   // destination row in some rank's buffer: (rank << 40) | row, -1 for a padding row
        const long long d = row_ok ? p.row_dst[row] : -1;
        row_ok = row_ok && d >= 0;
        const long long peer = row_ok ? (d >> 40) : 0;
        crow = (char*)p.peer_base[peer] + (size_t)(d & ((1ll << 40) - 1)) * p.ldc * (p.out_f32 ? 4 : 2);
      } else {
        crow = (char*)p.C + (size_t)row * p.ldc * (p.out_f32 ? 4 : 2);
      }
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
      if (p.done_counters) {   // this warp's rows of the tile are stored: count it towards the source's flag
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


// ------------------------------------------------------------------------------- 128-wide power-of-two blocks
// The FP8-Flow-MoE recipe scales activations per 1x128 block and weights per 128x128 block. With the scale
// restricted to a power of two (UE8M0, the form DeepSeek's own Blackwell kernels use) such a block is four
// consecutive 1x32 hardware blocks that carry the same exponent byte, so the block-scaled MMA above applies the
// recipe's scaling inside the tensor core and nothing is promoted in registers. The quantisers below write the
// e4m3 values and the exponent bytes straight into the chunk layout (four equal bytes per row and 128-wide block).
__device__ __forceinline__ int pow2_exp(float am) {   // ceil(log2(am / 448)), clamped; zero block -> smallest scale
  if (!(am > 0.f)) return -127;
  int ex;
  const float mant = frexpf(__fdiv_rn(am, 448.f), &ex);
  const int e = (mant == 0.5f) ? ex - 1 : ex;
  return max(-127, min(127, e));
}
__device__ __forceinline__ void sf_store_x4(uint8_t* sf, long long row, int kb, int nkb, int e) {
  const int r = (int)(row & 127);
  *reinterpret_cast<uint32_t*>(sf + ((size_t)(row >> 7) * nkb + kb) * SF_BYTES + (r & 31) * 16 + (r >> 5) * 4) =
      (uint32_t)(e + 127) * 0x01010101u;
}
__device__ __forceinline__ uint2 pack_e4m3x8(const float* f, float inv) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= to_e4m3(f[j] * inv) << (8 * j);
    hi |= to_e4m3(f[4 + j] * inv) << (8 * j);
  }
  return make_uint2(lo, hi);
}
__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = np::unpack_bf16(u.x), b = np::unpack_bf16(u.y), c = np::unpack_bf16(u.z), d = np::unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// 1x128 blocks: half a warp (16 lanes x 8 elements) per block. `swiglu`: the input row is [gate(K) | up(K)] and the
// quantised value is silu(gate) * up (the expert MLP's hidden activation), else the input itself.
__global__ void __launch_bounds__(256) flow_quant_act_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                             uint8_t* __restrict__ q, long long ldq,
                                                             uint8_t* __restrict__ sf, int rows, int K, int swiglu,
                                                             __nv_bfloat16* __restrict__ h_out, long long ldh) {
  const int nkb = K >> 7;
  const long long total = (long long)rows * nkb;
  const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
  const long long warp_g = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long b0 = warp_g * 2; b0 < total; b0 += nwarps * 2) {
    const long long b = b0 + half;
    const bool valid = b < total;
    const long long row = valid ? b / nkb : 0;
    const int kb = valid ? (int)(b - row * nkb) : 0;
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (valid) {
      const __nv_bfloat16* src = x + row * ldx + kb * 128 + l16 * 8;
      load8_bf16(src, f);
      if (swiglu) {
        float u[8];
        load8_bf16(src + K, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = np::silu_f(f[j]) * u[j];
        if (h_out)   // the unquantised activation too (the weight gradient of the down projection wants it)
          *reinterpret_cast<uint4*>(h_out + row * ldh + kb * 128 + l16 * 8) =
              make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]), np::pack_bf16(f[4], f[5]),
                         np::pack_bf16(f[6], f[7]));
      }
    }
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[j]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (!valid) continue;
    const int e = pow2_exp(am);
    *reinterpret_cast<uint2*>(q + row * ldq + kb * 128 + l16 * 8) = pack_e4m3x8(f, exp2f((float)-e));
    if (l16 == 0) sf_store_x4(sf, row, kb, nkb, e);
  }
}

// e4m3 + chunked exponent bytes -> bf16 (16 elements per thread).
__global__ void __launch_bounds__(256) mx_dequant_kernel(const uint8_t* __restrict__ q, long long ldq,
                                                         const uint8_t* __restrict__ sf, __nv_bfloat16* __restrict__ out,
                                                         long long ldo, int rows, int K) {
  const int vpr = K >> 4, nkb = K >> 7;
  const long long total = (long long)rows * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vpr;
    const int c16 = (int)(i - row * vpr);
    const int kb32 = c16 >> 1, r = (int)(row & 127);
    const uint8_t sb = sf[((size_t)(row >> 7) * nkb + (kb32 >> 2)) * SF_BYTES + (r & 31) * 16 + (r >> 5) * 4 + (kb32 & 3)];
    const float sc = exp2f((float)((int)sb - 127));
    const uint4 u = *reinterpret_cast<const uint4*>(q + row * ldq + c16 * 16);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)((w[j] >> (8 * k)) & 0xffu), __NV_E4M3);
        v[k] = __half2float(*reinterpret_cast<const __half*>(&hr)) * sc;
      }
      o[2 * j] = np::pack_bf16(v[0], v[1]);
      o[2 * j + 1] = np::pack_bf16(v[2], v[3]);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + row * ldo + c16 * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// 128x128 weight blocks, one CTA per block. Input: E experts of [R, C] bf16 stacked along the rows. Output (e4m3):
// the same shape, or with `trans` every expert transposed to [C, R] (the layout a GEMM that contracts over R needs);
// exponent bytes in the chunk layout of the OUTPUT matrix (contraction = its columns). Without `trans` expert e's rows
// land at output rows e * o_rows + o_row0 (o_rows >= R), which lets two weights share one output matrix
// ([gate; up] per expert for a single gate|up GEMM).
__global__ void __launch_bounds__(256) flow_quant_weight_kernel(const __nv_bfloat16* __restrict__ w,
                                                                uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                int E, int R, int C, int trans, int o_rows, int o_row0) {
  __shared__ float s_red[8];
  __shared__ __align__(16) uint8_t s_t[128][128 + 16];
  const int rb = R >> 7, cb = C >> 7;
  const int blk = blockIdx.x;
  const int e = blk / (rb * cb), bi = (blk / cb) % rb, bj = blk % cb;
  const int tid = threadIdx.x, r0 = tid >> 4, c8 = tid & 15;
  const __nv_bfloat16* src = w + ((size_t)e * R + (size_t)bi * 128) * C + (size_t)bj * 128;
  float f[8][8];
  float am = 0.f;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    load8_bf16(src + (size_t)(it * 16 + r0) * C + c8 * 8, f[it]);
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[it][j]));
  }
  am = np::warp_max(am);
  if ((tid & 31) == 0) s_red[tid >> 5] = am;
  __syncthreads();
  am = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) am = fmaxf(am, s_red[i]);
  const int ex = pow2_exp(am);
  const float inv = exp2f((float)-ex);
  if (!trans) {
    const size_t orow = (size_t)e * o_rows + o_row0 + (size_t)bi * 128;
    uint8_t* dst = q + orow * C + (size_t)bj * 128;
#pragma unroll
    for (int it = 0; it < 8; ++it)
      *reinterpret_cast<uint2*>(dst + (size_t)(it * 16 + r0) * C + c8 * 8) = pack_e4m3x8(f[it], inv);
    uint32_t* chunk = reinterpret_cast<uint32_t*>(sf + ((orow >> 7) * cb + bj) * SF_BYTES);
    if (tid < SF_BYTES / 4) chunk[tid] = (uint32_t)(ex + 127) * 0x01010101u;
  } else {
    // e4m3 tile row-major into shared memory (8-byte stores), then every thread gathers 64 bytes of one output row
    // (= one input column): a warp reads 32 consecutive bytes per step, which is conflict-free
#pragma unroll
    for (int it = 0; it < 8; ++it)
      *reinterpret_cast<uint2*>(&s_t[it * 16 + r0][c8 * 8]) = pack_e4m3x8(f[it], inv);
    __syncthreads();
    const int oc = tid & 127, hf = tid >> 7;
    uint8_t* dst = q + ((size_t)e * C + (size_t)bj * 128 + oc) * R + (size_t)bi * 128 + hf * 64;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t wv[4] = {0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < 16; ++k) wv[k >> 2] |= (uint32_t)s_t[hf * 64 + g * 16 + k][oc] << (8 * (k & 3));
      *reinterpret_cast<uint4*>(dst + g * 16) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    }
    uint32_t* chunk = reinterpret_cast<uint32_t*>(sf + ((size_t)(e * cb + bj) * rb + bi) * SF_BYTES);
    if (tid < SF_BYTES / 4) chunk[tid] = (uint32_t)(ex + 127) * 0x01010101u;
  }
}

}  // namespace

struct NpMxGemmArgs {
  const void* A; const void* B; void* C; const void* sfa; const void* sfb;
  long long lda, ldb, ldc, a_rows, b_rows;
  int M, N, K, out_f32, mode;
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;
  int max_ctas;
  const int* ready_flags; const int* mblk_flag; int epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  const long long* row_dst; void* const* peer_base;
  int* done_counters; const int* done_expected; int* const* done_flag_ptr;
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
  p.ready_flags = a.ready_flags; p.mblk_flag = a.mblk_flag; p.epoch = a.epoch; p.epoch_base = a.epoch_base;
  p.flag_limit_ns = a.flag_limit_ns ? a.flag_limit_ns : NP_WAIT_LIMIT_NS;
  p.row_dst = a.row_dst; p.peer_base = a.peer_base;
  p.done_counters = a.done_counters; p.done_expected = a.done_expected; p.done_flag_ptr = a.done_flag_ptr;
  constexpr int SMEM = STAGES * (BM * BK + BN * BK + SF_SMEM) + 1024 + 256;
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
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

// bf16 [rows, K] (or, with `swiglu`, [rows, 2K] = [gate | up] quantising silu(gate) * up) -> e4m3 [rows, K] with one
// power-of-two scale per 1x128 block, exponent bytes in the chunk layout. K a multiple of 128. With `swiglu`, `h_out`
// (optional, row stride ldh elements) also receives silu(gate) * up in bf16.
NP_API int np_flow_quant_act(const void* x, long long ldx, void* q, long long ldq, void* sf, int rows, int K,
                             int swiglu, void* h_out, long long ldh, void* stream) {
  if (rows <= 0) return 0;
  if (K % 128 || (ldx % 8) || (ldq % 8) || (((uintptr_t)x) & 15) || (((uintptr_t)q) & 7) || (((uintptr_t)sf) & 3)) return 1;
  const long long total = (long long)rows * (K / 128);
  long long blocks = (total + 15) / 16;   // 8 warps x 2 blocks per CTA iteration
  if (blocks > 148 * 128) blocks = 148 * 128;
  flow_quant_act_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                                                                        (uint8_t*)sf, rows, K, swiglu,
                                                                        (__nv_bfloat16*)h_out, ldh);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

NP_API int np_mx_dequant(const void* q, long long ldq, const void* sf, void* out, long long ldo, int rows, int K,
                         void* stream) {
  if (rows <= 0) return 0;
  if (K % 128 || (ldq % 16) || (ldo % 8) || (((uintptr_t)q) & 15) || (((uintptr_t)out) & 15)) return 1;
  const long long total = (long long)rows * (K / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  mx_dequant_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, ldq, (const uint8_t*)sf,
                                                                    (__nv_bfloat16*)out, ldo, rows, K);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// E stacked [R, C] bf16 matrices -> e4m3 with one power-of-two scale per 128x128 block (optionally every matrix
// transposed to [C, R]). R and C multiples of 128.
NP_API int np_flow_quant_weight(const void* w, void* q, void* sf, int E, int R, int C, int trans, int o_rows,
                                int o_row0, void* stream) {
  if (E <= 0) return 0;
  if (o_rows <= 0) o_rows = R;
  if (trans && (o_rows != R || o_row0 != 0)) return 1;
  if (R % 128 || C % 128 || o_rows % 128 || o_row0 % 128 || o_row0 + R > o_rows || (((uintptr_t)w) & 15) || (((uintptr_t)q) & 15) || (((uintptr_t)sf) & 15)) return 1;
  const long long blocks = (long long)E * (R / 128) * (C / 128);
  flow_quant_weight_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q,
                                                                           (uint8_t*)sf, E, R, C, trans, o_rows, o_row0);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}
