// bf16 GEMM family for sm_100a: persistent, warp-specialised, tcgen05.mma with the accumulator
// in TMEM (double buffered), operands staged by TMA into 128-byte-swizzled shared memory.
//
// One kernel covers forward (A,B K-major), dgrad (B MN-major) and wgrad (A,B MN-major), the
// ragged per-expert ("grouped") variants used by the MoE layers, a fused SwiGLU epilogue, and
// the two hooks that fuse a collective into the GEMM: a per-M-block arrival-flag wait in front
// of the loads (tokens pushed into this GPU's buffer by its peers) and an epilogue that stores
// output rows through a per-row destination table into peer memory and signals the peers.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> global). All waits are bounded (common.cuh).
//
// Replaces the cuBLAS calls behind nn.Linear / torch.bmm in the reference
// (model/attention.py:141-143,189; model/feed_forward.py:75; model/moe.py:1520-1538).
#include <cstdlib>
#include "common.cuh"

__device__ int g_np_status[8];
__device__ unsigned long long g_np_wait_end[NP_MAX_SMS];
__device__ unsigned long long g_np_wait_ns[NP_MAX_SMS];

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 B = one swizzle row
constexpr int KID_GEMM = 1;

struct GemmParams {
  void* C;            // output
  void* C2;           // swiglu: optional [gate | up] pre-activation output, (M, 2*N_out)
  int M, N, K;        // output rows / cols, contraction length
  long long ldc, ldc2;
  int a_mn, b_mn;     // 0: operand is K-major ([rows, K]); 1: MN-major ([K, rows])
  int out_f32;        // 0: bf16 output, 1: fp32 output
  int accumulate;     // C += A*B (read-modify-write)
  int epilogue;       // 0 plain, 1 swiglu (B tile = 128 gate rows + 128 up rows)
  int mode;           // 0 dense, 1 grouped rows (per-M-block B offset), 2 grouped K (wgrad)
  float alpha;
  const int* mblk_group;      // [m blocks] group of each 128-row block (mode 1) or nullptr
  const int* mblk_rows;       // [m blocks] valid rows of each block, 0 = skip; nullptr = all
  long long group_stride_b;   // rows of B per group (mode 1)
  int num_groups;             // mode 2
  int blocks_per_group;       // mode 2: 128-row blocks of the token axis per group
  long long group_stride_c;   // mode 2: elements of C per group
  const int* ready_flags;     // arrival flags (monotone epochs) or nullptr
  const int* mblk_flag;       // [m blocks] index into ready_flags
  int epoch;
  unsigned long long flag_limit_ns;
  const long long* row_dst;   // per output row: (peer << 40) | row, or < 0 to drop; nullptr = dense
  void* const* peer_base;     // [peers] base pointer of each peer's destination buffer
  int* done_counters;         // [flags] tiles finished per destination (local)
  const int* done_expected;   // [flags] M blocks expected per destination (x n_blocks tiles each)
  int* const* done_flag_ptr;  // [flags] peer flag word to release when a destination completes
  const void* Cin;            // accumulate source (same dtype as C), rows indexed like a dense C
  long long ldcin;
  const int* epoch_base;      // optional device counter added to `epoch` (keeps epochs valid under graph replay)
  const int* b_ready_flags;   // arrival flags of the B operand: flag i covers B rows [i * b_rows_per_flag, ...)
  int b_rows_per_flag;
  // Rows of A (K-major) / B (K-major) that this GPU produced itself are read from their source tensor through a
  // second tensor map, so nothing in this kernel waits for a copy made by another kernel of the same GPU.
  int a_loc_lo, a_loc_hi;     // A rows [lo, hi) come from tmAloc (row index - lo)
  int b_loc_lo, b_loc_hi;     // B rows [lo, hi) come from tmBloc
  int b_local_flag;           // index into b_ready_flags that needs no wait (the local shard), -1: none
  int m_rot, n_rot;           // tile order starts at this M / N block (the local shard first)
  // All-gather issued by this kernel itself: before the first tile every CTA stores its slice of `push_src` into
  // the peers' gather buffers; the CTA that finishes last releases this rank's arrival flag on every peer. The
  // grid is one resident wave, so the push never waits for a CTA that has not started.
  const uint4* push_src; long long push_vecs;
  uint4* push_dst[8]; int* push_flag[8]; int push_n;
  int* push_ctr;
  bool st32;                  // output rows and column chunks are 32-byte aligned: use 32-byte stores
  const float* bias;          // optional [N] fp32 added to every output row (plain epilogue)
};

// 64 bytes (32 bf16 packed in 16 registers) to a row: two 32-byte stores when the address allows it (a full sector
// per request - what a row pushed to a peer over NVLink is made of), else four 16-byte stores.
__device__ __forceinline__ void store64(void* dst, const uint32_t* o, bool st32) {
  if (st32) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                 "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"((char*)dst + 32), "r"(o[8]), "r"(o[9]),
                 "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15])
                 : "memory");
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
  }
}

template <class F>
__device__ __forceinline__ void for_each_k(const GemmParams& p, int g, F&& f) {
  if (p.mode != 2) {
    const int nkb = (p.K + BK - 1) / BK;
    for (int kb = 0; kb < nkb; ++kb) {
      if (!f(kb * BK)) return;
    }
  } else {
    const int b0 = g * p.blocks_per_group;
    for (int b = b0; b < b0 + p.blocks_per_group; ++b) {
      const int r = p.mblk_rows ? p.mblk_rows[b] : BM;
      if (r <= 0) continue;
      if (!f(b * BM)) return;
      if (!f(b * BM + BK)) return;
    }
  }
}

__device__ __forceinline__ int count_k(const GemmParams& p, int g) {
  if (p.mode != 2) return (p.K + BK - 1) / BK;
  int n = 0;
  const int b0 = g * p.blocks_per_group;
  for (int b = b0; b < b0 + p.blocks_per_group; ++b) {
    const int r = p.mblk_rows ? p.mblk_rows[b] : BM;
    if (r > 0) n += 2;
  }
  return n;
}

struct Tile {
  int g, m_blk, n_blk;
};

// MT = 1: one 128 x BN accumulator per tile, double-buffered in tensor memory (the epilogue of a tile runs under the
// MMAs of the next). MT = 2: a 256 x BN tile as two 128-row halves that share every B tile; per FLOP a third fewer
// operand bytes cross from L2 into shared memory, which is what bounds the 128 x 256 tile (the L2 -> SM fabric
// delivers about 16 TB/s, the 128 x 256 tile asks for 11.4 bytes per kFLOP). The two accumulators fill all 512
// tensor-memory columns, so they are single-buffered: MMA issue pauses while a tile drains.
template <int BN, int STAGES, int MT>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmAloc,
                 const __grid_constant__ CUtensorMap tmBloc, const GemmParams p) {
  constexpr int TM = BM * MT;                 // rows of a tile
  constexpr int A_HALF = BM * BK * 2;         // one 128-row half of the A tile
  constexpr int A_BYTES = TM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int NACC = MT == 1 ? 2 : 1;       // accumulator buffers in tensor memory
  static_assert(MT * BN * NACC <= 512, "tensor memory holds 512 columns");
  constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (np::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint8_t* tail = smem_raw + (bar_base - np::smem_u32(smem_raw)) + 8 * (2 * STAGES + 4);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0);

  const int m_blocks = (p.M + TM - 1) / TM;
  const int bn_out = (p.epilogue == 1) ? BN / 2 : BN;  // output columns per tile
  const int n_blocks = (p.N + bn_out - 1) / bn_out;
  const int groups = (p.mode == 2) ? p.num_groups : 1;
  const int tiles_per_group = m_blocks * n_blocks;
  const int num_tiles = tiles_per_group * groups;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      np::mbar_init(full_bar(s), 1);
      np::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      np::mbar_init(tfull_bar(a), 1);
      np::mbar_init(tempty_bar(a), 4);
    }
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

  if (p.push_src) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.push_vecs;
         i += (long long)gridDim.x * blockDim.x) {
      const uint4 v = p.push_src[i];
      for (int r = 0; r < p.push_n; ++r) p.push_dst[r][i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(p.push_ctr, 1) == (int)gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < p.push_n; ++r) np::st_release_sys(p.push_flag[r], epoch);
      *p.push_ctr = 0;
    }
  }

  auto decode = [&](int t) {
    Tile tl;
    tl.g = t / tiles_per_group;
    const int r = t - tl.g * tiles_per_group;
    // bands of 16 M blocks: one wave of CTAs touches ~16 A row-blocks and ~9 B row-blocks instead of all
    // of A, so both operands are re-read from L2 rather than from DRAM
    constexpr int BAND = 16;
    const int per_band = BAND * n_blocks;
    const int band = r / per_band;
    const int first_m = band * BAND;
    const int gsize = (m_blocks - first_m) < BAND ? (m_blocks - first_m) : BAND;
    const int within = r - band * per_band;
    tl.m_blk = first_m + within % gsize;
    tl.n_blk = within / gsize;
    if (p.m_rot) tl.m_blk = (tl.m_blk + p.m_rot) % m_blocks;
    if (p.n_rot) tl.n_blk = (tl.n_blk + p.n_rot) % n_blocks;
    return tl;
  };
  // rows of this M block that carry data (0 = nothing to do); waits for the arrival flag first.
  auto tile_rows = [&](const Tile& tl, int role) -> int {
    if (p.mode != 1 || MT != 1) return TM;   // the row-grouped form (per-128-row-block tables) runs with MT = 1
    if (p.ready_flags) {
      const int fi = p.mblk_flag ? p.mblk_flag[tl.m_blk] : 0;
      if (fi >= 0 && !np::wait_flag_ge(p.ready_flags + fi, epoch, p.flag_limit_ns, KID_GEMM, 100 + role)) {
        *abort_flag = 1;
        return -1;
      }
    }
    return p.mblk_rows ? p.mblk_rows[tl.m_blk] : BM;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const Tile tl = decode(t);
        const int rows = tile_rows(tl, 0);
        if (rows < 0) break;
        if (rows == 0) continue;
        const int m0 = tl.m_blk * TM;
        const int n0 = tl.n_blk * bn_out;
        long long goff = 0;  // row offset of this tile's group inside the stacked B tensor
        if (p.mode == 1 && p.mblk_group) goff = (long long)p.mblk_group[tl.m_blk] * p.group_stride_b;
        const long long brow = n0 + (p.b_mn ? 0 : goff);
        const int bk_off = p.b_mn ? (int)goff : 0;
        int b_flag_hi = -1;   // highest B shard this tile has already waited for (its row ranges only move up)
        auto wait_b_rows = [&](long long r0, long long r1) -> bool {   // rows [r0, r1] of B are about to be loaded
          if (!p.b_ready_flags) return true;
          const int f0 = (int)(r0 / p.b_rows_per_flag), f1 = (int)(r1 / p.b_rows_per_flag);
          for (int f = f0 > b_flag_hi ? f0 : b_flag_hi + 1; f <= f1; ++f)
            if (f != p.b_local_flag && !np::wait_flag_ge(p.b_ready_flags + f, epoch, p.flag_limit_ns, KID_GEMM, 110)) {
              *abort_flag = 1;
              return false;
            }
          if (f1 > b_flag_hi) b_flag_hi = f1;
          return true;
        };
        if (!p.b_mn) {
          const long long last = brow + bn_out - 1 < p.N + goff - 1 ? brow + bn_out - 1 : p.N + goff - 1;
          if (!wait_b_rows(brow, last)) break;
        }
        for_each_k(p, tl.g, [&](int k0) -> bool {
          if (p.b_mn && p.b_ready_flags) {
            const long long last = k0 + bk_off + BK - 1 < p.K + bk_off - 1 ? k0 + bk_off + BK - 1 : p.K + bk_off - 1;
            if (!wait_b_rows(k0 + bk_off, last)) return false;
          }
          if (!np::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, KID_GEMM, 1)) return false;
          const uint32_t sA = smem_base + stage * STAGE_BYTES;
          const uint32_t sB = sA + A_BYTES;
          np::mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (!p.a_mn) {
            if (MT == 1 && m0 >= p.a_loc_lo && m0 < p.a_loc_hi) {
              np::tma_load_2d(sA, &tmAloc, full_bar(stage), k0, m0 - p.a_loc_lo);
            } else {
#pragma unroll
              for (int h = 0; h < MT; ++h) np::tma_load_2d(sA + h * A_HALF, &tmA, full_bar(stage), k0, m0 + h * BM);
            }
          } else {
#pragma unroll
            for (int c = 0; c < TM / 64; ++c)
              np::tma_load_2d(sA + c * (64 * BK * 2), &tmA, full_bar(stage), m0 + c * 64, k0);
          }
          if (!p.b_mn) {
            if (p.epilogue == 1) {
              np::tma_load_2d(sB, &tmB, full_bar(stage), k0, (int)brow);
              np::tma_load_2d(sB + (BN / 2) * BK * 2, &tmB2, full_bar(stage), k0, (int)brow);
            } else if (brow >= p.b_loc_lo && brow < p.b_loc_hi) {
              np::tma_load_2d(sB, &tmBloc, full_bar(stage), k0, (int)brow - p.b_loc_lo);
            } else {
              np::tma_load_2d(sB, &tmB, full_bar(stage), k0, (int)brow);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              np::tma_load_2d(sB + c * (64 * BK * 2), &tmB, full_bar(stage), (int)brow + c * 64, k0 + bk_off);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          return true;
        });
      }
      if (*abort_flag) __nanosleep(1000000);  // let copies already issued land before exit
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = np::make_idesc(BM, BN, 1, 1, p.a_mn, p.b_mn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        const Tile tl = decode(t);
        const int rows = tile_rows(tl, 1);
        if (rows < 0) break;
        if (rows == 0) continue;
        if (count_k(p, tl.g) == 0) continue;
        if (!np::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, KID_GEMM, 2)) break;
        np::tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * MT * BN);
        uint32_t accum = 0;
        for_each_k(p, tl.g, [&](int) -> bool {
          if (!np::mbar_wait(full_bar(stage), phase, abort_flag, KID_GEMM, 3)) return false;
          np::tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES;
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t bd = p.b_mn ? np::make_smem_desc(sB + kk * 2048, 64 * BK * 2, 1024)
                                       : np::make_smem_desc(sB + kk * 32, 16, 1024);
#pragma unroll
            for (int h = 0; h < MT; ++h) {   // both halves read the same B tile
              const uint32_t sAh = sA + h * A_HALF;
              const uint64_t ad = p.a_mn ? np::make_smem_desc(sAh + kk * 2048, 64 * BK * 2, 1024)
                                         : np::make_smem_desc(sAh + kk * 32, 16, 1024);
              np::tc_mma_f16(tmem_d + (uint32_t)(h * BN), ad, bd, idesc, accum);
            }
            accum = 1;
          }
          np::tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          return true;
        });
        np::tc_commit(tfull_bar(acc));
        if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
      }
      if (*abort_flag) __nanosleep(1000000);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      const Tile tl = decode(t);
      const int rows = tile_rows(tl, 2);
      if (rows < 0) break;
      if (rows == 0) continue;
      const int nk = count_k(p, tl.g);
      const int n0 = tl.n_blk * bn_out;
      bool have_acc = nk > 0;
      if (have_acc) {
        if (!np::mbar_wait(tfull_bar(acc), acc_phase, abort_flag, KID_GEMM, 4)) break;
        np::tc_fence_after();
      }
#pragma unroll 1
      for (int h = 0; h < MT; ++h) {   // the 128-row halves of the tile, one accumulator each
      const int row = tl.m_blk * TM + h * BM + quarter * 32 + lane;
      bool row_ok = row < p.M;
      char* crow;
      if (p.row_dst) {
        const long long d = row_ok ? p.row_dst[row] : -1;
        row_ok = row_ok && d >= 0;
        const long long peer = row_ok ? (d >> 40) : 0;
        const long long drow = d & ((1ll << 40) - 1);
        crow = (char*)p.peer_base[peer] + (size_t)drow * p.ldc * (p.out_f32 ? 4 : 2);
      } else {
        crow = (char*)p.C + ((size_t)tl.g * p.group_stride_c + (size_t)row * p.ldc) * (p.out_f32 ? 4 : 2);
      }
      const char* cin_row = p.Cin ? (const char*)p.Cin + ((size_t)tl.g * p.group_stride_c + (size_t)row * p.ldcin) * (p.out_f32 ? 4 : 2)
                                  : nullptr;
      const uint32_t taddr = tmem_base + (uint32_t)((acc * MT + h) * BN) + ((uint32_t)(quarter * 32) << 16);
      if (p.epilogue == 1) {
        // gate = columns [0, BN/2), up = columns [BN/2, BN); out = silu(gate) * up
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          np::tmem_ld32(taddr + c * 32, g);
          np::tmem_ld32(taddr + BN / 2 + c * 32, u);
          np::tmem_ld_wait();
          const int col = n0 + c * 32;
          if (row_ok && col < p.N) {
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
              const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
              o[i] = np::pack_bf16(np::silu_f(g0) * u0, np::silu_f(g1) * u1);
            }
            __nv_bfloat16* dst = (__nv_bfloat16*)crow + col;
            if (col + 32 <= p.N) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col + i < p.N)
                dst[i] = reinterpret_cast<__nv_bfloat16*>(o)[i];
            }
            if (p.C2) {
              __nv_bfloat16* d2 = (__nv_bfloat16*)p.C2 + (size_t)row * p.ldc2 + col;
              if (col + 32 <= p.N) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  reinterpret_cast<uint4*>(d2)[i] =
                      make_uint4(np::pack_bf16(__uint_as_float(g[8 * i]), __uint_as_float(g[8 * i + 1])),
                                 np::pack_bf16(__uint_as_float(g[8 * i + 2]), __uint_as_float(g[8 * i + 3])),
                                 np::pack_bf16(__uint_as_float(g[8 * i + 4]), __uint_as_float(g[8 * i + 5])),
                                 np::pack_bf16(__uint_as_float(g[8 * i + 6]), __uint_as_float(g[8 * i + 7])));
                  reinterpret_cast<uint4*>(d2 + p.N)[i] =
                      make_uint4(np::pack_bf16(__uint_as_float(u[8 * i]), __uint_as_float(u[8 * i + 1])),
                                 np::pack_bf16(__uint_as_float(u[8 * i + 2]), __uint_as_float(u[8 * i + 3])),
                                 np::pack_bf16(__uint_as_float(u[8 * i + 4]), __uint_as_float(u[8 * i + 5])),
                                 np::pack_bf16(__uint_as_float(u[8 * i + 6]), __uint_as_float(u[8 * i + 7])));
                }
              } else {
                _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col + i < p.N) {
                  d2[i] = __float2bfloat16(__uint_as_float(g[i]));
                  d2[p.N + i] = __float2bfloat16(__uint_as_float(u[i]));
                }
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (have_acc) {
            np::tmem_ld32(taddr + c * 32, r);
            np::tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          const bool full = col + 32 <= p.N;
          if (p.bias) {  // the same 32 values for every row of the warp: broadcast loads
            const float inv_alpha = 1.f / p.alpha;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float b = (col + i < p.N) ? __ldg(p.bias + col + i) : 0.f;
              r[i] = __float_as_uint(fmaf(b, inv_alpha, __uint_as_float(r[i])));
            }
          }
          if (p.out_f32) {
            float* dst = (float*)crow + col;
            if (full) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 v = make_float4(__uint_as_float(r[4 * i]) * p.alpha, __uint_as_float(r[4 * i + 1]) * p.alpha,
                                       __uint_as_float(r[4 * i + 2]) * p.alpha, __uint_as_float(r[4 * i + 3]) * p.alpha);
                if (cin_row) {
                  const float4 o = reinterpret_cast<const float4*>((const float*)cin_row + col)[i];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(dst)[i] = v;
              }
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col + i < p.N) {
                float v = __uint_as_float(r[i]) * p.alpha;
                if (cin_row) v += ((const float*)cin_row + col)[i];
                dst[i] = v;
              }
            }
          } else {
            __nv_bfloat16* dst = (__nv_bfloat16*)crow + col;
            if (full) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * i + j]) * p.alpha;
                if (cin_row) {
                  const uint4 o = reinterpret_cast<const uint4*>((const __nv_bfloat16*)cin_row + col)[i];
                  const float2 o0 = np::unpack_bf16(o.x), o1 = np::unpack_bf16(o.y), o2 = np::unpack_bf16(o.z), o3 = np::unpack_bf16(o.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                pk[4 * i] = np::pack_bf16(f[0], f[1]); pk[4 * i + 1] = np::pack_bf16(f[2], f[3]);
                pk[4 * i + 2] = np::pack_bf16(f[4], f[5]); pk[4 * i + 3] = np::pack_bf16(f[6], f[7]);
              }
              store64(dst, pk, p.st32);
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col + i < p.N) {
                float v = __uint_as_float(r[i]) * p.alpha;
                if (cin_row) v += __bfloat162float(((const __nv_bfloat16*)cin_row + col)[i]);
                dst[i] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      }   // halves
      if (have_acc) {
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(tempty_bar(acc));
        if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
      }
      if (p.done_counters) {
        // all rows of this tile are stored (possibly into peer memory): publish, then count the
        // tile against its destination and release the peer's flag when the destination is done.
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          // each of the four epilogue warps counts once per tile: expected is in tiles
          const int fi = p.mblk_flag ? p.mblk_flag[tl.m_blk] : 0;
          const int done = atomicAdd(&p.done_counters[fi], 1) + 1;
          if (done == 4 * n_blocks * p.done_expected[fi]) {  // done_expected counts M blocks
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

int g_num_sms = 0;

}  // namespace

// ------------------------------------------------------------------ host side
static NpEncodeTiledFn g_encode = nullptr;
NpEncodeTiledFn np_get_encode_tiled() {
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = (NpEncodeTiledFn)fn;
  return g_encode;
}

int np_make_tmap_2d(CUtensorMap* out, const void* base, int elt_bytes, uint64_t rows, uint64_t cols,
                    uint64_t ld, uint32_t box_cols, uint32_t box_rows) {
  NpEncodeTiledFn enc = np_get_encode_tiled();
  if (!enc) return -1;
  CUtensorMapDataType dt = elt_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                          : (elt_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elt_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Arguments of np_gemm_bf16 (mirrored field by field by the ctypes Structure in ops/_lib.py).
struct NpGemmArgs {
  const void* A; const void* B; const void* B2; void* C; void* C2;
  long long lda, ldb, ldc, ldc2;
  long long a_rows, b_rows;  // total rows (K-major) or total K rows (MN-major) of the A / B tensors
  int M, N, K;
  int a_mn, b_mn, out_f32, accumulate, epilogue, mode;
  float alpha;
  const int* mblk_group; const int* mblk_rows; long long group_stride_b;
  int num_groups, blocks_per_group; long long group_stride_c;
  const int* ready_flags; const int* mblk_flag; int epoch; unsigned long long flag_limit_ns;
  const long long* row_dst; void* const* peer_base;
  int* done_counters; const int* done_expected; int* const* done_flag_ptr;
  int bn;        // 0 = choose, else 128 or 256
  int max_ctas;  // 0 = all SMs
  const void* Cin; long long ldcin;  // optional accumulate source (defaults to C when accumulate != 0)
  const int* epoch_base;             // optional device counter added to `epoch`
  // B arriving in row shards (a sharded weight being all-gathered while the GEMM runs): the producer waits for
  // the flag of every shard a tile touches before it loads from it
  const int* b_ready_flags; int b_rows_per_flag;
  // Local shard read in place (K-major operands only): A rows [a_loc_lo, a_loc_hi) from A_loc (row 0 = a_loc_lo),
  // B rows [b_loc_lo, b_loc_hi) from B_loc; the block boundaries must be multiples of the tile size. b_local_flag:
  // 1 + index of the B flag that needs no wait (0: none). m_rot / n_rot: first M / N block of the tile order.
  const void* A_loc; long long lda_loc; int a_loc_lo, a_loc_hi;
  const void* B_loc; long long ldb_loc; int b_loc_lo, b_loc_hi;
  int b_local_flag, m_rot, n_rot;
  // all-gather pushed by the GEMM's own CTAs before their first tile: push_bytes of push_src to push_dst[r]
  // (r < push_n <= 8; the destinations already point at this rank's slot), then *push_flag[r] = epoch (+ base);
  // push_ctr: a zeroed local int
  const void* push_src; long long push_bytes; void* const* push_dst; int* const* push_flag; int push_n; int* push_ctr;
  const float* bias;  // optional [N] fp32 bias added in the plain epilogue (alpha != 0)
  int mt;             // rows of a tile in units of 128: 0 = choose, 1, or 2 (256 x 256 tiles, dense and K-grouped forms)
};

template <int BN, int STAGES, int MT>
static int launch_gemm(const NpGemmArgs& a, cudaStream_t stream) {
  constexpr int TM = BM * MT;
  CUtensorMap tmA, tmB, tmB2, tmAloc, tmBloc;
  int rc;
  if (!a.a_mn) rc = np_make_tmap_2d(&tmA, a.A, 2, (uint64_t)a.a_rows, (uint64_t)a.K, (uint64_t)a.lda, BK, BM);
  else rc = np_make_tmap_2d(&tmA, a.A, 2, (uint64_t)a.a_rows, (uint64_t)a.M, (uint64_t)a.lda, 64, BK);
  if (rc) return 100 + rc;
  const uint32_t b_box_rows = a.epilogue == 1 ? BN / 2 : BN;
  if (!a.b_mn) rc = np_make_tmap_2d(&tmB, a.B, 2, (uint64_t)a.b_rows, (uint64_t)a.K, (uint64_t)a.ldb, BK, b_box_rows);
  else rc = np_make_tmap_2d(&tmB, a.B, 2, (uint64_t)a.b_rows, (uint64_t)a.N, (uint64_t)a.ldb, 64, BK);
  if (rc) return 200 + rc;
  tmB2 = tmB;
  if (a.epilogue == 1) {
    rc = np_make_tmap_2d(&tmB2, a.B2, 2, (uint64_t)a.b_rows, (uint64_t)a.K, (uint64_t)a.ldb, BK, b_box_rows);
    if (rc) return 300 + rc;
  }
  tmAloc = tmA;
  tmBloc = tmB;
  GemmParams p{};
  p.b_local_flag = a.b_local_flag - 1;
  // 32-byte stores need every (row, 32-column chunk) address 32-byte aligned; destinations behind peer_base are
  // allocations of the symmetric heap (256-byte aligned)
  static const bool st32_on = !(getenv("NPB200_ST32") != nullptr && getenv("NPB200_ST32")[0] == '0');
  p.st32 = st32_on && !a.out_f32 && a.epilogue != 1 && (a.ldc % 16 == 0) && (a.group_stride_c % 16 == 0) &&
           (a.row_dst || (((uintptr_t)a.C) % 32 == 0));
  if (a.push_src && a.push_n > 0) {
    if (a.push_n > 8 || (a.push_bytes & 15) || (((uintptr_t)a.push_src) & 15)) return 1;
    p.push_src = (const uint4*)a.push_src; p.push_vecs = a.push_bytes >> 4; p.push_n = a.push_n;
    p.push_ctr = a.push_ctr;
    for (int r = 0; r < a.push_n; ++r) { p.push_dst[r] = (uint4*)a.push_dst[r]; p.push_flag[r] = a.push_flag[r]; }
  }
  p.m_rot = a.m_rot; p.n_rot = a.n_rot;
  if (a.A_loc && !a.a_mn && a.a_loc_hi > a.a_loc_lo && a.a_loc_lo % BM == 0) {
    rc = np_make_tmap_2d(&tmAloc, a.A_loc, 2, (uint64_t)(a.a_loc_hi - a.a_loc_lo), (uint64_t)a.K, (uint64_t)a.lda_loc, BK, BM);
    if (rc) return 600 + rc;
    p.a_loc_lo = a.a_loc_lo; p.a_loc_hi = a.a_loc_hi;
  }
  if (a.B_loc && !a.b_mn && a.epilogue != 1 && a.b_loc_hi > a.b_loc_lo && a.b_loc_lo % b_box_rows == 0 &&
      (a.b_loc_hi - a.b_loc_lo) % b_box_rows == 0) {
    rc = np_make_tmap_2d(&tmBloc, a.B_loc, 2, (uint64_t)(a.b_loc_hi - a.b_loc_lo), (uint64_t)a.K, (uint64_t)a.ldb_loc, BK,
                         b_box_rows);
    if (rc) return 700 + rc;
    p.b_loc_lo = a.b_loc_lo; p.b_loc_hi = a.b_loc_hi;
  }
  p.C = a.C; p.C2 = a.C2; p.M = a.M; p.N = a.N; p.K = a.K; p.ldc = a.ldc; p.ldc2 = a.ldc2;
  p.bias = (a.epilogue == 0 && a.alpha != 0.f) ? a.bias : nullptr;
  p.a_mn = a.a_mn; p.b_mn = a.b_mn; p.out_f32 = a.out_f32; p.accumulate = a.accumulate;
  p.epilogue = a.epilogue; p.mode = a.mode; p.alpha = a.alpha;
  p.mblk_group = a.mblk_group; p.mblk_rows = a.mblk_rows; p.group_stride_b = a.group_stride_b;
  p.num_groups = a.num_groups; p.blocks_per_group = a.blocks_per_group; p.group_stride_c = a.group_stride_c;
  p.ready_flags = a.ready_flags; p.mblk_flag = a.mblk_flag; p.epoch = a.epoch;
  p.flag_limit_ns = a.flag_limit_ns ? a.flag_limit_ns : NP_WAIT_LIMIT_NS;
  p.row_dst = a.row_dst; p.peer_base = a.peer_base;
  p.done_counters = a.done_counters; p.done_expected = a.done_expected; p.done_flag_ptr = a.done_flag_ptr;
  p.Cin = a.Cin ? a.Cin : (a.accumulate ? a.C : nullptr);
  p.ldcin = a.Cin ? a.ldcin : a.ldc;
  p.epoch_base = a.epoch_base;
  p.b_ready_flags = a.b_ready_flags; p.b_rows_per_flag = a.b_rows_per_flag;

  constexpr int SMEM = STAGES * (TM * BK * 2 + BN * BK * 2) + 1024 + 256;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int bn_out = a.epilogue == 1 ? BN / 2 : BN;
  const int m_blocks = (a.M + TM - 1) / TM, n_blocks = (a.N + bn_out - 1) / bn_out;
  const long long tiles = (long long)m_blocks * n_blocks * (a.mode == 2 ? a.num_groups : 1);
  int cap = a.max_ctas > 0 ? a.max_ctas : g_num_sms;
  int grid = (int)(tiles < cap ? tiles : cap);
  if (grid <= 0) return 0;
  gemm_bf16_kernel<BN, STAGES, MT><<<grid, 192, SMEM, stream>>>(tmA, tmB, tmB2, tmAloc, tmBloc, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// C[M,N] (+)= alpha * A * B^T with the operand layouts described in NpGemmArgs.
// Returns 0 or a launch/setup error; device-side problems are reported via np_status_read.
NP_API int np_gemm_bf16(const NpGemmArgs* args, void* stream) {
  const NpGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0) return 0;
  // The tensor-map encode below is a driver call: make sure this host thread (e.g. an autograd
  // worker that has not touched the runtime yet) has the device's primary context bound.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)
      return 2;
    ctx_bound = true;
  }
  if ((a.lda % 8) || (a.ldb % 8) || (((uintptr_t)a.A) & 15) || (((uintptr_t)a.B) & 15)) return 1;
  int bn = a.bn;
  if (a.epilogue == 1) bn = 256;
  if (bn == 0) bn = (a.N >= 256 && (a.N % 256 == 0 || a.N >= 2048)) ? 256 : 128;
  if (bn == 256) {
    // 256 x 256 tiles where the form allows (no per-128-row-block tables, flags or pushes) and the problem has
    // enough of them to occupy the SMs; NPB200_GEMM_MT=1 keeps the 128-row tiles
    static const int mt_env = getenv("NPB200_GEMM_MT") ? atoi(getenv("NPB200_GEMM_MT")) : 0;
    int mt = a.mt ? a.mt : mt_env;
    const bool plain = a.mode != 1 && !a.row_dst && !a.ready_flags && !a.b_ready_flags && !a.push_src && !a.A_loc &&
                       !a.B_loc && !a.done_counters && a.m_rot == 0 && a.n_rot == 0;
    if (mt == 0) {
      // A 256-row tile costs about 1.68 tiles of 128 rows (measured on B200: 8192^3 1354 -> 1610 TFLOP/s, 4096 x 32000
      // x 2048 1282 -> 1444, 4096 x 2048 x 5632 1037 -> 1264), so it wins unless its coarser grain wastes the last wave
      const int bn_out = a.epilogue == 1 ? 128 : 256;
      const long long groups = a.mode == 2 ? a.num_groups : 1;
      const long long nb = (a.N + bn_out - 1) / bn_out;
      const long long tiles1 = (long long)((a.M + 127) / 128) * nb * groups;
      const long long tiles2 = (long long)((a.M + 255) / 256) * nb * groups;
      if (g_num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
      }
      const int sms = a.max_ctas > 0 ? a.max_ctas : (g_num_sms > 0 ? g_num_sms : 148);
      const long long w1 = (tiles1 + sms - 1) / sms, w2 = (tiles2 + sms - 1) / sms;
      mt = (plain && a.M >= 256 && 1.68 * (double)w2 < (double)w1) ? 2 : 1;
    }
    if (mt == 2 && plain) return launch_gemm<256, 3, 2>(a, (cudaStream_t)stream);
    return launch_gemm<256, 4, 1>(a, (cudaStream_t)stream);
  }
  return launch_gemm<128, 6, 1>(a, (cudaStream_t)stream);
}

NP_API int np_status_read(int* out8) {
  return (int)cudaMemcpyFromSymbol(out8, g_np_status, sizeof(int) * 8);
}
// Per-SM communication time in ns accumulated since the last reset (see account_interval): copies NP_MAX_SMS
// values into `out_ns` and, when `reset` is set, zeroes the counters. Synchronises the device.
NP_API int np_wait_stats_read(unsigned long long* out_ns, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out_ns, g_np_wait_ns, sizeof(unsigned long long) * NP_MAX_SMS);
  if (e != cudaSuccess) return (int)e;
  if (reset) {
    static const unsigned long long z[NP_MAX_SMS] = {0};
    e = cudaMemcpyToSymbol(g_np_wait_ns, z, sizeof(z));
  }
  return (int)e;
}
NP_API int np_wait_stats_slots() { return NP_MAX_SMS; }
NP_API int np_status_clear() {
  int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_np_status, z, sizeof(z));
}
NP_API int np_num_sms() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}
