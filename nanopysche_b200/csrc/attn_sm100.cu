// Flash attention for sm_100a (head_dim 128, bf16, causal or full, GQA-native), forward and backward,
// on tcgen05 tensor cores: S = Q K^T and O += P V (and the five backward products) are tcgen05.mma with
// TMEM accumulators, Q/K/V/dO tiles arrive by 4-D TMA straight from the strided [B, S, H, hd] tensors
// (so the q / k / v slices of the fused QKV GEMM output need no copy), softmax runs in registers on
// eight warps that read S out of TMEM (two threads per row, 64 columns each), and P / dS go back to tensor
// memory as bf16 and feed the next MMA as its TMEM A operand. The output accumulator stays in TMEM as well and
// is only rescaled when a row maximum has grown by more than 2^8. Scores never touch shared or global memory.
//
// K/V (forward, dQ) and Q/dO (dK/dV) may come from a *list* of tensor maps - one per context-parallel
// rank, pointing into that rank's symmetric memory - so a sequence sharded over GPUs is attended to by
// loading the peers' tiles directly over NVLink inside the kernel (plain TMA loads, no multicast):
// the context-parallel KV exchange is fused into the attention kernel. Causality uses global token
// positions of each 128-row block, which also expresses the zig-zag layout.
//
// Replaces F.scaled_dot_product_attention (reference: model/attention.py:121-127) and the dense
// per-step matmul+softmax of its ring attention (distributed/context_parallel.py:301-317).
#include "common.cuh"

namespace {

constexpr int KID_ATTN = 30;
constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;   // one [128 x 128] bf16 tile = two 64-column swizzled chunks
constexpr int CHUNK_BYTES = 128 * 64 * 2;
constexpr int MAX_SRC = 8;

struct TmapList {
  CUtensorMap m[MAX_SRC];
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// [128 rows x 128 cols] tile (cols = hd) of head `h`, rows starting at `s0`, batch `b`: two 64-col chunks
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int h, int s0, int b) {
  tma_load_4d(dst, tm, bar, 0, h, s0, b);
  tma_load_4d(dst + CHUNK_BYTES, tm, bar, 64, h, s0, b);
}
// K-major operand [rows, 128 k]: k-step kk (16 elements) -> chunk kk/4, +32 B per step inside the chunk
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kk) {
  return np::make_smem_desc(tile + (kk >> 2) * CHUNK_BYTES + (kk & 3) * 32, 16, 1024);
}
// MN-major operand stored as [k rows, 128 mn cols] (two 64-col chunks): k-step = 16 rows = +2048 B,
// LBO = distance between the two 64-wide chunks
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kk) {
  return np::make_smem_desc(tile + kk * 2048, CHUNK_BYTES, 1024);
}
// Sources that are still arriving in this GPU's memory (a peer is pushing them): flag[idx[s]] reaches the epoch
// once source s is complete. The TMA producer checks it before its first load from the source.
struct SrcFlags {
  const int* flags;     // nullptr: every source is ready at launch
  int idx[MAX_SRC];
  int own;                 // flag index guarding the kernel's resident operand (Q / dO or K / V), -1: none
  int epoch;
  const int* epoch_base;   // optional device counter added to `epoch` (keeps epochs valid under graph replay)
  unsigned long long limit_ns;
};
__device__ __forceinline__ bool src_ready(const SrcFlags& f, int s, int kid) {
  if (!f.flags || f.idx[s] < 0) return true;   // negative index: the source was produced by this GPU itself
  const int want = f.epoch + (f.epoch_base ? *f.epoch_base : 0);
  return np::wait_flag_ge(f.flags + f.idx[s], want, f.limit_ns, kid, 200 + s);
}
__device__ __forceinline__ bool own_ready(const SrcFlags& f, int kid) {
  if (!f.flags || f.own < 0) return true;
  const int want = f.epoch + (f.epoch_base ? *f.epoch_base : 0);
  return np::wait_flag_ge(f.flags + f.own, want, f.limit_ns, kid, 250);
}

// All-gather of this rank's K|V shard issued by the attention kernel itself: chunks are taken from an atomic
// counter by whichever CTAs run first (the grid may be several waves deep, so no chunk may be tied to a CTA that
// has not started), stored into every peer's gather buffer, and the CTA that completes the last chunk releases
// this rank's arrival flag on the peers. `ctr` ([2] ints) is zeroed by the host before the launch.
struct PushArgs {
  const uint4* src[2];      // K and V shards (contiguous)
  long long vecs_each;      // 16-byte vectors per shard
  uint4* dst[MAX_SRC];      // peer gather slots of this rank: K at [0, vecs_each), V behind it
  int* flag[MAX_SRC];
  int n;                    // peers to push to (0: no push)
  int* ctr;
  int epoch;
  const int* epoch_base;
};
// `s_chunk`: one int of the kernel's dynamic shared memory (a static __shared__ variable here would move the
// dynamic region off its 1024-byte boundary and past the size the launch asked for).
__device__ __forceinline__ void push_kv(const PushArgs& a, volatile int* s_chunk) {
  if (a.n <= 0) return;
  constexpr long long CH = 2048;   // vectors per chunk (32 KB)
  const long long total = 2 * a.vecs_each;
  const int nch = (int)((total + CH - 1) / CH);
  for (;;) {
    if (threadIdx.x == 0) *s_chunk = atomicAdd(&a.ctr[0], 1);
    __syncthreads();
    const int c = *s_chunk;
    __syncthreads();
    if (c >= nch) break;
    const long long hi = (c + 1) * CH < total ? (c + 1) * CH : total;
    for (long long i = c * CH + threadIdx.x; i < hi; i += blockDim.x) {
      const uint4 v = i < a.vecs_each ? a.src[0][i] : a.src[1][i - a.vecs_each];
      for (int r = 0; r < a.n; ++r) a.dst[r][i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&a.ctr[1], 1) == nch - 1) {
      __threadfence_system();
      const int ep = a.epoch + (a.epoch_base ? *a.epoch_base : 0);
      for (int r = 0; r < a.n; ++r) np::st_release_sys(a.flag[r], ep);
    }
  }
}

struct FwdParams {
  __nv_bfloat16* O; long long o_sb, o_ss, o_sh;   // output strides (elements): batch, seq, head
  float* lse;                                      // [B, Hq, Sq]
  int B, Sq, Hq, Hkv, causal;
  int lse_H;                                       // heads of the lse array (>= Hq when this launch covers a head slice)
  float scale_log2;
  int n_src;                                       // number of KV sources (1 without context parallelism)
  int src_blocks;                                  // 128-row KV blocks per source
  int src_len;                                     // valid KV rows per source
  SrcFlags fl;                                     // arrival flags of the KV sources (context parallelism)
  PushArgs push;                                   // this rank's K|V shard, pushed by the kernel's first CTAs
  const int* q_blk_pos;                            // [Sq/128] global position of each local Q block (nullptr: i*128 + q_off)
  const int* k_blk_pos;                            // [n_src * src_blocks] global position of each KV block (nullptr: j*128)
  int q_off;
};

// tcgen05.mma with the A operand in tensor memory: D[tmem] (+)= A[tmem, 128 lanes x K] * B[smem desc]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe (degree-4 polynomial on the fraction, exponent patched in with integer adds; relative error
// about 4e-5, 0 below 2^-125): used for a share of the scores so that the special-function unit is not the only
// pipe the exp2 phase runs on
__device__ __forceinline__ float ex2_poly(float x) {
  const bool tiny = x < -125.f;              // masked scores (-inf) must give exactly 0
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;            // 1.5 * 2^23: the integer part lands in the low mantissa bits
  const float f = x - (t - 12582912.f);      // [-0.5, 0.5]
  float p = fmaf(f, 0.0096181291f, 0.0555041087f);
  p = fmaf(p, f, 0.2402265070f);
  p = fmaf(p, f, 0.6931471806f);
  p = fmaf(p, f, 1.0f);
  return tiny ? 0.f : __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
#ifndef NP_FWD2_POLY
#define NP_FWD2_POLY 0   // 1: every fourth score of the two-Q-tile forward goes through ex2_poly (measured: 1.4x slower)
#endif
// mbarrier wait whose outcome is the same for every lane of the warp, so that the .sync.aligned tensor-memory
// instructions that follow are never reached by part of a warp
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int kid, int where) {
  return __all_sync(0xffffffffu, np::mbar_wait(bar, parity, abort_flag, kid, where));
}
// Named barrier of the NS warps that share the rows of one TMEM lane quarter (NS threads per row, 128/NS columns each). Every softmax
// thread reaches every such barrier in every iteration, also after a failed wait, so none is left waiting.
template <int NS>
__device__ __forceinline__ void row_sync(int quarter) {
  asm volatile("bar.sync %0, %1;" ::"r"(1 + quarter), "n"(NS * 32) : "memory");
}
template <int NS>
__device__ __forceinline__ void softmax_sync_all() {
  asm volatile("bar.sync 5, %0;" ::"n"(NS * 128) : "memory");
}
// CW consecutive fp32 columns of this thread's lane into registers / CW/2 packed columns back
template <int CW>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
#pragma unroll
  for (int c = 0; c < CW / 32; ++c) np::tmem_ld32(taddr + c * 32, r + c * 32);
  np::tmem_ld_wait();
}
template <int NCOLS>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
#pragma unroll
  for (int c = 0; c < NCOLS / 16; ++c) tmem_st16(taddr + c * 16, r + c * 16);
}

// warp 0: TMA, warp 1: MMA issue, then 4*NS softmax warps (NS per TMEM lane quarter)
constexpr int nthreads(int ns) { return 64 + ns * 128; }
constexpr float RESCALE_LOG2 = 8.f;

// Barrier slots of the forward kernel
enum { FB_Q = 0, FB_K = 1, FB_KE = 4, FB_V = 7, FB_VE = 10, FB_S = 13, FB_P = 15, FB_O = 16, FB_COUNT = 17 };
constexpr int F_KST = 3, F_VST = 3;   // three-deep K and V rings: a TMA load has two iterations to land

// Tensor memory map of the forward kernel (columns): S double buffer, O accumulator, P double buffer (bf16 pairs)
constexpr uint32_t F_S = 0, F_O = 256, F_P = 384;

template <int NS>
__global__ void __launch_bounds__(nthreads(NS), 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ TmapList tmK,
                const __grid_constant__ TmapList tmV, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_al[];
  const uint32_t base = np::smem_u32(smem_al);
  if (base & 1023u) {   // the swizzled tiles need it; nothing has been allocated or started yet
    if (threadIdx.x == 0) np::report(NP_ERR_BAD_ARG, KID_ATTN, (int)(base & 1023u));
    return;
  }
  const uint32_t sQ = base, sK0 = base + TILE_BYTES, sV0 = sK0 + F_KST * TILE_BYTES;
  const uint32_t bar = sV0 + F_VST * TILE_BYTES;
  auto B_ = [&](int i) { return bar + 8u * i; };
  uint8_t* tail = smem_al + (1 + F_KST + F_VST) * TILE_BYTES + 8 * FB_COUNT + 8;   // 16-byte aligned
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);
  float* xch = reinterpret_cast<float*>(tail + 16);   // [2 iterations][NS][128 rows]: row maxima, at the end row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Sq + BQ - 1) / BQ;
  // grid.x runs over (head, batch), grid.y over the Q blocks from the last (most KV blocks under causal
  // masking) to the first: CTAs are issued heaviest first across the whole grid
  const int qb = nqb - 1 - (int)blockIdx.y;
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q_pos0 = p.q_blk_pos ? p.q_blk_pos[qb] : qb * BQ + p.q_off;
  const int total_blocks = p.n_src * p.src_blocks;
  auto k_pos0 = [&](int j) { return p.k_blk_pos ? p.k_blk_pos[j] : (j % p.src_blocks) * BKV; };
  // Every role walks the same list: the KV blocks that causality does not hide from all rows of this Q block.
  auto next_vis = [&](int j) {
    while (j < total_blocks && p.causal && k_pos0(j) > q_pos0 + BQ - 1) ++j;
    return j;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < FB_COUNT; ++i) np::mbar_init(B_(i), i == FB_P ? 4 * NS : 1);
    *abort_flag = 0;
    np::mbar_fence_init();
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), 512);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;
  const uint32_t tO = tmem + F_O;
  push_kv(p.push, reinterpret_cast<volatile int*>(tail + 8));

  if (warp == 0) {
    if (lane == 0) {
      if (!own_ready(p.fl, KID_ATTN)) *abort_flag = 1;
      np::mbar_expect_tx(B_(FB_Q), TILE_BYTES);
      load_tile(sQ, &tmQ, B_(FB_Q), h, qb * BQ, b);
      int i = 0, last_src = -1;
      for (int j = next_vis(0); j < total_blocks && !*abort_flag; j = next_vis(j + 1), ++i) {
        const int ks = i % F_KST, vs = i % F_VST;
        const int src = j / p.src_blocks, jb = j - src * p.src_blocks;
        if (src != last_src) {
          if (!src_ready(p.fl, src, KID_ATTN)) { *abort_flag = 1; break; }
          last_src = src;
        }
        if (!np::mbar_wait(B_(FB_KE + ks), ((uint32_t)(i / F_KST) & 1u) ^ 1u, abort_flag, KID_ATTN, 1)) break;
        np::mbar_expect_tx(B_(FB_K + ks), TILE_BYTES);
        load_tile(sK0 + ks * TILE_BYTES, &tmK.m[src], B_(FB_K + ks), hkv, jb * BKV, b);
        if (!np::mbar_wait(B_(FB_VE + vs), ((uint32_t)(i / F_VST) & 1u) ^ 1u, abort_flag, KID_ATTN, 10)) break;
        np::mbar_expect_tx(B_(FB_V + vs), TILE_BYTES);
        load_tile(sV0 + vs * TILE_BYTES, &tmV.m[src], B_(FB_V + vs), hkv, jb * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = np::make_idesc(128, 128, 1, 1, 0, 0);   // Q (K-major) x K (K-major)
      const uint32_t idesc_pv = np::make_idesc(128, 128, 1, 1, 0, 1);   // P (TMEM) x V (MN-major)
      bool ok = np::mbar_wait(B_(FB_Q), 0, abort_flag, KID_ATTN, 2);
      auto issue_qk = [&](int i) {
        const int st = i & 1, ks = i % F_KST;
        if (!np::mbar_wait(B_(FB_K + ks), (uint32_t)(i / F_KST) & 1u, abort_flag, KID_ATTN, 3)) return false;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tmem + F_S + st * 128, desc_kmajor(sQ, kk), desc_kmajor(sK0 + ks * TILE_BYTES, kk), idesc_qk, kk > 0);
        np::tc_commit(B_(FB_S + st));
        np::tc_commit(B_(FB_KE + ks));
        return true;
      };
      int j = next_vis(0);
      if (ok && j < total_blocks) ok = issue_qk(0);
      for (int i = 0; j < total_blocks && ok && !*abort_flag; ++i) {
        const int st = i & 1, vs = i % F_VST;
        // S of the next block is computed while the softmax warps work on this one. Its S and P buffers were
        // last used for block i-1: S read before P of block i-1 arrived, P consumed by P V of block i-1 (issued).
        j = next_vis(j + 1);
        if (j < total_blocks) ok = issue_qk(i + 1);
        ok = ok && np::mbar_wait(B_(FB_P), (uint32_t)i & 1u, abort_flag, KID_ATTN, 5) &&   // P ready, O rescaled
             np::mbar_wait(B_(FB_V + vs), (uint32_t)(i / F_VST) & 1u, abort_flag, KID_ATTN, 4);
        if (!ok) break;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16_ts(tO, tmem + F_P + st * 64 + kk * 8, desc_mnmajor(sV0 + vs * TILE_BYTES, kk), idesc_pv,
                        (i > 0) || (kk > 0));
        np::tc_commit(B_(FB_O));
        np::tc_commit(B_(FB_VE + vs));
      }
    }
  } else {
    constexpr int CW = 128 / NS;
    const int quarter = warp & 3, hf = (warp - 2) >> 2;     // this thread: row r, columns [CW hf, CW hf + CW)
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int q_pos = q_pos0 + r;
    float m = -INFINITY, l = 0.f;                            // running maximum (log2 domain) and row sum
    bool ok = true;
    int nvis = 0;
    for (int j = next_vis(0); j < total_blocks; j = next_vis(j + 1), ++nvis) {
      const int i = nvis, st = i & 1;
      const int jb = j % p.src_blocks;
      const int kp0 = k_pos0(j);
      const int valid_cols = p.src_len - jb * BKV;           // columns beyond the source's length are padding
      const bool need_mask = (p.causal && kp0 + BKV - 1 > q_pos0) || valid_cols < BKV;
      ok = ok && !*abort_flag && warp_wait(B_(FB_S + st), (uint32_t)(i >> 1) & 1u, abort_flag, KID_ATTN, 7);
      uint32_t s[CW];
      float mloc = -INFINITY;
      if (ok) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tmem + F_S + st * 128 + lane_off + hf * CW, s);
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < CW; ++e) {
            const int col = hf * CW + e;
            if (col >= valid_cols || (p.causal && kp0 + col > q_pos)) s[e] = 0xff800000u;   // -inf
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < CW; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(s[e]));
        mloc = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      }
      xch[(st * NS + hf) * 128 + r] = mloc;
      row_sync<NS>(quarter);
      if (ok) {
        float mx = mloc;   // all NS threads of the row agree on it
#pragma unroll
        for (int o = 0; o < NS; ++o) mx = fmaxf(mx, xch[(st * NS + o) * 128 + r]);
        // the accumulator is only rescaled when some row of the warp outgrew its reference maximum by 2^8
        const bool grow = mx > m + RESCALE_LOG2 || (m == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m, mx);
          const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m - m_new);
          if (i > 0) {
            ok = warp_wait(B_(FB_O), (uint32_t)(i - 1) & 1u, abort_flag, KID_ATTN, 8);   // P V of block i-1 is done
            if (ok) {
              np::tc_fence_after();
              uint32_t t[CW];
              tmem_ld_cols<CW>(tO + lane_off + hf * CW, t);
#pragma unroll
              for (int e = 0; e < CW; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
              tmem_st_cols<CW>(tO + lane_off + hf * CW, t);
            }
          }
          l *= alpha;
          m = m_new;
        }
      }
      if (ok) {
        const float m_use = (m == -INFINITY) ? 0.f : m;
        float rs[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[CW / 2];
#pragma unroll
        for (int e = 0; e < CW; e += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(s[e]), p.scale_log2, -m_use));
          const float p1 = ex2(fmaf(__uint_as_float(s[e + 1]), p.scale_log2, -m_use));
          rs[e & 2] += p0;
          rs[(e & 2) + 1] += p1;
          pk[e >> 1] = np::pack_bf16(p0, p1);
        }
        l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
        tmem_st_cols<CW / 2>(tmem + F_P + st * 64 + lane_off + hf * (CW / 2), pk);
        tmem_st_wait();
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(B_(FB_P));
      }
    }
    // all threads of a row hold the same maximum; their partial sums add up
    row_sync<NS>(quarter);   // everyone has read the last maxima: the slots can carry the sums now
    xch[hf * 128 + r] = l;
    row_sync<NS>(quarter);
    float l_tot = 0.f;
#pragma unroll
    for (int o = 0; o < NS; ++o) l_tot += xch[o * 128 + r];
    ok = ok && !*abort_flag;
    if (nvis > 0) ok = ok && warp_wait(B_(FB_O), (uint32_t)(nvis - 1) & 1u, abort_flag, KID_ATTN, 9);
    ok = __all_sync(0xffffffffu, ok);
    const int row = qb * BQ + r;
    if (ok) {
      uint32_t t[CW];
      if (nvis > 0) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tO + lane_off + hf * CW, t);
      } else {
#pragma unroll
        for (int e = 0; e < CW; ++e) t[e] = 0u;
      }
      if (row < p.Sq) {
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        __nv_bfloat16* dst = p.O + (size_t)b * p.o_sb + (size_t)row * p.o_ss + (size_t)h * p.o_sh + hf * CW;
#pragma unroll
        for (int g = 0; g < CW / 8; ++g) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(t[8 * g + e]) * inv;
          reinterpret_cast<uint4*>(dst)[g] = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                                        np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
        }
        if (p.lse && hf == 0)
          p.lse[((size_t)b * p.lse_H + h) * p.Sq + row] = l_tot > 0.f ? (m * 0.6931471805599453f + logf(l_tot)) : -INFINITY;
      }
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Forward with two Q tiles per CTA (plain single-source case: no arrival flags, no push, positions j * 128).
//
// One CTA owns 256 query rows of a (head, batch): tile 0 = rows [0, 128), tile 1 = rows [128, 256). Warps 2-5 are
// the softmax group of tile 0 and warps 6-9 that of tile 1, one thread per row and all 128 score columns of a KV
// block per thread, so no row exchange is needed. Both tiles share every K and V block, which halves the K/V
// traffic per query row, and the MMA warp interleaves them:  P V of tile 0, S of tile 0 for the next block,
// P V of tile 1, S of tile 1 ...  While one group is in its exp2 phase (which saturates the special-function
// unit) the other group's maximum / rescale phases and the tensor pipe run. TMEM: S of tile t at columns [128 t,
// 128 t + 128), O of tile t at [256 + 128 t, ...); P (bf16 pairs, 64 columns) overwrites the S it came from, which
// is safe because a thread loads its whole row of S before it stores P, and S of the next block is only issued
// after the P V that read P.
enum { G_Q = 0, G_K = 1, G_KE = 4, G_V = 7, G_VE = 9, G_S = 11, G_P = 13, G_O = 15, G_COUNT = 17 };
#ifdef NP_ATTN_PROF   // development build only: cycles per softmax phase, summed over (lane 0 of) all warps
__device__ unsigned long long g_fwd2_prof[8];
#define PROF_T(v) const long long v = clock64()
#define PROF_ADD(i, a, b) do { if (lane == 0) atomicAdd(&g_fwd2_prof[i], (unsigned long long)((b) - (a))); } while (0)
#else
#define PROF_T(v) do {} while (0)
#define PROF_ADD(i, a, b) do {} while (0)
#endif
constexpr int G_KST = 3, G_VST = 2;   // Q0, Q1, three K stages, two V stages: seven 32 KB tiles

__global__ void __launch_bounds__(320, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_al[];
  const uint32_t base = np::smem_u32(smem_al);
  if (base & 1023u) {
    if (threadIdx.x == 0) np::report(NP_ERR_BAD_ARG, KID_ATTN, (int)(base & 1023u));
    return;
  }
  const uint32_t sQ = base, sK0 = base + 2 * TILE_BYTES, sV0 = sK0 + G_KST * TILE_BYTES;
  const uint32_t bar = sV0 + G_VST * TILE_BYTES;
  auto B_ = [&](int i) { return bar + 8u * i; };
  uint8_t* tail = smem_al + (2 + G_KST + G_VST) * TILE_BYTES + 8 * G_COUNT + 8;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb2 = (p.Sq + 2 * BQ - 1) / (2 * BQ);
  const int qb2 = nqb2 - 1 - (int)blockIdx.y;             // heaviest (most visible KV blocks) first
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int row0 = qb2 * 2 * BQ;                          // first query row of tile 0
  // number of KV blocks tile t has to look at: the blocks form a prefix of the source
  auto nvis = [&](int t) -> int {
    if (row0 + t * BQ >= p.Sq) return 0;                  // tile past the end of the sequence
    if (!p.causal) return p.src_blocks;
    const int last = row0 + t * BQ + p.q_off + BQ - 1;    // position of the tile's last row
    if (last < 0) return 0;
    const int n = last / BKV + 1;
    return n < p.src_blocks ? n : p.src_blocks;
  };
  const int nv0 = nvis(0), nv1 = nvis(1);
  const int nv = nv0 > nv1 ? nv0 : nv1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < G_COUNT; ++i) np::mbar_init(B_(i), (i == G_P || i == G_P + 1) ? 4 : 1);
    *abort_flag = 0;
    np::mbar_fence_init();
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), 512);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;

  if (warp == 0) {
    if (lane == 0) {
      np::mbar_expect_tx(B_(G_Q), 2 * TILE_BYTES);
      load_tile(sQ, &tmQ, B_(G_Q), h, row0, b);
      load_tile(sQ + TILE_BYTES, &tmQ, B_(G_Q), h, row0 + BQ, b);   // rows past the end read as zero
      for (int i = 0; i < nv && !*abort_flag; ++i) {
        const int ks = i % G_KST, vs = i % G_VST;
        if (!np::mbar_wait(B_(G_KE + ks), ((uint32_t)(i / G_KST) & 1u) ^ 1u, abort_flag, KID_ATTN, 21)) break;
        np::mbar_expect_tx(B_(G_K + ks), TILE_BYTES);
        load_tile(sK0 + ks * TILE_BYTES, &tmK, B_(G_K + ks), hkv, i * BKV, b);
        if (!np::mbar_wait(B_(G_VE + vs), ((uint32_t)(i / G_VST) & 1u) ^ 1u, abort_flag, KID_ATTN, 22)) break;
        np::mbar_expect_tx(B_(G_V + vs), TILE_BYTES);
        load_tile(sV0 + vs * TILE_BYTES, &tmV, B_(G_V + vs), hkv, i * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = np::make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_pv = np::make_idesc(128, 128, 1, 1, 0, 1);
      bool ok = np::mbar_wait(B_(G_Q), 0, abort_flag, KID_ATTN, 23);
      // S of tile t for block i (the K stage must have landed; the caller has waited for it)
      auto issue_s = [&](int t, int i) {
        const int ks = i % G_KST;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tmem + t * 128, desc_kmajor(sQ + t * TILE_BYTES, kk), desc_kmajor(sK0 + ks * TILE_BYTES, kk),
                         idesc_qk, kk > 0);
        np::tc_commit(B_(G_S + t));
      };
      auto wait_k = [&](int i) {
        const bool w = np::mbar_wait(B_(G_K + i % G_KST), (uint32_t)(i / G_KST) & 1u, abort_flag, KID_ATTN, 24);
        np::tc_fence_after();
        return w;
      };
      auto issue_pv = [&](int t, int i) {
        const int vs = i % G_VST;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, desc_mnmajor(sV0 + vs * TILE_BYTES, kk), idesc_pv,
                        (i > 0) || (kk > 0));
        np::tc_commit(B_(G_O + t));
      };
      if (ok && nv > 0) {
        ok = wait_k(0);
        if (ok) {
          if (nv0 > 0) issue_s(0, 0);
          if (nv1 > 0) issue_s(1, 0);
          np::tc_commit(B_(G_KE + 0));
        }
      }
      for (int i = 0; i < nv && ok && !*abort_flag; ++i) {
        const int vs = i % G_VST;
        bool have_k = false;
        ok = np::mbar_wait(B_(G_V + vs), (uint32_t)(i / G_VST) & 1u, abort_flag, KID_ATTN, 25);
        if (ok && i < nv0) {
          ok = np::mbar_wait(B_(G_P + 0), (uint32_t)i & 1u, abort_flag, KID_ATTN, 26);   // P of tile 0 stored, O rescaled
          if (!ok) break;
          np::tc_fence_after();
          issue_pv(0, i);
          if (i + 1 < nv0) {
            ok = wait_k(i + 1);
            if (!ok) break;
            have_k = true;
            issue_s(0, i + 1);
          }
        }
        if (ok && i < nv1) {
          ok = np::mbar_wait(B_(G_P + 1), (uint32_t)i & 1u, abort_flag, KID_ATTN, 27);
          if (!ok) break;
          np::tc_fence_after();
          issue_pv(1, i);
        }
        if (!ok) break;
        np::tc_commit(B_(G_VE + vs));
        if (i + 1 < nv) {
          if (i + 1 < nv1) {
            if (!have_k) ok = wait_k(i + 1);
            if (!ok) break;
            issue_s(1, i + 1);
          }
          np::tc_commit(B_(G_KE + (i + 1) % G_KST));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax groups: one thread per query row
    const int t = (warp - 2) >> 2;                        // tile of this warp's group
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + t * 128 + lane_off, tO = tmem + 256 + t * 128 + lane_off;
    const int row = row0 + t * BQ + r;
    const int q_pos = row + p.q_off;
    const int q_pos_first = row0 + t * BQ + p.q_off;
    const int my_nv = t == 0 ? nv0 : nv1;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < my_nv; ++i) {
      const int kp0 = i * BKV;
      const int valid_cols = p.src_len - kp0;
      const bool need_mask = (p.causal && kp0 + BKV - 1 > q_pos_first) || valid_cols < BKV;
      PROF_T(c0);
      ok = ok && !*abort_flag && warp_wait(B_(G_S + t), (uint32_t)i & 1u, abort_flag, KID_ATTN, 28);
      if (!ok) break;
      np::tc_fence_after();
      PROF_T(c1);
      uint32_t s[128];
      tmem_ld_cols<128>(tS, s);
      PROF_T(c2);
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 128; ++e)
          if (e >= valid_cols || (p.causal && kp0 + e > q_pos)) s[e] = 0xff800000u;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 128; e += 8) {      // three-input maxima: 64 instructions for the 128 scores
        mx4[0] = fmax3(mx4[0], __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
        mx4[1] = fmax3(mx4[1], __uint_as_float(s[e + 2]), __uint_as_float(s[e + 3]));
        mx4[2] = fmax3(mx4[2], __uint_as_float(s[e + 4]), __uint_as_float(s[e + 5]));
        mx4[3] = fmax3(mx4[3], __uint_as_float(s[e + 6]), __uint_as_float(s[e + 7]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const bool grow = mx > m + RESCALE_LOG2 || (m == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m, mx);
        const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m - m_new);
        if (i > 0) {
          ok = warp_wait(B_(G_O + t), (uint32_t)(i - 1) & 1u, abort_flag, KID_ATTN, 29);   // P V of block i-1 is done
          if (!ok) break;
          np::tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_cols<32>(tO + c * 32, o);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_cols<32>(tO + c * 32, o);
          }
        }
        l *= alpha;
        m = m_new;
      }
      PROF_T(c3);
      const float m_use = (m == -INFINITY) ? 0.f : m;
      float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {                      // 32 scores -> 16 packed columns of P, over the S they came from
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float x0 = fmaf(__uint_as_float(s[c * 32 + e]), p.scale_log2, -m_use);
          const float x1 = fmaf(__uint_as_float(s[c * 32 + e + 1]), p.scale_log2, -m_use);
          const float p0 = ex2(x0);
          const float p1 = (NP_FWD2_POLY && (e & 2)) ? ex2_poly(x1) : ex2(x1);
          rs[e & 2] += p0;
          rs[(e & 2) + 1] += p1;
          pk[e >> 1] = np::pack_bf16(p0, p1);
        }
        tmem_st16(tS + c * 16, pk);
      }
      l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
      PROF_T(c4);
      tmem_st_wait();
      np::tc_fence_before();
      __syncwarp();
      if (lane == 0) np::mbar_arrive(B_(G_P + t));
      PROF_T(c5);
      PROF_ADD(0, c0, c1); PROF_ADD(1, c1, c2); PROF_ADD(2, c2, c3); PROF_ADD(3, c3, c4); PROF_ADD(4, c4, c5);
      PROF_ADD(5, c0, c0 + 1);
    }
    ok = ok && !*abort_flag;
    if (ok && my_nv > 0) ok = warp_wait(B_(G_O + t), (uint32_t)(my_nv - 1) & 1u, abort_flag, KID_ATTN, 30);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && row0 + t * BQ < p.Sq) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.O + (size_t)b * p.o_sb + (size_t)row * p.o_ss + (size_t)h * p.o_sh;
      if (my_nv > 0) np::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (my_nv > 0) {
          tmem_ld_cols<32>(tO + c * 32, o);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[8 * g + e]) * inv;
            reinterpret_cast<uint4*>(dst + c * 32)[g] = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                                                   np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
          }
        }
      }
      if (p.lse && row < p.Sq)
        p.lse[((size_t)b * p.lse_H + h) * p.Sq + row] = l > 0.f ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem, 512);
  }
}

int make_tmap_4d(CUtensorMap* out, const void* base, long long B, long long S, long long H, long long sb, long long ss,
                 long long sh) {
  NpEncodeTiledFn enc = np_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <class A>
int fill_push(PushArgs* q, const A* a) {
  q->n = 0;
  if (!a->push_k || a->push_n <= 0) return 0;
  if (a->push_n > MAX_SRC || (a->push_bytes & 15) || (((uintptr_t)a->push_k | (uintptr_t)a->push_v) & 15)) return 1;
  q->src[0] = (const uint4*)a->push_k; q->src[1] = (const uint4*)a->push_v;
  q->vecs_each = a->push_bytes >> 4;
  q->n = a->push_n; q->ctr = a->push_ctr; q->epoch = a->flag_epoch; q->epoch_base = a->epoch_base;
  for (int r = 0; r < a->push_n; ++r) { q->dst[r] = (uint4*)a->push_dst[r]; q->flag[r] = a->push_flag[r]; }
  return 0;
}

void fill_flags(SrcFlags* f, const int* flags, const int* idx, int n_src, int epoch, const int* epoch_base,
                unsigned long long limit_ns, int own) {
  f->flags = flags;
  f->own = own;
  f->epoch = epoch;
  f->epoch_base = epoch_base;
  f->limit_ns = limit_ns ? limit_ns : NP_WAIT_LIMIT_NS;
  for (int s = 0; s < MAX_SRC; ++s) f->idx[s] = (flags && idx && s < n_src) ? idx[s] : 0;
}

bool bind_ctx() {
  static thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)
      return false;
    bound = true;
  }
  return true;
}

}  // namespace

// Tensor layout of q / k / v / o: [B, S, H, 128] bf16 with element strides (sb, ss, sh); the last dim is
// contiguous. k_ptrs / v_ptrs: one base pointer per KV source (n_src = 1 without context parallelism).
struct NpAttnFwdArgs {
  const void* q; long long q_sb, q_ss, q_sh;
  const void* const* k_ptrs; const void* const* v_ptrs; long long k_sb, k_ss, k_sh;
  void* o; long long o_sb, o_ss, o_sh;
  float* lse;
  int B, Sq, Hq, Hkv, causal, n_src, src_len, q_off;
  float scale;
  const int* q_blk_pos; const int* k_blk_pos;
  int split;       // unused (two softmax threads per row)
  int lse_heads;   // heads of the lse array when q / o are a head slice of larger tensors (0: Hq)
  // KV sources that peers are still pushing into this GPU's memory: flags[flag_idx[s]] >= flag_epoch + *epoch_base
  const int* src_flags; const int* flag_idx; int flag_epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  int flag_own;    // 1 + flag index that guards q itself (0: none)
  // this rank's K|V shard pushed by the kernel itself: push_bytes of push_k then push_v to push_dst[r] (r < push_n),
  // then *push_flag[r] = flag_epoch (+ *epoch_base); push_ctr: two local ints the caller zeroes before the launch
  const void* push_k; const void* push_v; long long push_bytes; void* const* push_dst; int* const* push_flag;
  int push_n; int* push_ctr;
};

#ifdef NP_ATTN_PROF
NP_API int np_attn_prof_read(unsigned long long* out8, int reset) {
  cudaMemcpyFromSymbol(out8, g_fwd2_prof, sizeof(unsigned long long) * 8);
  if (reset) { unsigned long long z[8] = {0}; cudaMemcpyToSymbol(g_fwd2_prof, z, sizeof(z)); }
  return 0;
}
#endif

NP_API int np_attn_fwd(const NpAttnFwdArgs* a, void* stream) {
  if (a->B <= 0 || a->Sq <= 0 || a->src_len <= 0) return 0;
  if (a->n_src < 1 || a->n_src > MAX_SRC || a->Hq % a->Hkv) return 1;
  if ((a->q_ss | a->q_sh | a->q_sb | a->k_ss | a->k_sh | a->k_sb | a->o_ss | a->o_sh | a->o_sb) % 8 ||
      (((uintptr_t)a->q | (uintptr_t)a->o) & 15))
    return 1;
  if (!bind_ctx()) return 2;
  CUtensorMap tmQ;
  TmapList tmK, tmV;
  int rc = make_tmap_4d(&tmQ, a->q, a->B, a->Sq, a->Hq, a->q_sb, a->q_ss, a->q_sh);
  if (rc) return 100 + rc;
  for (int s = 0; s < a->n_src; ++s) {
    rc = make_tmap_4d(&tmK.m[s], a->k_ptrs[s], a->B, a->src_len, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
    if (rc) return 200 + rc;
    rc = make_tmap_4d(&tmV.m[s], a->v_ptrs[s], a->B, a->src_len, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
    if (rc) return 300 + rc;
  }
  for (int s = a->n_src; s < MAX_SRC; ++s) { tmK.m[s] = tmK.m[0]; tmV.m[s] = tmV.m[0]; }
  FwdParams p{};
  p.O = (__nv_bfloat16*)a->o; p.o_sb = a->o_sb; p.o_ss = a->o_ss; p.o_sh = a->o_sh; p.lse = a->lse;
  p.B = a->B; p.Sq = a->Sq; p.Hq = a->Hq; p.Hkv = a->Hkv; p.causal = a->causal;
  p.lse_H = a->lse_heads > 0 ? a->lse_heads : a->Hq;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.n_src = a->n_src; p.src_len = a->src_len; p.src_blocks = (a->src_len + BKV - 1) / BKV;
  p.q_blk_pos = a->q_blk_pos; p.k_blk_pos = a->k_blk_pos; p.q_off = a->q_off;
  fill_flags(&p.fl, a->src_flags, a->flag_idx, a->n_src, a->flag_epoch, a->epoch_base, a->flag_limit_ns,
             a->flag_own - 1);
  if (fill_push(&p.push, a)) return 1;
  // Plain single-source case with more than one Q block: two Q tiles per CTA (attn_fwd2_kernel)
  static const bool fwd2_on = [] { const char* e = getenv("NPB200_ATTN_FWD2"); return !(e && e[0] == '0'); }();
  if (fwd2_on && a->n_src == 1 && !a->src_flags && !a->push_k && !a->q_blk_pos && !a->k_blk_pos && a->flag_own == 0 &&
      a->Sq > BQ) {
    constexpr int SMEM2 = (2 + G_KST + G_VST) * TILE_BYTES + 8 * G_COUNT + 8 + 16;
    static_assert(SMEM2 <= 227 * 1024, "shared memory budget");
    static NpPerDeviceOnce attr2_once;
    bool& attr2_set = *attr2_once.slot();
    if (!attr2_set) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2);
      if (e != cudaSuccess) return 400 + (int)e;
      attr2_set = true;
    }
    dim3 grid2(a->Hq * a->B, (a->Sq + 2 * BQ - 1) / (2 * BQ));
    attn_fwd2_kernel<<<grid2, 320, SMEM2, (cudaStream_t)stream>>>(tmQ, tmK.m[0], tmV.m[0], p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 500 + (int)e;
  }
  constexpr int NS = 2;   // softmax threads per row
  constexpr int SMEM = (1 + F_KST + F_VST) * TILE_BYTES + 8 * FB_COUNT + 8 + 16 + 2 * NS * 128 * 4 + 16;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  dim3 grid(a->Hq * a->B, (a->Sq + BQ - 1) / BQ);
  attn_fwd_kernel<NS><<<grid, nthreads(NS), SMEM, (cudaStream_t)stream>>>(tmQ, tmK, tmV, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}

// ====================================================================================== backward
// Two kernels, neither needs atomics and each only *reads* remote tensors, so with a sharded sequence
// they pull the peers' tiles over NVLink exactly like the forward:
//   dQ  kernel: one CTA per (Q block, head, batch) loops over the visible KV blocks of every source:
//               S = Q K^T, dP = dO V^T, dS = P o (dP - delta), dQ += dS K  (dQ stays in TMEM).
//   dKV kernel: one CTA per (local KV block, kv head, batch) loops over every query head of the group
//               and every visible Q block of every source, on the transposed problem so that the
//               operands land in TMEM lanes the way the next MMA wants them:
//               S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q  (dV, dK stay in TMEM).
// P and dS never leave tensor memory: they are written as bf16 over the S / dP columns they were
// computed from and consumed as TMEM A operands.
namespace {

constexpr int KID_ATTN_DQ = 31, KID_ATTN_DKV = 32;
constexpr float LOG2E = 1.4426950408889634f;

struct PtrList {
  const float* p[MAX_SRC];
};

struct BwdParams {
  SrcFlags fl;                     // arrival flags of the looped sources
  PushArgs push;                   // dQ kernel: this rank's K|V shard, pushed by the kernel's first CTAs
  int B, Sq, Hq, Hkv, causal;      // Sq: rows of the (local or per-source) Q tensor
  int lse_H;                       // heads of the lse / delta arrays (>= Hq for a head slice)
  float scale, scale_log2;
  int n_src, src_blocks, src_len;  // sources of the *looped* operand (KV for dQ, Q/dO for dKV)
  const int* q_blk_pos; const int* k_blk_pos; int q_off;
  // dQ kernel
  const float* lse; const float* delta;         // local [B, Hq, Sq]
  __nv_bfloat16* dQ; long long dq_sb, dq_ss, dq_sh;
  // dKV kernel
  PtrList lse_src, delta_src;                   // per Q source [B, Hq, src_len]
  int Sk;                                       // local KV rows
  __nv_bfloat16* dK; __nv_bfloat16* dV; long long dk_sb, dk_ss, dk_sh;
};

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_ss, long long o_sh,
                                  const __nv_bfloat16* __restrict__ d_o, long long d_sb, long long d_ss, long long d_sh,
                                  float* __restrict__ delta, int B, int S, int H) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= B * S * H) return;
  const int h = w % H, s = (w / H) % S, b = w / (H * S);
  const uint2 a = *reinterpret_cast<const uint2*>(o + (size_t)b * o_sb + (size_t)s * o_ss + (size_t)h * o_sh + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + (size_t)b * d_sb + (size_t)s * d_ss + (size_t)h * d_sh + lane * 4);
  const float2 a0 = np::unpack_bf16(a.x), a1 = np::unpack_bf16(a.y), g0 = np::unpack_bf16(g.x), g1 = np::unpack_bf16(g.y);
  float v = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
  v = np::warp_sum(v);
  if (lane == 0) delta[((size_t)b * H + h) * S + s] = v;
}

enum { QB_QDO = 0, QB_K = 1, QB_KE = 4, QB_V = 7, QB_VE = 9, QB_S = 11, QB_DP = 13, QB_DS = 14, QB_FIN = 15, QB_COUNT = 16 };
// K tiles live from S = Q K^T (issued one block ahead) to dQ += dS K: three of them; V tiles only feed dP: two.
constexpr int Q_KST = 3, Q_VST = 2;
constexpr int BWD_TILES = 7;   // seven 32 KB tiles: the dynamic shared memory must itself start on a 1024-byte boundary

template <int NS>
__global__ void __launch_bounds__(nthreads(NS), 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ TmapList tmK, const __grid_constant__ TmapList tmV, const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_al[];
  const uint32_t base = np::smem_u32(smem_al);
  if (base & 1023u) {   // the swizzled tiles need it; nothing has been allocated or started yet
    if (threadIdx.x == 0) np::report(NP_ERR_BAD_ARG, KID_ATTN_DQ, (int)(base & 1023u));
    return;
  }
  const uint32_t sQ = base, sdO = base + TILE_BYTES, sK0 = sdO + TILE_BYTES, sV0 = sK0 + Q_KST * TILE_BYTES;
  const uint32_t bar = sV0 + Q_VST * TILE_BYTES;
  auto B_ = [&](int i) { return bar + 8u * i; };
  uint8_t* tail = smem_al + BWD_TILES * TILE_BYTES + 8 * QB_COUNT;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Sq + BQ - 1) / BQ;
  const int qb = nqb - 1 - (int)blockIdx.y;   // heaviest first across the whole grid, as in the forward
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q_pos0 = p.q_blk_pos ? p.q_blk_pos[qb] : qb * BQ + p.q_off;
  const int total_blocks = p.n_src * p.src_blocks;
  auto k_pos0 = [&](int j) { return p.k_blk_pos ? p.k_blk_pos[j] : (j % p.src_blocks) * BKV; };
  auto next_vis = [&](int j) {   // next KV block that causality does not hide from every row of this Q block
    while (j < total_blocks && p.causal && k_pos0(j) > q_pos0 + BQ - 1) ++j;
    return j;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < QB_COUNT; ++i) np::mbar_init(B_(i), i == QB_DS ? 4 * NS : 1);
    *abort_flag = 0;
    np::mbar_fence_init();
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), 512);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;
  const uint32_t tdP = tmem + 256, tdQ = tmem + 384;   // S buffers at columns 0 and 128
  push_kv(p.push, reinterpret_cast<volatile int*>(tail + 12));

  if (warp == 0) {
    if (lane == 0) {
      if (!own_ready(p.fl, KID_ATTN_DQ)) *abort_flag = 1;
      np::mbar_expect_tx(B_(QB_QDO), 2 * TILE_BYTES);
      load_tile(sQ, &tmQ, B_(QB_QDO), h, qb * BQ, b);
      load_tile(sdO, &tmdO, B_(QB_QDO), h, qb * BQ, b);
      int i = 0, last_src = -1;
      for (int j = next_vis(0); j < total_blocks && !*abort_flag; j = next_vis(j + 1), ++i) {
        const int ks = i % Q_KST, vs = i % Q_VST;
        const int src = j / p.src_blocks, jb = j - src * p.src_blocks;
        if (src != last_src) {
          if (!src_ready(p.fl, src, KID_ATTN_DQ)) { *abort_flag = 1; break; }
          last_src = src;
        }
        if (!np::mbar_wait(B_(QB_KE + ks), ((uint32_t)(i / Q_KST) & 1u) ^ 1u, abort_flag, KID_ATTN_DQ, 1)) break;
        np::mbar_expect_tx(B_(QB_K + ks), TILE_BYTES);
        load_tile(sK0 + ks * TILE_BYTES, &tmK.m[src], B_(QB_K + ks), hkv, jb * BKV, b);
        if (!np::mbar_wait(B_(QB_VE + vs), ((uint32_t)(i / Q_VST) & 1u) ^ 1u, abort_flag, KID_ATTN_DQ, 10)) break;
        np::mbar_expect_tx(B_(QB_V + vs), TILE_BYTES);
        load_tile(sV0 + vs * TILE_BYTES, &tmV.m[src], B_(QB_V + vs), hkv, jb * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_kk = np::make_idesc(128, 128, 1, 1, 0, 0);   // both operands K-major (over hd)
      const uint32_t idesc_mn = np::make_idesc(128, 128, 1, 1, 0, 1);   // A from TMEM, B MN-major
      bool ok = np::mbar_wait(B_(QB_QDO), 0, abort_flag, KID_ATTN_DQ, 2);
      auto issue_s = [&](int i) {
        const int st = i & 1, ks = i % Q_KST;
        if (!np::mbar_wait(B_(QB_K + ks), (uint32_t)(i / Q_KST) & 1u, abort_flag, KID_ATTN_DQ, 3)) return false;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tmem + st * 128, desc_kmajor(sQ, kk), desc_kmajor(sK0 + ks * TILE_BYTES, kk), idesc_kk, kk > 0);
        np::tc_commit(B_(QB_S + st));
        return true;
      };
      auto issue_dp = [&](int i) {
        const int vs = i % Q_VST;
        if (!np::mbar_wait(B_(QB_V + vs), (uint32_t)(i / Q_VST) & 1u, abort_flag, KID_ATTN_DQ, 4)) return false;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tdP, desc_kmajor(sdO, kk), desc_kmajor(sV0 + vs * TILE_BYTES, kk), idesc_kk, kk > 0);
        np::tc_commit(B_(QB_DP));
        np::tc_commit(B_(QB_VE + vs));
        return true;
      };
      int j = next_vis(0);
      if (ok && j < total_blocks) ok = issue_s(0) && issue_dp(0);
      for (int i = 0; j < total_blocks && ok && !*abort_flag; ++i) {
        const int ks = i % Q_KST;
        j = next_vis(j + 1);
        if (j < total_blocks) ok = issue_s(i + 1);   // its buffer was read for block i-1 before dS of block i-1 arrived
        ok = ok && np::mbar_wait(B_(QB_DS), (uint32_t)i & 1u, abort_flag, KID_ATTN_DQ, 5);
        if (!ok) break;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16_ts(tdQ, tdP + kk * 8, desc_mnmajor(sK0 + ks * TILE_BYTES, kk), idesc_mn, (i > 0) || (kk > 0));
        np::tc_commit(B_(QB_KE + ks));
        if (j < total_blocks) ok = issue_dp(i + 1);  // overwrites dS after the dQ product above has consumed it
      }
      np::tc_commit(B_(QB_FIN));
    }
  } else {
    constexpr int CW = 128 / NS;
    const int quarter = warp & 3, hf = (warp - 2) >> 2;     // this thread: row r, KV columns [CW hf, CW hf + CW)
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int row = qb * BQ + r;
    const int q_pos = q_pos0 + r;
    float lse2 = INFINITY, dlt = 0.f;
    bool ok = own_ready(p.fl, KID_ATTN_DQ);   // lse / delta belong to the same arriving shard as Q / dO
    if (!ok) *abort_flag = 1;
    if (row < p.Sq) {
      const size_t idx = ((size_t)b * p.lse_H + h) * p.Sq + row;
      const float l = p.lse[idx];
      lse2 = (l == -INFINITY) ? INFINITY : l * LOG2E;
      dlt = p.delta[idx];
    }
    int nvis = 0;
    for (int j = next_vis(0); j < total_blocks; j = next_vis(j + 1), ++nvis) {
      const int i = nvis, st = i & 1;
      const int jb = j % p.src_blocks;
      const int kp0 = k_pos0(j);
      const int valid_cols = p.src_len - jb * BKV;
      const bool need_mask = (p.causal && kp0 + BKV - 1 > q_pos0) || valid_cols < BKV;
      ok = ok && !*abort_flag && warp_wait(B_(QB_S + st), (uint32_t)(i >> 1) & 1u, abort_flag, KID_ATTN_DQ, 7);
      float pr[CW];
      uint32_t t[CW];
      if (ok) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tmem + st * 128 + lane_off + hf * CW, t);
#pragma unroll
        for (int e = 0; e < CW; ++e) pr[e] = ex2(fmaf(__uint_as_float(t[e]), p.scale_log2, -lse2));
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < CW; ++e) {
            const int col = hf * CW + e;
            if (col >= valid_cols || (p.causal && kp0 + col > q_pos)) pr[e] = 0.f;
          }
        }
        ok = warp_wait(B_(QB_DP), (uint32_t)i & 1u, abort_flag, KID_ATTN_DQ, 8);
      }
      if (ok) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tdP + lane_off + hf * CW, t);
      }
      row_sync<NS>(quarter);   // both threads of the row hold their dP values: dS may now overwrite those columns
      if (ok) {
        uint32_t pk[CW / 2];
#pragma unroll
        for (int e = 0; e < CW; e += 2)
          pk[e >> 1] = np::pack_bf16(pr[e] * (__uint_as_float(t[e]) - dlt), pr[e + 1] * (__uint_as_float(t[e + 1]) - dlt));
        tmem_st_cols<CW / 2>(tdP + lane_off + hf * (CW / 2), pk);
        tmem_st_wait();
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(B_(QB_DS));
      }
    }
    ok = __all_sync(0xffffffffu, ok && !*abort_flag) && warp_wait(B_(QB_FIN), 0, abort_flag, KID_ATTN_DQ, 9);
    if (ok) {   // warp-uniform: the tensor-memory loads are executed by whole warps, only the stores are guarded
      uint32_t t[CW];
      if (nvis > 0) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tdQ + lane_off + hf * CW, t);
      } else {
#pragma unroll
        for (int e = 0; e < CW; ++e) t[e] = 0u;
      }
      if (row < p.Sq) {
        __nv_bfloat16* dst = p.dQ + (size_t)b * p.dq_sb + (size_t)row * p.dq_ss + (size_t)h * p.dq_sh + hf * CW;
#pragma unroll
        for (int g = 0; g < CW / 8; ++g) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(t[8 * g + e]) * p.scale;
          reinterpret_cast<uint4*>(dst)[g] = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                                        np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
        }
      }
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem, 512);
  }
}

enum { KB_KV = 0, KB_Q = 1, KB_QE = 4, KB_DO = 7, KB_DOE = 9, KB_ST = 11, KB_DPT = 12, KB_P = 13, KB_DS = 14, KB_FIN = 15,
       KB_COUNT = 16 };
// Q tiles live from S^T = K Q^T (issued one block ahead) to dK += dS^T Q: three of them; dO tiles are done after
// dV += P^T dO: two.
constexpr int K_QST = 3, K_DOST = 2;

template <int NS>
__global__ void __launch_bounds__(nthreads(NS), 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ TmapList tmQ, const __grid_constant__ TmapList tmdO, const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_al[];
  const uint32_t base = np::smem_u32(smem_al);
  if (base & 1023u) {   // the swizzled tiles need it; nothing has been allocated or started yet
    if (threadIdx.x == 0) np::report(NP_ERR_BAD_ARG, KID_ATTN_DKV, (int)(base & 1023u));
    return;
  }
  const uint32_t sK = base, sV = base + TILE_BYTES, sQ0 = sV + TILE_BYTES, sdO0 = sQ0 + K_QST * TILE_BYTES;
  const uint32_t bar = sdO0 + K_DOST * TILE_BYTES;
  auto B_ = [&](int i) { return bar + 8u * i; };
  uint8_t* tail = smem_al + BWD_TILES * TILE_BYTES + 8 * KB_COUNT;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);
  float* s_lse = reinterpret_cast<float*>(tail + 16);          // [2][128]
  float* s_dlt = s_lse + 256;                                   // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid.x over (kv head, batch), grid.y over KV blocks: the first KV block is seen by the most Q blocks
  const int jb = blockIdx.y, hkv = blockIdx.x % p.Hkv, b = blockIdx.x / p.Hkv;
  const int n_rep = p.Hq / p.Hkv;
  const int k_pos0 = p.k_blk_pos ? p.k_blk_pos[jb] : jb * BKV;
  auto q_pos0_of = [&](int src, int i) {
    return p.q_blk_pos ? p.q_blk_pos[src * p.src_blocks + i] : i * BQ + p.q_off;
  };

  // Work list, walked identically by every role: candidate c = (source, head of the group, Q block), kept when
  // causality lets at least one row of the Q block see this KV block.
  const int total = p.n_src * n_rep * p.src_blocks;
  auto next_vis = [&](int c) {
    while (c < total && p.causal) {
      const int i = c % p.src_blocks, src = c / (p.src_blocks * n_rep);
      if (k_pos0 <= q_pos0_of(src, i) + BQ - 1) break;
      ++c;
    }
    return c;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < KB_COUNT; ++i) np::mbar_init(B_(i), (i == KB_P || i == KB_DS) ? 4 * NS : 1);
    *abort_flag = 0;
    np::mbar_fence_init();
  }
  if (warp == 1) {
    np::tmem_alloc(np::smem_u32((const void*)tmem_ptr_smem), 512);
    np::tmem_relinquish();
  }
  np::tc_fence_before();
  __syncthreads();
  np::tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;
  const uint32_t tSt = tmem, tdPt = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      if (!own_ready(p.fl, KID_ATTN_DKV)) *abort_flag = 1;
      np::mbar_expect_tx(B_(KB_KV), 2 * TILE_BYTES);
      load_tile(sK, &tmK, B_(KB_KV), hkv, jb * BKV, b);
      load_tile(sV, &tmV, B_(KB_KV), hkv, jb * BKV, b);
      int i = 0, last_src = -1;
      for (int c = next_vis(0); c < total && !*abort_flag; c = next_vis(c + 1), ++i) {
        const int qs = i % K_QST, ds = i % K_DOST;
        const int qi = c % p.src_blocks, h = hkv * n_rep + (c / p.src_blocks) % n_rep, src = c / (p.src_blocks * n_rep);
        if (src != last_src) {
          if (!src_ready(p.fl, src, KID_ATTN_DKV)) { *abort_flag = 1; break; }
          last_src = src;
        }
        if (!np::mbar_wait(B_(KB_QE + qs), ((uint32_t)(i / K_QST) & 1u) ^ 1u, abort_flag, KID_ATTN_DKV, 1)) break;
        np::mbar_expect_tx(B_(KB_Q + qs), TILE_BYTES);
        load_tile(sQ0 + qs * TILE_BYTES, &tmQ.m[src], B_(KB_Q + qs), h, qi * BQ, b);
        if (!np::mbar_wait(B_(KB_DOE + ds), ((uint32_t)(i / K_DOST) & 1u) ^ 1u, abort_flag, KID_ATTN_DKV, 2)) break;
        np::mbar_expect_tx(B_(KB_DO + ds), TILE_BYTES);
        load_tile(sdO0 + ds * TILE_BYTES, &tmdO.m[src], B_(KB_DO + ds), h, qi * BQ, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_kk = np::make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t idesc_mn = np::make_idesc(128, 128, 1, 1, 0, 1);
      bool ok = np::mbar_wait(B_(KB_KV), 0, abort_flag, KID_ATTN_DKV, 3);
      auto issue_st = [&](int i) {
        const int qs = i % K_QST;
        if (!np::mbar_wait(B_(KB_Q + qs), (uint32_t)(i / K_QST) & 1u, abort_flag, KID_ATTN_DKV, 4)) return false;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tSt, desc_kmajor(sK, kk), desc_kmajor(sQ0 + qs * TILE_BYTES, kk), idesc_kk, kk > 0);
        np::tc_commit(B_(KB_ST));
        return true;
      };
      auto issue_dpt = [&](int i) {
        const int ds = i % K_DOST;
        if (!np::mbar_wait(B_(KB_DO + ds), (uint32_t)(i / K_DOST) & 1u, abort_flag, KID_ATTN_DKV, 5)) return false;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          np::tc_mma_f16(tdPt, desc_kmajor(sV, kk), desc_kmajor(sdO0 + ds * TILE_BYTES, kk), idesc_kk, kk > 0);
        np::tc_commit(B_(KB_DPT));
        return true;
      };
      int c = next_vis(0);
      if (ok && c < total) ok = issue_st(0) && issue_dpt(0);
      for (int i = 0; c < total && ok && !*abort_flag; ++i) {
        const int qs = i % K_QST, ds = i % K_DOST;
        c = next_vis(c + 1);
        ok = np::mbar_wait(B_(KB_P), (uint32_t)i & 1u, abort_flag, KID_ATTN_DKV, 6);
        if (!ok) break;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)   // dV += P^T dO
          tc_mma_f16_ts(tdV, tSt + kk * 8, desc_mnmajor(sdO0 + ds * TILE_BYTES, kk), idesc_mn, (i > 0) || (kk > 0));
        np::tc_commit(B_(KB_DOE + ds));
        if (c < total) ok = issue_st(i + 1);        // overwrites P^T after the product above consumed it
        ok = ok && np::mbar_wait(B_(KB_DS), (uint32_t)i & 1u, abort_flag, KID_ATTN_DKV, 7);
        if (!ok) break;
        np::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)   // dK += dS^T Q
          tc_mma_f16_ts(tdK, tdPt + kk * 8, desc_mnmajor(sQ0 + qs * TILE_BYTES, kk), idesc_mn, (i > 0) || (kk > 0));
        np::tc_commit(B_(KB_QE + qs));
        if (c < total) ok = issue_dpt(i + 1);       // overwrites dS^T after the product above consumed it
      }
      np::tc_commit(B_(KB_FIN));
    }
  } else {
    constexpr int CW = 128 / NS;
    const int quarter = warp & 3, hf = (warp - 2) >> 2;   // this thread: KV row r, Q columns [CW hf, CW hf + CW)
    const int r = quarter * 32 + lane;
    const int t256 = threadIdx.x - 64;                    // index among the softmax threads
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int k_pos = k_pos0 + r;
    bool ok = true;
    int nvis = 0, last_src = -1;
    // every thread runs every iteration: the named barriers need all of them
    for (int c = next_vis(0); c < total; c = next_vis(c + 1), ++nvis) {
      const int i = nvis, st = i & 1;
      const int qi = c % p.src_blocks, h = hkv * n_rep + (c / p.src_blocks) % n_rep, src = c / (p.src_blocks * n_rep);
      const int q_pos0 = q_pos0_of(src, qi);
      if (src != last_src) {   // lse / delta of a source are read below: it has to be complete
        if (ok && !src_ready(p.fl, src, KID_ATTN_DKV)) { *abort_flag = 1; ok = false; }
        last_src = src;
      }
      {  // stage this Q block's log-sum-exp (threads 0-127) and delta (threads 128-255), one column each
        const int qrow = qi * BQ + (t256 & 127);
        float val = (t256 < 128) ? INFINITY : 0.f;
        if (qrow < p.src_len && t256 < 256) {
          const size_t idx = ((size_t)b * p.lse_H + h) * p.src_len + qrow;
          if (t256 < 128) {
            const float l = p.lse_src.p[src][idx];
            val = (l == -INFINITY) ? INFINITY : l * LOG2E;
          } else {
            val = p.delta_src.p[src][idx];
          }
        }
        if (t256 < 256) (t256 < 128 ? s_lse : s_dlt)[st * 128 + (t256 & 127)] = val;
        softmax_sync_all<NS>();
      }
      const bool need_mask = p.causal && k_pos0 + BKV - 1 > q_pos0;
      ok = ok && !*abort_flag && warp_wait(B_(KB_ST), (uint32_t)i & 1u, abort_flag, KID_ATTN_DKV, 8);
      float pr[CW];
      uint32_t t[CW], pk[CW / 2];
      if (ok) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tSt + lane_off + hf * CW, t);
#pragma unroll
        for (int e = 0; e < CW; e += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(&s_lse[st * 128 + hf * CW + e]);
          pr[e] = ex2(fmaf(__uint_as_float(t[e]), p.scale_log2, -l4.x));
          pr[e + 1] = ex2(fmaf(__uint_as_float(t[e + 1]), p.scale_log2, -l4.y));
          pr[e + 2] = ex2(fmaf(__uint_as_float(t[e + 2]), p.scale_log2, -l4.z));
          pr[e + 3] = ex2(fmaf(__uint_as_float(t[e + 3]), p.scale_log2, -l4.w));
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < CW; ++e)
            if (k_pos > q_pos0 + hf * CW + e) pr[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < CW; e += 2) pk[e >> 1] = np::pack_bf16(pr[e], pr[e + 1]);
      }
      row_sync<NS>(quarter);   // both threads of the row hold their S^T values: P^T may now overwrite those columns
      if (ok) {
        tmem_st_cols<CW / 2>(tSt + lane_off + hf * (CW / 2), pk);
        tmem_st_wait();
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(B_(KB_P));
        ok = warp_wait(B_(KB_DPT), (uint32_t)i & 1u, abort_flag, KID_ATTN_DKV, 9);
      }
      if (ok) {
        np::tc_fence_after();
        tmem_ld_cols<CW>(tdPt + lane_off + hf * CW, t);
#pragma unroll
        for (int e = 0; e < CW; e += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(&s_dlt[st * 128 + hf * CW + e]);
          pk[e >> 1] = np::pack_bf16(pr[e] * (__uint_as_float(t[e]) - d4.x), pr[e + 1] * (__uint_as_float(t[e + 1]) - d4.y));
          pk[(e >> 1) + 1] =
              np::pack_bf16(pr[e + 2] * (__uint_as_float(t[e + 2]) - d4.z), pr[e + 3] * (__uint_as_float(t[e + 3]) - d4.w));
        }
      }
      row_sync<NS>(quarter);   // same for dP^T -> dS^T
      if (ok) {
        tmem_st_cols<CW / 2>(tdPt + lane_off + hf * (CW / 2), pk);
        tmem_st_wait();
        np::tc_fence_before();
        __syncwarp();
        if (lane == 0) np::mbar_arrive(B_(KB_DS));
      }
    }
    ok = __all_sync(0xffffffffu, ok && !*abort_flag) && warp_wait(B_(KB_FIN), 0, abort_flag, KID_ATTN_DKV, 10);
    const int row = jb * BKV + r;
    if (ok) {   // warp-uniform; only the stores are guarded by the row bound
      np::tc_fence_after();
      const size_t off = (size_t)b * p.dk_sb + (size_t)row * p.dk_ss + (size_t)hkv * p.dk_sh + hf * CW;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which ? p.dK : p.dV) + off;
        const float mul = which ? p.scale : 1.f;
        uint32_t t[CW];
        if (nvis > 0) {
          tmem_ld_cols<CW>((which ? tdK : tdV) + lane_off + hf * CW, t);
        } else {
#pragma unroll
          for (int e = 0; e < CW; ++e) t[e] = 0u;
        }
        if (row < p.Sk) {
#pragma unroll
          for (int g = 0; g < CW / 8; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(t[8 * g + e]) * mul;
            reinterpret_cast<uint4*>(dst)[g] = make_uint4(np::pack_bf16(f[0], f[1]), np::pack_bf16(f[2], f[3]),
                                                          np::pack_bf16(f[4], f[5]), np::pack_bf16(f[6], f[7]));
          }
        }
      }
    }
  }
  np::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    np::tc_fence_after();
    np::tmem_dealloc(tmem, 512);
  }
}

}  // namespace

// Backward of np_attn_fwd. q / o / d_o / dq are local [B, Sq, Hq, 128]; k / v / dk / dv local
// [B, Sk, Hkv, 128]. kv sources (for dQ) and q / d_o / lse / delta sources (for dK, dV) are lists so a
// context-parallel rank reads its peers' tensors in place; without context parallelism both lists have
// one entry, the local tensors. delta = rowsum(dO o O) is computed here into `delta` ([B, Hq, Sq] fp32).
// phase: 1 = delta only, 2 = dQ + dKV only (delta already published), 3 = all.
struct NpAttnBwdArgs {
  const void* q; long long q_sb, q_ss, q_sh;
  const void* k; const void* v; long long k_sb, k_ss, k_sh;
  const void* o; long long o_sb, o_ss, o_sh;
  const void* d_o; long long do_sb, do_ss, do_sh;
  const float* lse; float* delta;
  void* dq; long long dq_sb, dq_ss, dq_sh;
  void* dk; void* dv; long long dk_sb, dk_ss, dk_sh;
  const void* const* k_src; const void* const* v_src;           // n_src KV sources (layout of k)
  const void* const* q_src; const void* const* do_src;          // n_src Q / dO sources (layouts of q / d_o)
  const float* const* lse_src; const float* const* delta_src;   // n_src [B, Hq, Sq] sources
  int B, Sq, Sk, Hq, Hkv, causal, n_src, q_off, phase;
  float scale;
  const int* q_blk_pos_local; const int* k_blk_pos_all;         // for dQ: local Q blocks vs all KV blocks
  const int* k_blk_pos_local; const int* q_blk_pos_all;         // for dKV: local KV blocks vs all Q blocks
  int split;                                                    // softmax threads per row: 2 (default) or 4
  int lse_heads;                                                // heads of the lse / delta arrays (0: Hq)
  // sources still arriving (as in NpAttnFwdArgs); which = 1: the flags guard the KV sources of the dQ kernel,
  // 2: the Q / dO / lse / delta sources of the dK/dV kernel, 3: both
  const int* src_flags; const int* flag_idx; int flag_epoch; const int* epoch_base; unsigned long long flag_limit_ns;
  int flag_which;
  int skip;       // 1: no dQ kernel, 2: no dK/dV kernel
  int flag_own;   // 1 + flag index that guards the resident operands (q, d_o, lse, delta / k, v), 0: none
  // K|V shard pushed by the dQ kernel itself (as in NpAttnFwdArgs)
  const void* push_k; const void* push_v; long long push_bytes; void* const* push_dst; int* const* push_flag;
  int push_n; int* push_ctr;
};

NP_API int np_attn_bwd(const NpAttnBwdArgs* a, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->B <= 0 || a->Sq <= 0 || a->Sk <= 0) return 0;
  if (a->n_src < 1 || a->n_src > MAX_SRC || a->Hq % a->Hkv) return 1;
  if (!bind_ctx()) return 2;
  if (a->phase & 1) {
    const long long warps = (long long)a->B * a->Sq * a->Hq;
    attn_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)a->o, a->o_sb, a->o_ss, a->o_sh, (const __nv_bfloat16*)a->d_o, a->do_sb, a->do_ss, a->do_sh,
        a->delta, a->B, a->Sq, a->Hq);
  }
  if (!(a->phase & 2)) return cudaGetLastError() == cudaSuccess ? 0 : 500;
  const int qblocks = (a->Sq + BQ - 1) / BQ, kblocks = (a->Sk + BKV - 1) / BKV;
  CUtensorMap tmQ, tmdO, tmK, tmV;
  TmapList lK, lV, lQ, ldO;
  int rc = make_tmap_4d(&tmQ, a->q, a->B, a->Sq, a->Hq, a->q_sb, a->q_ss, a->q_sh);
  rc = rc ? rc : make_tmap_4d(&tmdO, a->d_o, a->B, a->Sq, a->Hq, a->do_sb, a->do_ss, a->do_sh);
  rc = rc ? rc : make_tmap_4d(&tmK, a->k, a->B, a->Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
  rc = rc ? rc : make_tmap_4d(&tmV, a->v, a->B, a->Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
  for (int s = 0; s < a->n_src && !rc; ++s) {
    rc = make_tmap_4d(&lK.m[s], a->k_src[s], a->B, a->Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
    rc = rc ? rc : make_tmap_4d(&lV.m[s], a->v_src[s], a->B, a->Sk, a->Hkv, a->k_sb, a->k_ss, a->k_sh);
    rc = rc ? rc : make_tmap_4d(&lQ.m[s], a->q_src[s], a->B, a->Sq, a->Hq, a->q_sb, a->q_ss, a->q_sh);
    rc = rc ? rc : make_tmap_4d(&ldO.m[s], a->do_src[s], a->B, a->Sq, a->Hq, a->do_sb, a->do_ss, a->do_sh);
  }
  if (rc) return 100 + rc;
  for (int s = a->n_src; s < MAX_SRC; ++s) { lK.m[s] = lK.m[0]; lV.m[s] = lV.m[0]; lQ.m[s] = lQ.m[0]; ldO.m[s] = ldO.m[0]; }
  BwdParams p{};
  p.B = a->B; p.Sq = a->Sq; p.Hq = a->Hq; p.Hkv = a->Hkv; p.causal = a->causal;
  p.lse_H = a->lse_heads > 0 ? a->lse_heads : a->Hq;
  p.scale = a->scale; p.scale_log2 = a->scale * LOG2E;
  p.n_src = a->n_src; p.q_off = a->q_off;
  p.lse = a->lse; p.delta = a->delta;
  p.dQ = (__nv_bfloat16*)a->dq; p.dq_sb = a->dq_sb; p.dq_ss = a->dq_ss; p.dq_sh = a->dq_sh;
  p.Sk = a->Sk; p.dK = (__nv_bfloat16*)a->dk; p.dV = (__nv_bfloat16*)a->dv;
  p.dk_sb = a->dk_sb; p.dk_ss = a->dk_ss; p.dk_sh = a->dk_sh;
  for (int s = 0; s < MAX_SRC; ++s) {
    p.lse_src.p[s] = a->lse_src[s < a->n_src ? s : 0];
    p.delta_src.p[s] = a->delta_src[s < a->n_src ? s : 0];
  }
  constexpr int SMEM_DQ = BWD_TILES * TILE_BYTES + 8 * QB_COUNT + 16 + 16;
  constexpr int SMEM_DKV = BWD_TILES * TILE_BYTES + 8 * KB_COUNT + 16 + 2048 + 16;
  static_assert(SMEM_DKV <= 227 * 1024, "shared memory budget");
  static NpPerDeviceOnce attr_once;
  bool& attr_set = *attr_once.slot();
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DQ);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_dq_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DQ);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DKV);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DKV);
    if (e != cudaSuccess) return 400 + (int)e;
    attr_set = true;
  }
  // dQ: local Q blocks against every source's KV blocks
  BwdParams pq = p;
  pq.src_blocks = kblocks; pq.src_len = a->Sk;
  pq.q_blk_pos = a->q_blk_pos_local; pq.k_blk_pos = a->k_blk_pos_all;
  fill_flags(&pq.fl, (a->flag_which & 1) ? a->src_flags : nullptr, a->flag_idx, a->n_src, a->flag_epoch, a->epoch_base,
             a->flag_limit_ns, a->flag_own - 1);
  if (fill_push(&pq.push, a)) return 1;
  // dK, dV: local KV blocks against every source's Q blocks
  BwdParams pk = p;
  pk.src_blocks = qblocks; pk.src_len = a->Sq;
  pk.q_blk_pos = a->q_blk_pos_all; pk.k_blk_pos = a->k_blk_pos_local;
  fill_flags(&pk.fl, (a->flag_which & 2) ? a->src_flags : nullptr, a->flag_idx, a->n_src, a->flag_epoch, a->epoch_base,
             a->flag_limit_ns, a->flag_own - 1);
  const dim3 gq(a->Hq * a->B, qblocks), gk(a->Hkv * a->B, kblocks);
  if (a->split == 4) {
    if (!(a->skip & 1)) attn_bwd_dq_kernel<4><<<gq, nthreads(4), SMEM_DQ, stream>>>(tmQ, tmdO, lK, lV, pq);
    if (!(a->skip & 2)) attn_bwd_dkv_kernel<4><<<gk, nthreads(4), SMEM_DKV, stream>>>(tmK, tmV, lQ, ldO, pk);
  } else {
    if (!(a->skip & 1)) attn_bwd_dq_kernel<2><<<gq, nthreads(2), SMEM_DQ, stream>>>(tmQ, tmdO, lK, lV, pq);
    if (!(a->skip & 2)) attn_bwd_dkv_kernel<2><<<gk, nthreads(2), SMEM_DKV, stream>>>(tmK, tmV, lQ, ldO, pk);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 500 + (int)e;
}
