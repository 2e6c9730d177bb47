// Prefill attention forward for sm_100a: dense causal / non-causal varlen GQA and
// the reference's window sparsity (local sliding window + global prefix).
// Stands in for flash_attn_fwd_kernel (flash_attn_triton/flash_attn_triton.py:52-180)
// and its window twin (flash_attn_triton/flash_attn_sparse_attn_triton.py:47-234).
//
// One CTA owns 256 consecutive query rows of one (sequence, query head) as two
// 128-row tiles and walks the visible KV tiles once for both:
//
//   warp 9   TMA producer: Q_0, K_0, Q_1, then V_0, K_1, V_1, ... into a ring of
//            128-byte-swizzled shared-memory stages (mbarrier full/empty pairs)
//   warp 8   MMA issuer (one thread): S_t = Q_t K_j^T and O_t += P_t V_j with
//            tcgen05.mma; S, P and O live in tensor memory (TMEM)
//   warps 0-3 / 4-7   softmax warpgroup of tile 0 / tile 1: one thread per query
//            row reads its S row from TMEM, keeps the running max and sum in
//            registers (base-2 exponentials), writes P back over S as packed
//            16-bit values for the P V product, rescales O in TMEM only when
//            the row max has grown by more than 2^8, and writes the output (a
//            tile inside its sequence through the dead Q buffer and a TMA store).
//
// While one warpgroup computes the softmax of its tile the tensor core works on
// the other tile, so MMA and exponentials overlap.  TMEM columns: S0 [0,128),
// S1 [128,256), O0 [256,256+D), O1 [384,384+D); P_t aliases the first half of S_t.
// Every mbarrier wait is bounded; a timeout sets *status_word and the CTA drains.
#include <mutex>
#include <algorithm>
#include <climits>
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {
using namespace sm100;

constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 9;
constexpr int kPrefillThreads = 384;        // warps 10, 11 only complete the third warpgroup
constexpr int kSoftmaxRegs = 216;           // per thread, after setmaxnreg (8 warps)
constexpr int kOtherRegs = 72;              // MMA / TMA / idle warps
// setmaxnreg.inc can only take registers that setmaxnreg.dec of the same CTA
// released, so with R registers per thread at launch the budgets must satisfy
// 128 (R - kOtherRegs) >= 256 (kSoftmaxRegs - R); R = 168 is what 384 threads
// per CTA allow.  The launcher refuses to run a build whose R is smaller.
constexpr int kLaunchRegs = 168;
static_assert(128 * (kLaunchRegs - kOtherRegs) >= 256 * (kSoftmaxRegs - kLaunchRegs),
              "setmaxnreg budgets would deadlock");
constexpr int kTileM = 128;            // query rows per tile
constexpr int kPairM = 2 * kTileM;     // query rows per CTA
constexpr float kLazyRescaleLog2 = 8.f;
#ifndef B200ATTN_HEAD_GROUP
#define B200ATTN_HEAD_GROUP 8
#endif
constexpr int kHeadGroup = B200ATTN_HEAD_GROUP;   // (sequence, head) pairs scheduled together

struct PrefillParams {
  void* o;
  float* lse;
  const int32_t* cu_seqlens;
  long long o_sb, o_st, o_sh, lse_sb, lse_st, lse_sh;
  int batch, heads_q, heads_kv, group, head_dim;
  int seqlen, n_pairs;
  int pair_begin, pair_count;   // the 256-row query blocks this launch computes: [pair_begin, pair_begin + pair_count)
  int prefetch_ahead;   // CTAs resident at once: a CTA asks for the first tiles of CTA + this into L2
  int causal, window, win_local, win_global;
  float scale_log2;
  int lse_base2;
  int* status_word;
  // block-list sparsity (block size 64): null block_idx = dense / window
  const int32_t* block_idx;  // [batch, heads_q, n_qblocks, max_nnz]
  const int32_t* block_cnt;  // [batch, heads_q, n_qblocks]
  int n_qblocks, max_nnz;
};

constexpr int kBlk = 64;              // block-list granularity (tokens)
constexpr int kMaxBlocks = 2048;      // KV blocks per sequence the merged list can hold

// The ascending sequence of KV tiles a 256-row query block visits: optionally
// a global prefix range [0, g_cnt) followed by the local range starting at l_lo.
struct TileSeq {
  int n, g_cnt, l_lo;
  __device__ __forceinline__ int kv(int j) const { return j < g_cnt ? j : l_lo + (j - g_cnt); }
};

template <int BN>
__device__ __forceinline__ TileSeq make_seq(const PrefillParams& p, int q0, int len) {
  TileSeq s;
  const int q_end = min(len, q0 + kPairM);
  const int hi = ((p.causal ? q_end : len) + BN - 1) / BN;
  s.n = hi; s.g_cnt = 0; s.l_lo = 0;
  if (p.window) {
    const int lo_tok = max(0, q0 - p.win_local + 1);
    const int l_lo = min(lo_tok / BN, hi);
    const int g_hi = (min(p.win_global, q_end) + BN - 1) / BN;
    if (g_hi < l_lo) { s.g_cnt = g_hi; s.l_lo = l_lo; s.n = g_hi + (hi - l_lo); }
  }
  return s;
}

// Does query tile t (rows q0t .. q0t+127) see anything of KV tile kvt?
template <int BN>
__device__ __forceinline__ bool tile_active(const PrefillParams& p, int q0t, int len, int kvt) {
  if (q0t >= len) return false;
  const int qlast = min(len, q0t + kTileM) - 1;
  const int kv0 = kvt * BN, kvl = kv0 + BN - 1;
  if (p.causal && kv0 > qlast) return false;
  if (p.window && !(kv0 < p.win_global) && !(kvl > q0t - p.win_local)) return false;
  return true;
}

// Is some (query, key) pair of the tile pair masked?  (conservative: may say yes)
template <int BN>
__device__ __forceinline__ bool tile_needs_mask(const PrefillParams& p, int q0t, int len, int kvt) {
  const int kv0 = kvt * BN, kv_end = kv0 + BN;
  bool full = kv_end <= len;
  if (p.causal) full = full && (kv_end - 1 <= q0t);
  if (p.window) full = full && ((kv_end <= p.win_global) || (q0t + kTileM - 1 - kv0 < p.win_local));
  return !full;
}


__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// (d0, d1) = (a0, a1) * (b, b) + (c, c) in one packed instruction
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1) {
  asm("{.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}
// (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1)
__device__ __forceinline__ void ffma2v(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
// 2^x for a pair of values on the FMA pipe instead of the MUFU pipe (which does 16 per clock
// per SM and is as busy as the tensor core in this kernel): x = n + f with n = round(x),
// 2^f by a cubic on [-0.5, 0.5] (relative error 1e-4, below the 16-bit P it feeds), n added
// into the exponent field.  x <= ~9 here; x below -125, masked scores (-inf) included, gives
// 2^-125 = 2.4e-38 rather than 0: every row that reaches this code has a visible key whose
// term is at least 2^-8, so the difference is below 1e-35 relative (guarding it with a
// compare + select per value cost more than the cubic saved: 1034 instead of 1070 TFLOP/s).
__device__ __forceinline__ void exp2_fma_pair(float& e0, float& e1, float x0, float x1) {
  const float magic = 12582912.f;   // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
  x0 = fmaxf(x0, -125.f);
  x1 = fmaxf(x1, -125.f);
  float t0, t1, n0, n1, f0, f1, p0, p1;
  ffma2(t0, t1, x0, x1, 1.f, magic);
  ffma2(n0, n1, t0, t1, 1.f, -magic);
  ffma2v(f0, f1, n0, n1, -1.f, -1.f, x0, x1);
  ffma2(p0, p1, f0, f1, 0.05550357f, 0.24022652f);
  ffma2v(p0, p1, p0, p1, f0, f1, 0.69314720f, 0.69314720f);
  ffma2v(p0, p1, p0, p1, f0, f1, 1.f, 1.f);
  e0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  e1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <int DP, int BN, int NSTAGE>
struct PrefillSmem {
  static constexpr int kQBytes = kTileM * DP * 2;
  static constexpr int kQPanel = kTileM * 128;  // one 64-column swizzled panel of Q
  static constexpr int kStageBytes = BN * DP * 2;
  static constexpr int kKvPanel = BN * 128;
  static constexpr int kBarOffset = 2 * kQBytes + NSTAGE * kStageBytes;
  static constexpr int kNumBars = 2 + 2 * NSTAGE + 6;
  // block-list mode: 4 bitmaps (one per 64-row query block of the CTA), then per
  // query tile the merged ascending list of KV blocks with a 2-bit membership mask
  static constexpr int kBitmapOffset = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kUlistOffset = kBitmapOffset + 4 * (kMaxBlocks / 32) * 4;
  static constexpr int kUflagOffset = kUlistOffset + 2 * kMaxBlocks * 2;
  static constexpr int kBytes = kUflagOffset + 2 * kMaxBlocks;
  static constexpr int kAlloc = kBytes + 1024;  // slack to align the base to 1024 bytes
};

// BLK: block-list sparsity (own instantiation so the dense / window paths carry none of its branches)
template <typename T, int DP, int BN, int NSTAGE, bool BLK>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
               const PrefillParams p) {
  using L = PrefillSmem<DP, BN, NSTAGE>;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdescQK = idesc_f16(kFmt, false, kTileM, BN);
  constexpr uint32_t kIdescPV = idesc_f16(kFmt, true, kTileM, DP);
  constexpr int kPanels = DP / 64;

  // ---- which 256 query rows.  (sequence, head) pairs are taken in groups of
  // kHeadGroup: inside a group the heaviest query blocks of all its heads come
  // first (longest-first keeps the tail of the launch short), and the group is
  // small enough that its K/V stay in L2 while its CTAs are resident.
  const int n_bh = p.batch * p.heads_q;
  const int per_group = kHeadGroup * p.pair_count;
  const int grp = blockIdx.x / per_group;
  const int in_grp = blockIdx.x - grp * per_group;
  const int g_heads = min(kHeadGroup, n_bh - grp * kHeadGroup);
  const int pair = p.pair_begin + p.pair_count - 1 - in_grp / g_heads;
  const int bh = grp * kHeadGroup + in_grp % g_heads;
  const int h = bh % p.heads_q, b = bh / p.heads_q;
  const int hk = h / p.group;
  int seq_start = 0, len = p.seqlen, bcoord = b;
  if (p.cu_seqlens) {
    seq_start = p.cu_seqlens[b];
    // a sequence longer than the max_seqlen the grid was sized for is cut there
    len = min(p.cu_seqlens[b + 1] - seq_start, p.n_pairs * kPairM);
    bcoord = 0;
  }
  const int q0 = pair * kPairM;
  if (q0 >= len) return;
  const TileSeq seq = make_seq<BN>(p, q0, len);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sKV = smem_base + 2 * L::kQBytes;
  const uint32_t bars = smem_base + L::kBarOffset;
  auto q_full = [&](int t) { return bars + 8 * t; };
  auto kv_full = [&](int s) { return bars + 8 * (2 + s); };
  auto kv_empty = [&](int s) { return bars + 8 * (2 + NSTAGE + s); };
  auto s_full = [&](int t) { return bars + 8 * (2 + 2 * NSTAGE + t); };
  auto p_full = [&](int t) { return bars + 8 * (4 + 2 * NSTAGE + t); };
  auto o_full = [&](int t) { return bars + 8 * (6 + 2 * NSTAGE + t); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(q_full(t), 1);
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), kTileM);
      mbar_init(o_full(t), 1);
    }
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  auto tS = [&](int t) { return tmem + 128u * t; };
  auto tO = [&](int t) { return tmem + 256u + 128u * t; };

  // ---- block-list mode: each 128-row query tile walks the union of the lists
  // of its two 64-row query blocks, two KV blocks per 128-key step, with its own
  // K/V stream.  The union is built as a bitmap per query block, merged and
  // compacted into an ascending list with a 2-bit membership mask per entry.
  // Entries out of range, or above the diagonal when causal, are dropped here,
  // so nothing later can index out of bounds.
  constexpr bool blk = BLK;
  unsigned int* bitmap = reinterpret_cast<unsigned int*>(smem_gen + L::kBitmapOffset);
  volatile unsigned short* ulist_all = reinterpret_cast<volatile unsigned short*>(smem_gen + L::kUlistOffset);
  volatile unsigned char* uflags_all = reinterpret_cast<volatile unsigned char*>(smem_gen + L::kUflagOffset);
  volatile int* n_u_slot = reinterpret_cast<volatile int*>(smem_gen + L::kBarOffset + L::kNumBars * 8 + 8);
  auto ulist = [&](int t, int i) -> int { return (int)ulist_all[t * kMaxBlocks + i]; };
  auto uflags = [&](int t, int i) -> unsigned { return (unsigned)uflags_all[t * kMaxBlocks + i]; };
  int n_u[2] = {0, 0};
  if (blk) {
    constexpr int kWords = kMaxBlocks / 32;
    for (int i = threadIdx.x; i < 4 * kWords; i += kPrefillThreads) bitmap[i] = 0u;
    __syncthreads();
    if (warp < 4) {
      const int qb = q0 / kBlk + warp;
      if (qb < p.n_qblocks && qb * kBlk < len) {
        const long long rowi = ((long long)b * p.heads_q + h) * p.n_qblocks + qb;
        const int32_t* lst = p.block_idx + rowi * p.max_nnz;
        const int cnt = min(p.block_cnt[rowi], p.max_nnz);
        for (int i = lane; i < cnt; i += 32) {
          const int u = lst[i];
          if (u >= 0 && u < kMaxBlocks && u * kBlk < len && (!p.causal || u <= qb))
            atomicOr(&bitmap[warp * kWords + (u >> 5)], 1u << (u & 31));
        }
      }
    }
    __syncthreads();
    if (warp < 2) {
      const int t = warp;
      int base = 0;
      for (int w0 = 0; w0 < kWords; w0 += 32) {
        const int w = w0 + lane;
        const unsigned m0 = bitmap[(2 * t) * kWords + w], m1 = bitmap[(2 * t + 1) * kWords + w];
        unsigned any = m0 | m1;
        const int cnt = __popc(any);
        int incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += v;
        }
        int pos = base + incl - cnt;
        while (any) {
          const int bit = __ffs(any) - 1;
          any &= any - 1;
          ulist_all[t * kMaxBlocks + pos] = (unsigned short)(w * 32 + bit);
          uflags_all[t * kMaxBlocks + pos] = (unsigned char)(((m0 >> bit) & 1u) | (((m1 >> bit) & 1u) << 1));
          ++pos;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) n_u_slot[t] = base;
    }
    __syncthreads();
    n_u[0] = n_u_slot[0];
    n_u[1] = n_u_slot[1];
  }
  // steps of each tile in block-list mode (its own K/V stream), else of the CTA
  const int ns0 = (q0 < len) ? (n_u[0] + 1) / 2 : 0;
  const int ns1 = (q0 + kTileM < len) ? (n_u[1] + 1) / 2 : 0;
  const int n_steps = blk ? max(ns0, ns1) : seq.n;
  // does query tile t take part in step j?
  auto step_active = [&](int t, int j) -> bool {
    if (!blk) return tile_active<BN>(p, q0 + kTileM * t, len, seq.kv(j));
    return j < (t ? ns1 : ns0);
  };

  if (warp >= 8) {
    // third warpgroup: TMA producer, MMA issuer and two idle warps give registers away
    setmaxnreg_dec<kOtherRegs>();
    if (warp == kLoadWarp) {
    // ================================================================= TMA
    {
      if (elect_one()) { prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_o); }
      auto load_q = [&](int t) {
        if (q0 + kTileM * t >= len) return;
        if (elect_one()) {
          mbar_expect_tx(q_full(t), L::kQBytes);
          for (int pn = 0; pn < kPanels; ++pn)
            tma_load_4d(sQ + t * L::kQBytes + pn * L::kQPanel, &tmap_q, q_full(t), 64 * pn,
                        seq_start + q0 + kTileM * t, h, bcoord);
        }
        __syncwarp();
      };
      load_q(0);
      // The CTA that will start when one of the resident ones ends finds its Q tiles (read by
      // nobody else, so not in L2 yet) and its first K / V tile on the way: a CTA otherwise
      // spends ~2.5 us before its first product can start.  Issued behind this CTA's own
      // first loads (in front of them it delayed them: 1041 instead of 1086 TFLOP/s).
      auto prefetch_next_cta = [&]() {
        if (p.prefetch_ahead > 0 && blockIdx.x + p.prefetch_ahead < gridDim.x && elect_one()) {
          const int bi = blockIdx.x + p.prefetch_ahead;
          const int grp2 = bi / per_group, in2 = bi - grp2 * per_group;
          const int gh2 = min(kHeadGroup, n_bh - grp2 * kHeadGroup);
          const int pair2 = p.pair_begin + p.pair_count - 1 - in2 / gh2;
          const int bh2 = grp2 * kHeadGroup + in2 % gh2;
          const int h2 = bh2 % p.heads_q, b2 = bh2 / p.heads_q;
          int ss2 = 0, len2 = p.seqlen, bc2 = b2;
          if (p.cu_seqlens) { ss2 = p.cu_seqlens[b2]; len2 = min(p.cu_seqlens[b2 + 1] - ss2, p.n_pairs * kPairM); bc2 = 0; }
          const int q02 = pair2 * kPairM;
          if (q02 < len2) {
            const TileSeq seq2 = make_seq<BN>(p, q02, len2);
            for (int pn = 0; pn < kPanels; ++pn) {
              tma_prefetch_4d(&tmap_q, 64 * pn, ss2 + q02, h2, bc2);
              if (q02 + kTileM < len2) tma_prefetch_4d(&tmap_q, 64 * pn, ss2 + q02 + kTileM, h2, bc2);
              if (!blk && seq2.n > 0) {   // (block lists: the first K / V blocks are not known here)
                tma_prefetch_4d(&tmap_k, 64 * pn, ss2 + seq2.kv(0) * BN, h2 / p.group, bc2);
                tma_prefetch_4d(&tmap_v, 64 * pn, ss2 + seq2.kv(0) * BN, h2 / p.group, bc2);
              }
            }
          }
        }
        __syncwarp();
      };
      __syncwarp();
      int cnt = 0;
      // one stage: a 128-row box (dense / window) or two 64-row boxes (block list;
      // the K/V tensor maps are then built with 64-row boxes)
      auto load_stage = [&](const CUtensorMap* m, int row0, int row1, bool two) {
        const int s = cnt % NSTAGE;
        const uint32_t ph = (cnt / NSTAGE) & 1;
        mbar_wait(kv_empty(s), ph ^ 1, abort_flag);
        if (elect_one()) {
          mbar_expect_tx(kv_full(s), L::kStageBytes);
          for (int pn = 0; pn < kPanels; ++pn) {
            const uint32_t dst = sKV + s * L::kStageBytes + pn * L::kKvPanel;
            tma_load_4d(dst, m, kv_full(s), 64 * pn, row0, hk, bcoord);
            if (two) tma_load_4d(dst + kBlk * 128, m, kv_full(s), 64 * pn, row1, hk, bcoord);
          }
        }
        __syncwarp();
        ++cnt;
      };
      if (!blk) {
        // the first product needs Q of tile 0 and the first K tile: those two first, then Q of tile 1
        if (n_steps > 0) load_stage(&tmap_k, seq_start + seq.kv(0) * BN, 0, false);
        load_q(1);
        for (int j = 0; j < n_steps; ++j) {
          const int row = seq_start + seq.kv(j) * BN;
          if (j > 0) load_stage(&tmap_k, row, 0, false);
          load_stage(&tmap_v, row, 0, false);
          if (j == 1 || n_steps == 1) prefetch_next_cta();   // behind this CTA's own first loads
        }
      } else {
        load_q(1);
        // per tile its own stream, in the order the MMA warp consumes the stages:
        // K(0,0) K(1,0), then per step V(0,j) K(0,j+1) V(1,j) K(1,j+1).  An odd
        // list repeats its last block in the second box (those columns are masked).
        auto load_blk = [&](const CUtensorMap* m, int t, int j) {
          const int nu = n_u[t];
          load_stage(m, seq_start + ulist(t, 2 * j) * kBlk,
                     seq_start + ulist(t, min(2 * j + 1, nu - 1)) * kBlk, true);
        };
        if (ns0 > 0) load_blk(&tmap_k, 0, 0);
        if (ns1 > 0) load_blk(&tmap_k, 1, 0);
        for (int j = 0; j < n_steps; ++j) {
          if (j == 1 || (j == 0 && n_steps == 1)) prefetch_next_cta();
          if (j < ns0) load_blk(&tmap_v, 0, j);
          if (j + 1 < ns0) load_blk(&tmap_k, 0, j + 1);
          if (j < ns1) load_blk(&tmap_v, 1, j);
          if (j + 1 < ns1) load_blk(&tmap_k, 1, j + 1);
        }
      }
      // every issued copy must have landed before the CTA may exit
      for (int c = max(cnt - NSTAGE, 0); c < cnt; ++c)
        if (!mbar_wait(kv_full(c % NSTAGE), (c / NSTAGE) & 1, abort_flag)) mbar_drain(kv_full(c % NSTAGE), (c / NSTAGE) & 1);
    }
    } else if (warp == kMmaWarp) {
    // ================================================================= MMA
    // The whole warp walks the loop in lock step and every lane executes the
    // (predicated) MMA instructions; only `issue`'s lane really issues them, so
    // there is no divergent branch and descriptors stay warp-uniform.
    {
      const uint32_t issue = elect_one() ? 1u : 0u;
      int cnt = 0;
      int pv_cnt[2] = {0, 0};
      bool q_ready[2] = {false, false};
      // descriptors of stage 0 / tile 0; other stages and k-steps add to the address field
      const uint64_t dq0 = smem_desc_sw128(sQ, 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(sKV, 16, 1024);
      const uint64_t dv0 = smem_desc_sw128(sKV, L::kKvPanel, 1024);
      auto wait_stage = [&]() {
        const int s = cnt % NSTAGE;
        mbar_wait(kv_full(s), (cnt / NSTAGE) & 1, abort_flag);
        tc_fence_after();
        ++cnt;
        return s;
      };
      auto issue_qk = [&](int t, int s) {
        if (!q_ready[t]) { mbar_wait(q_full(t), 0, abort_flag); tc_fence_after(); q_ready[t] = true; }
        const uint64_t da = dq0 + (uint64_t)((t * L::kQBytes) >> 4);
        const uint64_t db = dk0 + (uint64_t)((s * L::kStageBytes) >> 4);
        static_assert(BN == 128, "the grouped issue assumes 16 KB panels");
        if (DP == 128)
          mma_ss_x8(tS(t), (uint32_t)da, (uint32_t)(da >> 32), (uint32_t)db, (uint32_t)(db >> 32), kIdescQK, issue);
        else
          mma_ss_x4(tS(t), (uint32_t)da, (uint32_t)(da >> 32), (uint32_t)db, (uint32_t)(db >> 32), kIdescQK, issue);
        mma_commit(s_full(t), issue);
      };
      auto issue_pv = [&](int t, int s) {
        mbar_wait(p_full(t), pv_cnt[t] & 1, abort_flag);
        tc_fence_after();
        const uint64_t db = dv0 + (uint64_t)((s * L::kStageBytes) >> 4);
        mma_ts_x8(tO(t), tS(t), (uint32_t)db, (uint32_t)(db >> 32), kIdescPV, pv_cnt[t] > 0 ? 1u : 0u, issue);
        mma_commit(o_full(t), issue);
        ++pv_cnt[t];
      };
      if (!blk) {
        // both tiles share every K/V stage
        int sK = n_steps > 0 ? wait_stage() : 0;
        for (int t = 0; t < 2; ++t)
          if (n_steps > 0 && step_active(t, 0)) issue_qk(t, sK);
        if (n_steps > 0) mma_commit(kv_empty(sK), issue);
        for (int j = 0; j < n_steps; ++j) {
          const int sV = wait_stage();
          // Rows of the V tile past the sequence end belong to the next packed sequence (or to
          // nobody): P is 0 there, but 0 * Inf/NaN would still poison O, so they are cleared
          // like the reference's zero-padded loads (flash_attn_triton.py:155-165).
          if (seq.kv(j) * BN + BN > len)
            zero_tile_rows(smem_gen + 2 * L::kQBytes + sV * L::kStageBytes, kPanels, L::kKvPanel,
                           max(len - seq.kv(j) * BN, 0), BN, lane);
          const bool more = j + 1 < n_steps;
          int sKn = 0;
          for (int t = 0; t < 2; ++t) {
            if (step_active(t, j)) issue_pv(t, sV);
            if (t == 1) mma_commit(kv_empty(sV), issue);
            if (more) {
              if (t == 0) sKn = wait_stage();
              if (step_active(t, j + 1)) issue_qk(t, sKn);
              if (t == 1) mma_commit(kv_empty(sKn), issue);
            }
          }
        }
      } else {
        // block lists: each tile consumes its own stages (same order as the loader)
        for (int t = 0; t < 2; ++t)
          if ((t ? ns1 : ns0) > 0) { const int s = wait_stage(); issue_qk(t, s); mma_commit(kv_empty(s), issue); }
        for (int j = 0; j < n_steps; ++j) {
          for (int t = 0; t < 2; ++t) {
            const int ns = t ? ns1 : ns0;
            if (j < ns) {
              const int s = wait_stage();
              // (rows past the sequence end inside the last KV block are cleared, see above)
              for (int bx = 0; bx < 2; ++bx) {
                const int u = ulist(t, min(2 * j + bx, n_u[t] - 1));
                if ((u + 1) * kBlk > len)
                  zero_tile_rows(smem_gen + 2 * L::kQBytes + s * L::kStageBytes, kPanels, L::kKvPanel,
                                 kBlk * bx + max(len - u * kBlk, 0), kBlk * (bx + 1), lane);
              }
              issue_pv(t, s);
              mma_commit(kv_empty(s), issue);
            }
            if (j + 1 < ns) { const int s = wait_stage(); issue_qk(t, s); mma_commit(kv_empty(s), issue); }
          }
        }
      }
    }
    }
  } else {
    // ============================================================= softmax
    setmaxnreg_inc<kSoftmaxRegs>();
    const int t = warp >> 2;                       // query tile of this warpgroup
    const int row = threadIdx.x & (kTileM - 1);    // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int q0t = q0 + kTileM * t;
    const int qi = q0t + row;                      // query index inside the sequence
    const float c = p.scale_log2;
    float m_run = -INFINITY;  // max the stored P / O are relative to (raw score units)
    float l_run = 0.f;
    int items = 0;
    if (q0t < len) {
      for (int j = 0; j < n_steps; ++j) {
        const int kvt = blk ? 0 : seq.kv(j);
        if (!step_active(t, j)) continue;
        mbar_wait(s_full(t), items & 1, abort_flag);
        tc_fence_after();
        uint32_t sr[BN];
#pragma unroll
        for (int cc = 0; cc < BN / 32; ++cc) tmem_ld32(tS(t) + lane_off + 32 * cc, &sr[32 * cc]);
        tmem_wait_ld();
        bool vis0 = true, vis1 = true;   // does this warp's query block see each 64-column half?
        if (blk) {
          // columns [0,64) belong to KV block u0, [64,128) to u1; a row sees a
          // prefix of each half: nothing if its query block does not list the KV
          // block, else up to the causal diagonal and the sequence end
          const int u0 = ulist(t, 2 * j);
          const bool has1 = 2 * j + 1 < n_u[t];
          const int u1 = has1 ? ulist(t, 2 * j + 1) : 0;
          const unsigned f0 = uflags(t, 2 * j), f1 = has1 ? uflags(t, 2 * j + 1) : 0u;
          const int qa = row >> 6;                 // query block inside the tile (uniform per warp)
          vis0 = (f0 >> qa) & 1u;
          vis1 = (f1 >> qa) & 1u;
          // A half this warp's query block does not list is skipped below (no maximum, no
          // exponentials, P = 0), so only a listed half that the sequence end or the causal
          // diagonal cuts for some row of this warp needs the element mask: with random lists
          // most steps hold a block of one of the two query blocks only, and none of them does.
          const int q_lo = q0t + 32 * (warp & 3);  // first query row of this warp
          const bool cut0 = vis0 && ((u0 + 1) * kBlk > len || (p.causal && (u0 + 1) * kBlk - 1 > q_lo));
          const bool cut1 = vis1 && ((u1 + 1) * kBlk > len || (p.causal && (u1 + 1) * kBlk - 1 > q_lo));
          if (cut0 || cut1) {
            int lim0 = vis0 ? min(kBlk, len - u0 * kBlk) : 0;
            int lim1 = vis1 ? min(kBlk, len - u1 * kBlk) : 0;
            if (p.causal) { lim0 = min(lim0, qi - u0 * kBlk + 1); lim1 = min(lim1, qi - u1 * kBlk + 1); }
#pragma unroll
            for (int x = 0; x < kBlk; ++x) {
              if (x >= lim0) sr[x] = 0xff800000u;  // -inf
              if (x >= lim1) sr[kBlk + x] = 0xff800000u;
            }
          }
        } else if (tile_needs_mask<BN>(p, q0t, len, kvt)) {
          // Column x of this tile is visible iff x < lim and (x >= lo or x < gl):
          // lim from the causal diagonal and the sequence end, lo from the local
          // window, gl from the global prefix.  Kept to a compare + select per
          // element: this code runs once or twice per CTA, so its size (cold
          // instruction fetches) matters more than its issue count.
          const int kv0 = kvt * BN;
          int lim = len - kv0;
          if (p.causal) lim = min(lim, qi - kv0 + 1);
          if (!p.window) {
#pragma unroll
            for (int x = 0; x < BN; ++x)
              if (x >= lim) sr[x] = 0xff800000u;  // -inf
          } else {
            const int lo = qi - p.win_local + 1 - kv0;
            const int gl = p.win_global - kv0;
#pragma unroll
            for (int x = 0; x < BN; ++x)
              if (x >= lim || (x < lo && x >= gl)) sr[x] = 0xff800000u;
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          if (hb == 0 ? vis0 : vis1) {   // (warp-uniform) an unlisted half is all -inf
#pragma unroll
            for (int x = hb * (BN / 2); x < (hb + 1) * (BN / 2); x += 8) {
              mx0 = fmax3(mx0, __uint_as_float(sr[x]), __uint_as_float(sr[x + 1]));
              mx1 = fmax3(mx1, __uint_as_float(sr[x + 2]), __uint_as_float(sr[x + 3]));
              mx2 = fmax3(mx2, __uint_as_float(sr[x + 4]), __uint_as_float(sr[x + 5]));
              mx3 = fmax3(mx3, __uint_as_float(sr[x + 6]), __uint_as_float(sr[x + 7]));
            }
          }
        }
        const float m_new = fmax3(m_run, fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // keep the stale max unless it is too far behind (first tile: always take)
        const bool grow = (items == 0) || ((m_new - m_run) * c > kLazyRescaleLog2) ||
                          (m_run == -INFINITY && m_new != -INFINITY);
        const float m_use = grow ? m_new : m_run;
        const float alpha = (m_use == m_run) ? 1.f : ex2((m_run - m_use) * c);
        if (items > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // O_t must hold every product issued so far before it is rescaled
          mbar_wait(o_full(t), (items - 1) & 1, abort_flag);
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < DP / 32; ++cc) {
            uint32_t orr[32];
            tmem_ld32(tO(t) + lane_off + 32 * cc, orr);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) orr[x] = __float_as_uint(__uint_as_float(orr[x]) * alpha);
            tmem_st32(tO(t) + lane_off + 32 * cc, orr);
          }
        }
        const float mc = (m_use == -INFINITY) ? 0.f : m_use * c;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        uint32_t pr[BN / 2];
        const float neg_mc = -mc;
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          if (hb == 0 ? vis0 : vis1) {
#pragma unroll
            for (int x = hb * (BN / 4); x < (hb + 1) * (BN / 4); x += 2) {
              float e0, e1, e2, e3;
              ffma2(e0, e1, __uint_as_float(sr[2 * x]), __uint_as_float(sr[2 * x + 1]), c, neg_mc);
              ffma2(e2, e3, __uint_as_float(sr[2 * x + 2]), __uint_as_float(sr[2 * x + 3]), c, neg_mc);
#ifndef B200ATTN_POLY_MASK
#define B200ATTN_POLY_MASK 2
#endif
              if ((x & B200ATTN_POLY_MASK) == 0) {   // one value in four on the FMA pipe (more measured slower)
                exp2_fma_pair(e0, e1, e0, e1);
              } else {
                e0 = ex2(e0); e1 = ex2(e1);
              }
              e2 = ex2(e2); e3 = ex2(e3);
              fadd2(sum0, sum1, e0, e1);
              fadd2(sum2, sum3, e2, e3);
              pr[x] = pack2<T>(e0, e1);
              pr[x + 1] = pack2<T>(e2, e3);
            }
          } else {   // block-list mode: this query block does not list that KV block
#pragma unroll
            for (int x = hb * (BN / 4); x < (hb + 1) * (BN / 4); ++x) pr[x] = 0u;
          }
        }
        sum0 += sum2; sum1 += sum3;
#pragma unroll
        for (int cc = 0; cc < BN / 64; ++cc) tmem_st32(tS(t) + lane_off + 32 * cc, &pr[32 * cc]);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full(t));
        l_run = l_run * alpha + (sum0 + sum1);
        m_run = m_use;
        ++items;
      }
      // ------------------------------------------------------- epilogue
      // A tile that lies wholly inside its sequence leaves as 16-bit through its dead Q buffer
      // (same swizzled layout) and one copy-engine store per 64-column panel: written row by row
      // from the threads, 16 bytes per lane at a stride of a token, the 32 KB of a tile keep the
      // store path busy for thousands of cycles.  A tile that the sequence end cuts keeps the
      // per-thread stores, which leave the next packed sequence's rows alone.
      const bool row_ok = qi < len;
      const bool whole = q0t + kTileM <= len;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const long long tok = (long long)seq_start + qi;
      T* orow = (T*)p.o + (p.cu_seqlens ? 0 : (long long)b * p.o_sb) + tok * p.o_st + (long long)h * p.o_sh;
      uint8_t* sOut = smem_gen + t * L::kQBytes;       // every Q K^T product of this tile has completed
      if (items > 0) {
        mbar_wait(o_full(t), (items - 1) & 1, abort_flag);
        tc_fence_after();
      }
#pragma unroll
      for (int cc = 0; cc < DP / 32; ++cc) {
        uint32_t orr[32];
        if (items > 0) {
          tmem_ld32(tO(t) + lane_off + 32 * cc, orr);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) orr[x] = 0u;
        }
#pragma unroll
        for (int x = 0; x < 32; x += 8) {
          uint4 pk;
          pk.x = pack2<T>(__uint_as_float(orr[x]) * inv, __uint_as_float(orr[x + 1]) * inv);
          pk.y = pack2<T>(__uint_as_float(orr[x + 2]) * inv, __uint_as_float(orr[x + 3]) * inv);
          pk.z = pack2<T>(__uint_as_float(orr[x + 4]) * inv, __uint_as_float(orr[x + 5]) * inv);
          pk.w = pack2<T>(__uint_as_float(orr[x + 6]) * inv, __uint_as_float(orr[x + 7]) * inv);
          if (whole) {
            const int col = 32 * cc + x;               // 16-byte chunk (col % 64) / 8 of panel col / 64
            *reinterpret_cast<uint4*>(sOut + (col >> 6) * L::kQPanel + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4)) = pk;
          } else if (row_ok && 32 * cc < p.head_dim) {
            *reinterpret_cast<uint4*>(orow + 32 * cc + x) = pk;
          }
        }
      }
      if (whole) {
        fence_proxy_async();
        if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        if (row == 0) {
          for (int pn = 0; pn < kPanels; ++pn)
            tma_store_4d(&tmap_o, sQ + t * L::kQBytes + pn * L::kQPanel, 64 * pn, seq_start + q0t, h, bcoord);
          bulk_commit_group();
          bulk_wait_read_all();
        }
      }
      if (row_ok && p.lse) {
        float l2 = (l_run > 0.f) ? m_run * c + log2f(l_run) : -INFINITY;
        if (!p.lse_base2) l2 *= 0.6931471805599453f;
        p.lse[(p.cu_seqlens ? 0 : (long long)b * p.lse_sb) + tok * p.lse_st + (long long)h * p.lse_sh] = l2;
      }
    }
  }

  // ---- teardown (the single-lane roles above reconverge first)
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status_word) atomicExch(p.status_word, 1);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// --------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// [D, tokens, heads, batch] view of a 16-bit tensor, box = 64 x rows x 1 x 1, 128B swizzle.
static bool make_tmap(CUtensorMap* m, int dtype, const void* base, int D, long long tokens, int heads,
                      int batch, long long st, long long sh, long long sb, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)tokens, (cuuint64_t)heads, (cuuint64_t)batch};
  if (batch <= 1 || sb <= 0) sb = st * tokens;
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, dtype == B200ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static int validate_prefill(const b200attn_prefill_args* a, bool sparse) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return B200ATTN_ERR_NULL;
  if (a->dtype != B200ATTN_F16 && a->dtype != B200ATTN_BF16) return B200ATTN_ERR_DTYPE;
  if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 96 && a->head_dim != 128)
    return B200ATTN_ERR_HEAD_DIM;
  if (a->batch <= 0 || a->heads_q <= 0 || a->heads_kv <= 0) return B200ATTN_ERR_SHAPE;
  if (a->heads_q % a->heads_kv != 0) return B200ATTN_ERR_GQA;
  if (a->cu_seqlens) {
    if (a->max_seqlen < 0 || a->total_tokens <= 0) return B200ATTN_ERR_SHAPE;
  } else if (a->seqlen <= 0) {
    return B200ATTN_ERR_SHAPE;
  }
  const void* ptrs[4] = {a->q, a->k, a->v, a->o};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr & 15) return B200ATTN_ERR_ALIGN;
  const long long strides[12] = {a->q_stride_b, a->q_stride_t, a->q_stride_h, a->k_stride_b,
                                 a->k_stride_t, a->k_stride_h, a->v_stride_b, a->v_stride_t,
                                 a->v_stride_h, a->o_stride_b, a->o_stride_t, a->o_stride_h};
  for (long long s : strides)
    if (s % 8 != 0 || s < 0) return B200ATTN_ERR_STRIDE;
  if (!(a->softmax_scale > 0.f)) return B200ATTN_ERR_SHAPE;
  int mode = sparse ? a->sparsity : B200ATTN_DENSE;
  if (mode == B200ATTN_WINDOW) {
    if (a->window_local < 0 || a->window_global < 0) return B200ATTN_ERR_MODE;
  } else if (mode == B200ATTN_BLOCK_LIST) {
    if (!a->block_idx || !a->block_cnt) return B200ATTN_ERR_NULL;
    if (a->block_size != kBlk || a->n_qblocks <= 0 || a->max_nnz <= 0) return B200ATTN_ERR_MODE;
    const long long maxlen = a->cu_seqlens ? a->max_seqlen : a->seqlen;
    if ((maxlen + kBlk - 1) / kBlk > kMaxBlocks) return B200ATTN_ERR_TOO_LARGE;
  } else if (mode != B200ATTN_DENSE) {
    return B200ATTN_ERR_MODE;
  }
  return B200ATTN_OK;
}

template <typename T, int DP>
static int launch_prefill(const b200attn_prefill_args* a, const PrefillParams& p, cudaStream_t stream) {
  constexpr int BN = 128;
  constexpr int NSTAGE = DP == 128 ? 4 : 6;
  using L = PrefillSmem<DP, BN, NSTAGE>;
  const long long tokens = a->cu_seqlens ? a->total_tokens : a->seqlen;
  const int tb = a->cu_seqlens ? 1 : a->batch;
  CUtensorMap tq, tk, tv, to;
  if (!make_tmap(&tq, a->dtype, a->q, a->head_dim, tokens, a->heads_q, tb, a->q_stride_t, a->q_stride_h, a->q_stride_b, kTileM) ||
      !make_tmap(&tk, a->dtype, a->k, a->head_dim, tokens, a->heads_kv, tb, a->k_stride_t, a->k_stride_h, a->k_stride_b, p.block_idx ? kBlk : BN) ||
      !make_tmap(&tv, a->dtype, a->v, a->head_dim, tokens, a->heads_kv, tb, a->v_stride_t, a->v_stride_h, a->v_stride_b, p.block_idx ? kBlk : BN) ||
      !make_tmap(&to, a->dtype, a->o, a->head_dim, tokens, a->heads_q, tb, a->o_stride_t, a->o_stride_h, a->o_stride_b, kTileM))
    return B200ATTN_ERR_CUDA;
  auto kern = p.block_idx ? prefill_kernel<T, DP, BN, NSTAGE, true> : prefill_kernel<T, DP, BN, NSTAGE, false>;
  // the register count is a property of the binary: checked once per instantiation and mode
  static std::once_flag regs_once[2];
  static int regs_status[2];
  const int mode = p.block_idx ? 1 : 0;
  std::call_once(regs_once[mode], [kern, mode] {
    cudaFuncAttributes fa;
    regs_status[mode] = (cudaFuncGetAttributes(&fa, kern) == cudaSuccess && fa.numRegs >= kLaunchRegs)
                            ? B200ATTN_OK
                            : B200ATTN_ERR_CUDA;   // fewer registers: the hand-over would not balance
  });
  if (regs_status[mode] != B200ATTN_OK) return regs_status[mode];
  // the shared-memory opt-in is per device: set on every call (a process may drive several GPUs)
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc) != cudaSuccess)
    return B200ATTN_ERR_CUDA;
  const long long blocks = (long long)p.pair_count * a->heads_q * a->batch;
  if (blocks <= 0) return B200ATTN_OK;
  if (blocks > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  kern<<<(unsigned)blocks, kPrefillThreads, L::kAlloc, stream>>>(tq, tk, tv, to, p);
  set_launch_count(1);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

int prefill_fwd(const b200attn_prefill_args* a, bool sparse, cudaStream_t stream, int row_begin, int row_end) {
  int st = validate_prefill(a, sparse);
  if (st != B200ATTN_OK) return st;
  const bool all_rows = row_begin == 0 && row_end == INT_MAX;
  if (!all_rows) {
    if (sparse) return B200ATTN_ERR_MODE;
    if (row_begin < 0 || row_end <= row_begin || row_begin % kPairM != 0) return B200ATTN_ERR_SHAPE;
  }
  PrefillParams p;
  p.o = a->o; p.lse = a->lse; p.cu_seqlens = a->cu_seqlens;
  p.o_sb = a->o_stride_b; p.o_st = a->o_stride_t; p.o_sh = a->o_stride_h;
  p.lse_sb = a->lse_stride_b; p.lse_st = a->lse_stride_t; p.lse_sh = a->lse_stride_h;
  p.batch = a->batch; p.heads_q = a->heads_q; p.heads_kv = a->heads_kv;
  p.group = a->heads_q / a->heads_kv; p.head_dim = a->head_dim;
  p.seqlen = a->seqlen;
  const int maxlen = a->cu_seqlens ? a->max_seqlen : a->seqlen;
  p.n_pairs = (maxlen + kPairM - 1) / kPairM;
  // a row range ends on a 256-row boundary unless it runs to the end of the longest sequence
  if (!all_rows && row_end < maxlen && row_end % kPairM != 0) return B200ATTN_ERR_SHAPE;
  p.pair_begin = row_begin / kPairM;
  p.pair_count = (int)std::min<long long>(p.n_pairs, ((long long)row_end + kPairM - 1) / kPairM) - p.pair_begin;
  if (p.pair_count <= 0) return B200ATTN_OK;
  {
    const DeviceInfo* di = nullptr;
    st = device_info(&di);
    if (st != B200ATTN_OK) return st;
#ifndef B200ATTN_PREFETCH_WAVES
#define B200ATTN_PREFETCH_WAVES 1
#endif
    p.prefetch_ahead = di->sm_count * B200ATTN_PREFETCH_WAVES;   // one CTA per SM
  }
  const bool window = sparse && a->sparsity == B200ATTN_WINDOW;
  p.causal = window ? 1 : (a->causal ? 1 : 0);
  p.window = window ? 1 : 0;
  p.win_local = window ? (a->window_local > (1 << 30) ? (1 << 30) : a->window_local) : 0;
  p.win_global = window ? a->window_global : 0;
  p.scale_log2 = a->softmax_scale * (a->scale_has_log2e ? 1.f : 1.4426950408889634f);
  p.lse_base2 = a->lse_base2;
  p.status_word = a->status_word;
  const bool lists = sparse && a->sparsity == B200ATTN_BLOCK_LIST;
  p.block_idx = lists ? a->block_idx : nullptr;
  p.block_cnt = lists ? a->block_cnt : nullptr;
  p.n_qblocks = a->n_qblocks; p.max_nnz = a->max_nnz;
  const bool dp64 = a->head_dim <= 64;
  if (a->dtype == B200ATTN_F16)
    return dp64 ? launch_prefill<__half, 64>(a, p, stream) : launch_prefill<__half, 128>(a, p, stream);
  return dp64 ? launch_prefill<__nv_bfloat16, 64>(a, p, stream)
              : launch_prefill<__nv_bfloat16, 128>(a, p, stream);
}

}  // namespace b200attn
