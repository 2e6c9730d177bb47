// Dense prefill backward for sm_100a (dQ, dK, dV of causal / non-causal varlen GQA
// attention).  Stands in for flash_attn_triton_bwd and its three kernels
// (flash_attn_triton/flash_attn_triton.py:184-592, :661-813).
//
//   D_i  = sum_d dO_i O_i                                   (bwd_rowsum_kernel)
//   P    = exp2(Q K^T c - lse2)        dP = dO V^T
//   dS   = P o (dP - D)
//   dV  += P^T dO     dK += scale dS^T Q     dQ += scale dS K
//
// One CTA owns one 128-key tile of one (sequence, KV head) and walks every
// query head of the GQA group and every 128-row query tile that can see it:
// dK and dV of the tile accumulate in tensor memory across that whole walk
// (which also sums the group's query heads, done on the host in the
// reference, :813), dQ tiles are added to an fp32 accumulator in global memory
// by the copy engine and converted at the end.  All five products are
// tcgen05.mma.  The scores are formed transposed, S^T = K Q^T and dP^T = V dO^T
// (keys on the TMEM lanes), so that P^T and dS^T, written back over them as
// 16-bit, are the A operands of dV and dK straight from tensor memory; only
// dS^T also goes to shared memory ([key][query], 128-byte swizzle), where
// dQ = dS K reads it as an MN-major A operand.  TMEM columns: S^T [0,128) with
// P^T in [0,32) and [64,96), dP^T then dQ [128,256) with dS^T in [128,160) and
// [192,224), dK [256,384), dV [384,512).  Pipelining across (query tile, key
// tile) pairs: Q and dO tiles are double buffered (a dO fetch takes ~3000 cycles
// while the reduce-adds keep the L2 busy), the next pair's S^T is issued right
// behind this pair's dQ, and the fp32 dQ tile leaves through shared memory and a
// copy-engine reduce-add that runs while the next pair is computed.
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {
using namespace sm100;

namespace {

constexpr int kBwdComputeWarps = 8;   // warps 0-7: two threads per key row (64 query columns each)
constexpr int kBwdCtrlWarp = kBwdComputeWarps;                // issues the five products of every pair
constexpr int kBwdLoadWarp = kBwdComputeWarps + 1;            // every load, and the dQ reduce-adds
constexpr int kBwdThreads = 32 * (kBwdComputeWarps + 2);
constexpr int kBwdComputeThreads = 32 * kBwdComputeWarps;
constexpr int kT = 128;            // rows / keys per tile

struct BwdParams {
  const float* lse;
  const float* dvec;       // D, fp32 [tokens, heads_q]
  float* dq_acc;           // fp32 [tokens, heads_q, DP]
  void* dk;
  void* dv;
  const int32_t* cu_seqlens;
  long long lse_sb, lse_st, lse_sh;
  long long dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh;
  int batch, heads_q, heads_kv, group, head_dim;
  int seqlen, n_kvtiles;
  int causal;
  float scale_log2, scale;   // q.k multiplier in base-2 and natural form
  int lse_base2;
  int prefetch_ahead;        // CTAs resident at once: a CTA asks for the first tiles of CTA + this into L2
  int* status_word;
};

// (sequence, KV head) pairs are taken in groups of kBwdHeadGroup: inside a group the key tiles
// with the most query tiles to visit (the first ones when causal) of all its heads come first,
// which keeps the tail of the launch short, and the group is small enough for its fp32 dQ
// accumulators (the target of every reduce-add) to stay in L2 while its CTAs are resident.
#ifndef B200ATTN_BWD_HEAD_GROUP
#define B200ATTN_BWD_HEAD_GROUP 8
#endif
constexpr int kBwdHeadGroup = B200ATTN_BWD_HEAD_GROUP;
struct BwdCta { int jt, hk, b; };
__device__ __forceinline__ BwdCta bwd_cta_of(const BwdParams& p, int bid) {
  const int n_bh = p.batch * p.heads_kv;
  const int per_group = kBwdHeadGroup * p.n_kvtiles;
  const int grp = bid / per_group, in_grp = bid - grp * per_group;
  const int g_heads = min(kBwdHeadGroup, n_bh - grp * kBwdHeadGroup);
  const int bh = grp * kBwdHeadGroup + in_grp % g_heads;
  BwdCta c;
  c.jt = in_grp / g_heads;
  c.hk = bh % p.heads_kv;
  c.b = bh / p.heads_kv;
  return c;
}

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


template <int DP>
struct BwdSmem {
  static constexpr int kOperand = kT * DP * 2;       // K, V, Q, dO tiles
  static constexpr int kPanel = kT * 128;            // one 64-column swizzled panel
  static constexpr int kPds = kT * kT * 2;           // dS^T tile
  static constexpr int kK = 0, kV = kOperand, kQ = 2 * kOperand, kQ1 = 3 * kOperand;   // Q and dO: two buffers each
  static constexpr int kDO = 4 * kOperand, kDO1 = 5 * kOperand;
  static constexpr int kDS = 6 * kOperand;
  // The fp32 dQ tile leaves through shared memory in panels of 32 columns (128 rows,
  // 128-byte swizzle): the first half of the panels in the dS^T tile, the second half in
  // the pair's own Q buffer, both dead by the time dQ exists.
  static constexpr int kStagePanel = kT * 128;
  static_assert((DP / 64) * kStagePanel <= kPds && (DP / 64) * kStagePanel <= kOperand, "dQ staging fits");
  static constexpr int kStats = kDS + kPds;          // (lse2, D) of the pair's 128 query rows
  static constexpr int kBarOffset = kStats + kT * 8;
  static constexpr int kNumBars = 14;
  static constexpr int kBytes = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kAlloc = kBytes + 1024;
  static_assert(kAlloc <= 232448, "shared memory of one CTA");
};

template <typename T, int DP>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
           const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
           const __grid_constant__ CUtensorMap tmap_dq, const __grid_constant__ CUtensorMap tmap_dk,
           const __grid_constant__ CUtensorMap tmap_dv, const BwdParams p) {
  using L = BwdSmem<DP>;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdSS = idesc_f16(kFmt, false, kT, kT);           // S^T, dP^T: A, B K-major
  constexpr uint32_t kIdTS = idesc_f16(kFmt, true, kT, DP, false);     // dV, dK: A from tensor memory, B MN-major
  constexpr uint32_t kIdDQ = idesc_f16(kFmt, true, kT, DP, true);      // dQ: A, B MN-major
  constexpr int kPanels = DP / 64;

  const BwdCta me = bwd_cta_of(p, blockIdx.x);
  const int jt = me.jt;                      // key tile
  const int hk = me.hk, b = me.b;
  int seq_start = 0, len = p.seqlen, bcoord = b;
  if (p.cu_seqlens) {
    seq_start = p.cu_seqlens[b];
    // a sequence longer than the max_seqlen the grid was sized for is cut there
    len = min(p.cu_seqlens[b + 1] - seq_start, p.n_kvtiles * kT);
    bcoord = 0;
  }
  const int kv0 = jt * kT;
  if (kv0 >= len) return;
  const int n_qtiles = (len + kT - 1) / kT;
  const int i_first = p.causal ? jt : 0;     // first query tile that sees this key tile
  const int n_iter = (n_qtiles - i_first) * p.group;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bars = sbase + L::kBarOffset;
  const uint32_t bar_kv = bars, bar_q0 = bars + 8 /* +16: second buffer */, bar_do0 = bars + 24 /* +32 */,
                 bar_s = bars + 40, bar_dp = bars + 48, bar_pds = bars + 56, bar_dv0 = bars + 64 /* +72 */,
                 bar_dq = bars + 80, bar_free = bars + 88, bar_pfree = bars + 96, bar_p = bars + 104;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_q0, 1);
    mbar_init(bar_q0 + 8, 1);
    mbar_init(bar_do0, 1);
    mbar_init(bar_do0 + 8, 1);
    mbar_init(bar_dv0, 1);
    mbar_init(bar_dv0 + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_pfree, 1);
    mbar_init(bar_pds, kBwdComputeThreads);
    mbar_init(bar_p, kBwdComputeThreads);
    mbar_init(bar_dq, 1);
    mbar_init(bar_free, kBwdComputeThreads);
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
  const uint32_t tS = tmem, tDP = tmem + 128, tDK = tmem + 256, tDV = tmem + 384;
  // P^T / dS^T of the 16 queries of contraction step ks, as written by the compute warps:
  // queries [64 h, 64 h + 64) of a key row are packed into columns [64 h, 64 h + 32)
  auto a_cols = [](int ks) -> uint32_t { return (uint32_t)(64 * (ks / 4) + 8 * (ks % 4)); };

  // query tile and head of pair `it`
  auto pair_of = [&](int it, int& i, int& hq) { i = i_first + it / p.group; hq = hk * p.group + it % p.group; };
  if (warp == kBwdLoadWarp) {
    // ============================================ loader warp: every load, and the dQ reduce-adds
    if (elect_one()) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      int n_q[2] = {0, 0}, n_do[2] = {0, 0};     // loads sent into each buffer so far
      auto load_do = [&](int it) {
        int i, hq;
        pair_of(it, i, hq);
        ++n_do[it & 1];
        const uint32_t dst = sbase + ((it & 1) ? L::kDO1 : L::kDO), bar = bar_do0 + 8 * (it & 1);
        mbar_expect_tx(bar, L::kOperand);
        for (int pn = 0; pn < kPanels; ++pn)
          tma_load_4d(dst + pn * L::kPanel, &tmap_do, bar, 64 * pn, seq_start + i * kT, hq, bcoord);
      };
      auto load_q = [&](int it) {
        int i, hq;
        pair_of(it, i, hq);
        ++n_q[it & 1];
        const uint32_t dst = sbase + ((it & 1) ? L::kQ1 : L::kQ), bar = bar_q0 + 8 * (it & 1);
        mbar_expect_tx(bar, L::kOperand);
        for (int pn = 0; pn < kPanels; ++pn)
          tma_load_4d(dst + pn * L::kPanel, &tmap_q, bar, 64 * pn, seq_start + i * kT, hq, bcoord);
      };
      // in the order the first products need them: K and Q(0) for S^T, V and dO(0) for dP^T
      mbar_expect_tx(bar_kv, 2 * L::kOperand);
      for (int pn = 0; pn < kPanels; ++pn)
        tma_load_4d(sbase + L::kK + pn * L::kPanel, &tmap_k, bar_kv, 64 * pn, seq_start + kv0, hk, bcoord);
      load_q(0);
      for (int pn = 0; pn < kPanels; ++pn)
        tma_load_4d(sbase + L::kV + pn * L::kPanel, &tmap_v, bar_kv, 64 * pn, seq_start + kv0, hk, bcoord);
      load_do(0);
      if (n_iter > 1) { load_q(1); load_do(1); }
      // The CTA that will start when one of the resident ones ends finds its K / V tile and its
      // first Q / dO tiles on their way into L2.
      if (p.prefetch_ahead > 0 && blockIdx.x + p.prefetch_ahead < gridDim.x) {
        const BwdCta nx = bwd_cta_of(p, blockIdx.x + p.prefetch_ahead);
        int ss2 = 0, len2 = p.seqlen, bc2 = nx.b;
        if (p.cu_seqlens) { ss2 = p.cu_seqlens[nx.b]; len2 = min(p.cu_seqlens[nx.b + 1] - ss2, p.n_kvtiles * kT); bc2 = 0; }
        if (nx.jt * kT < len2) {
          const int i2 = p.causal ? nx.jt : 0, hq2 = nx.hk * p.group;
          for (int pn = 0; pn < kPanels; ++pn) {
            tma_prefetch_4d(&tmap_k, 64 * pn, ss2 + nx.jt * kT, nx.hk, bc2);
            tma_prefetch_4d(&tmap_q, 64 * pn, ss2 + i2 * kT, hq2, bc2);
            tma_prefetch_4d(&tmap_v, 64 * pn, ss2 + nx.jt * kT, nx.hk, bc2);
            tma_prefetch_4d(&tmap_do, 64 * pn, ss2 + i2 * kT, hq2, bc2);
          }
        }
      }
      // Per pair: the dO tile two pairs ahead (into the buffer this pair's dV product frees), the
      // pair's dQ tile added to the fp32 accumulator in global memory once the compute warps have
      // staged it (first half of the columns in the dS^T tile, second half in the pair's Q buffer,
      // one bulk group each; rows past the sequence end hold exact zeros), and the Q tile two pairs
      // ahead into that Q buffer once the copy engine has read it.  All of it here and not in the
      // MMA warp: issuing the reduce-adds alone blocks for ~1000 cycles while the engine is busy.
      mbar_arrive(bar_pfree);         // nothing is being read out of the dS^T tile before the first pair
      for (int it = 0; it < n_iter; ++it) {
        int i, hq;
        pair_of(it, i, hq);
        if (it + 2 < n_iter) {
          if (it + 3 < n_iter) {      // the pair after that into L2
            int in, hqn;
            pair_of(it + 3, in, hqn);
            for (int pn = 0; pn < kPanels; ++pn) {
              tma_prefetch_4d(&tmap_do, 64 * pn, seq_start + in * kT, hqn, bcoord);
              tma_prefetch_4d(&tmap_q, 64 * pn, seq_start + in * kT, hqn, bcoord);
            }
          }
          // (one barrier per dO buffer: the product that completes it again cannot run before the
          // load below, so the phase waited for here is never more than one behind)
          if (!mbar_wait(bar_dv0 + 8 * (it & 1), (it >> 1) & 1, abort_flag)) break;
          load_do(it + 2);
        }
        if (!mbar_wait(bar_free, it & 1, abort_flag)) break;
        const int tl0 = (p.cu_seqlens ? seq_start : b * p.seqlen) + i * kT;
        const uint32_t q_off = (it & 1) ? L::kQ1 : L::kQ;
        for (int pn = 0; pn < DP / 64; ++pn)
          tma_reduce_add_3d(&tmap_dq, sbase + L::kDS + pn * L::kStagePanel, 32 * pn, tl0, hq);
        bulk_commit_group();
        for (int pn = 0; pn < DP / 64; ++pn)
          tma_reduce_add_3d(&tmap_dq, sbase + q_off + pn * L::kStagePanel, 32 * (DP / 64 + pn), tl0, hq);
        bulk_commit_group();
        bulk_wait_read_but_one();     // the dS^T tile may be rewritten (the next pair's compute warps wait for this)
        mbar_arrive(bar_pfree);
        if (it + 2 < n_iter) {
          bulk_wait_read_all();       // and the Q buffer refilled
          load_q(it + 2);
        }
      }
      bulk_wait_all();
      // after a wait gave up somewhere, loads may still be on their way into shared memory that
      // nobody waits for any more: they must have landed before the CTA may exit
      if (*abort_flag) {
        mbar_drain(bar_kv, 0);
        for (int bf = 0; bf < 2; ++bf) {
          if (n_q[bf] > 0) mbar_drain(bar_q0 + 8 * bf, (n_q[bf] - 1) & 1);
          if (n_do[bf] > 0) mbar_drain(bar_do0 + 8 * bf, (n_do[bf] - 1) & 1);
        }
      }
    }
    __syncwarp();
  } else if (warp == kBwdCtrlWarp) {
    // ============================================ MMA warp: the five products of every pair
    const uint32_t issue = elect_one() ? 1u : 0u;
    const uint64_t d_k = smem_desc_sw128(sbase + L::kK, 16, 1024);
    const uint64_t d_v = smem_desc_sw128(sbase + L::kV, 16, 1024);
    const uint64_t d_dst_mn = smem_desc_sw128(sbase + L::kDS, L::kPanel, 1024);  // [k][q] read with M = q
    const uint64_t d_k_mn = smem_desc_sw128(sbase + L::kK, L::kPanel, 1024);     // [k][d] read with K = k
    auto issue_s = [&](int itx) {      // S^T = K Q^T of pair itx (its Q buffer must have landed)
      const uint64_t dq_x = smem_desc_sw128(sbase + ((itx & 1) ? L::kQ1 : L::kQ), 16, 1024);
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        const uint64_t off = (uint64_t)(((ks / 4) * L::kPanel + (ks % 4) * 32) >> 4);
        mma_ss(tS, d_k + off, dq_x + off, kIdSS, ks > 0, issue);
      }
    };
    for (int it = 0; it < n_iter; ++it) {
      int i, hq;
      pair_of(it, i, hq);
      const uint32_t q_off = (it & 1) ? L::kQ1 : L::kQ;
      const uint32_t do_off = (it & 1) ? L::kDO1 : L::kDO;
      const uint64_t d_q_mn = smem_desc_sw128(sbase + q_off, L::kPanel, 1024);     // [q][d] read with K = q
      const uint64_t d_do = smem_desc_sw128(sbase + do_off, 16, 1024);
      const uint64_t d_do_mn = smem_desc_sw128(sbase + do_off, L::kPanel, 1024);   // [q][d] read with K = q
      // Operand rows past the sequence end belong to the next packed sequence (or to nobody).
      // P and dS are exact zeros there, but 0 * Inf/NaN would still poison the sums they are
      // contracted over (K rows feed dQ, V rows dP; Q and dO rows feed dK and dV), so those
      // rows are cleared, like the reference's zero-padded loads (flash_attn_triton.py:155-165).
      const bool q_ragged = (i + 1) * kT > len;
      if (it == 0) {
        mbar_wait(bar_kv, 0, abort_flag);
        mbar_wait(bar_q0, 0, abort_flag);
        if (kv0 + kT > len) {
          zero_tile_rows(sgen + L::kK, kPanels, L::kPanel, len - kv0, kT, lane);
          zero_tile_rows(sgen + L::kV, kPanels, L::kPanel, len - kv0, kT, lane);
        }
        if (q_ragged) zero_tile_rows(sgen + L::kQ, kPanels, L::kPanel, max(len - i * kT, 0), kT, lane);
        tc_fence_after();
        issue_s(0);
        mma_commit(bar_s, issue);
      }
      // (S^T of later pairs is issued at the end of the pair before, behind its dQ product)
      mbar_wait(bar_do0 + 8 * (it & 1), (it >> 1) & 1, abort_flag);
      if (q_ragged) zero_tile_rows(sgen + do_off, kPanels, L::kPanel, max(len - i * kT, 0), kT, lane);
      tc_fence_after();
      // dP^T = V dO^T (its columns held the previous pair's dQ, read out before bar_free)
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        const uint64_t off = (uint64_t)(((ks / 4) * L::kPanel + (ks % 4) * 32) >> 4);
        mma_ss(tDP, d_v + off, d_do + off, kIdSS, ks > 0, issue);
      }
      mma_commit(bar_dp, issue);
      // P^T is in tensor memory: dV runs while the compute warps form dS^T
      mbar_wait(bar_p, it & 1, abort_flag);
      tc_fence_after();
      const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {   // dV += P^T dO, contraction over the 128 queries
        const uint64_t off = (uint64_t)((ks * 2048) >> 4);
        mma_ts(tDV, tS + a_cols(ks), d_do_mn + off, kIdTS, ks > 0 ? 1u : acc, issue);
      }
      mma_commit(bar_dv0 + 8 * (it & 1), issue);      // the loader may refill this dO buffer
      // dS^T in tensor memory and in shared memory
      mbar_wait(bar_pds, it & 1, abort_flag);
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {   // dK += dS^T Q
        const uint64_t off = (uint64_t)((ks * 2048) >> 4);
        mma_ts(tDK, tDP + a_cols(ks), d_q_mn + off, kIdTS, ks > 0 ? 1u : acc, issue);
      }
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {   // dQ = dS K, contraction over the 128 keys; takes the dP^T columns
        const uint64_t off = (uint64_t)((ks * 2048) >> 4);
        mma_ss(tDP, d_dst_mn + off, d_k_mn + off, kIdDQ, ks > 0, issue);
      }
      mma_commit(bar_dq, issue);
      // start the next pair's scores now (they overwrite P^T, which dV has read: products
      // run in issue order), so they are computed while this pair's dQ tile is being moved out
      if (it + 1 < n_iter) {
        mbar_wait(bar_q0 + 8 * ((it + 1) & 1), ((it + 1) >> 1) & 1, abort_flag);
        int in, hqn;
        pair_of(it + 1, in, hqn);
        if ((in + 1) * kT > len)
          zero_tile_rows(sgen + (((it + 1) & 1) ? L::kQ1 : L::kQ), kPanels, L::kPanel, max(len - in * kT, 0), kT, lane);
        tc_fence_after();
        issue_s(it + 1);
        mma_commit(bar_s, issue);
      }
      // the next pair's dP^T takes the columns of this pair's dQ: the compute warps must have
      // moved it out
      mbar_wait(bar_free, it & 1, abort_flag);
    }
  } else if (warp < kBwdComputeWarps) {
    // ============================================ compute warps: two threads per key row
    // Warps w and w + 4 share TMEM lanes 32 (w % 4) .. (one key row per lane); each takes half
    // of the columns (64 queries), so every scheduler has two warps to switch between.
    const int row = threadIdx.x & (kT - 1);              // key row in the tile (query row when dQ is moved out)
    const int half = threadIdx.x >> 7;                   // which half of the columns
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* sDS = sgen + L::kDS;
    float* s_lse = reinterpret_cast<float*>(sgen + L::kStats);     // lse2 and D of the pair's query rows
    float* s_dsum = s_lse + kT;
    const int kj = kv0 + row;
    // lse and D of a pair's query rows are fetched a pair ahead by the threads of the first half
    // (global loads take thousands of cycles while the reduce-adds keep the L2 busy) and passed
    // through shared memory: every thread needs them for all of its 64 columns.  A query row past
    // the sequence end, or one without a visible key (lse = -inf), gets lse2 = +inf: P = 0 there.
    float lse2_nx = INFINITY, dsum_nx = 0.f;
    auto fetch_row_stats = [&](int itx) {
      lse2_nx = INFINITY; dsum_nx = 0.f;
      if (half != 0 || itx >= n_iter) return;
      const int gx = itx % p.group, ix = i_first + itx / p.group;
      const int hqx = hk * p.group + gx, qix = ix * kT + row;
      if (qix < len) {
        const long long tokx = (long long)seq_start + qix;
        const float l = p.lse[(p.cu_seqlens ? 0 : (long long)b * p.lse_sb) + tokx * p.lse_st + (long long)hqx * p.lse_sh];
        if (l != -INFINITY) lse2_nx = p.lse_base2 ? l : l * 1.4426950408889634f;
        const long long tl = p.cu_seqlens ? tokx : (long long)b * p.seqlen + qix;
        dsum_nx = p.dvec[tl * p.heads_q + hqx];
      }
    };
    fetch_row_stats(0);
    for (int it = 0; it < n_iter; ++it) {
      const int i = i_first + it / p.group;
      // every thread is past its reads of the previous pair's statistics (it waited for that
      // pair's dQ, which is issued only after all of them handed P^T and dS^T over)
      if (half == 0) { s_lse[row] = lse2_nx; s_dsum[row] = dsum_nx; }
      asm volatile("bar.sync 1, %0;" ::"n"(kBwdComputeThreads) : "memory");
      // Column x of this row (query i * 128 + x) is visible iff x >= xmin: the causal diagonal
      // when this is the diagonal tile, nothing at all for a key row past the sequence end.
      int xmin = p.causal ? kj - i * kT : 0;
      if (kj >= len) xmin = 1 << 20;
      const bool masked = (p.causal && kv0 + kT - 1 > i * kT) || (kv0 + kT > len);   // (same for the whole CTA)
      // P^T from S^T alone: the exponentials run while dP^T, which had to wait for the previous
      // pair's dQ to leave its columns, is still being computed
      mbar_wait(bar_s, it & 1, abort_flag);
      tc_fence_after();
      float pf[kT / 2];
#pragma unroll
      for (int c2 = 0; c2 < kT / 64; ++c2) {
        const int cc = 2 * half + c2;                    // 32-column group: queries [32 cc, 32 cc + 32)
        uint32_t sr[32];
        tmem_ld32(tS + lane_off + 32 * cc, sr);
        tmem_wait_ld();
        uint32_t pp[16];
        const float4* l4 = reinterpret_cast<const float4*>(s_lse + 32 * cc);
        float4 st = make_float4(0.f, 0.f, 0.f, 0.f);     // lse2 of queries x .. x + 3
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          if ((x & 2) == 0) st = l4[x / 4];
          const float l0 = (x & 2) ? st.z : st.x, l1 = (x & 2) ? st.w : st.y;
          float p0 = ex2f(fmaf(__uint_as_float(sr[x]), p.scale_log2, -l0));
          float p1 = ex2f(fmaf(__uint_as_float(sr[x + 1]), p.scale_log2, -l1));
          if (masked) {
            // masked entries are exact zeros whatever S holds there
            if (32 * cc + x < xmin) p0 = 0.f;
            if (32 * cc + x + 1 < xmin) p1 = 0.f;
          }
          pf[32 * c2 + x] = p0;
          pf[32 * c2 + x + 1] = p1;
          pp[x / 2] = pack2<T>(p0, p1);
        }
        // P^T back into tensor memory, over columns of S^T this thread has read
        tmem_st16(tS + lane_off + 64 * half + 16 * c2, pp);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);
      // dS^T = P^T o (dP^T - D)
      mbar_wait(bar_dp, it & 1, abort_flag);
      tc_fence_after();
#pragma unroll
      for (int c2 = 0; c2 < kT / 64; ++c2) {
        const int cc = 2 * half + c2;
        uint32_t dr[32];
        tmem_ld32(tDP + lane_off + 32 * cc, dr);
        tmem_wait_ld();
        uint32_t dd[16];
        const float4* d4 = reinterpret_cast<const float4*>(s_dsum + 32 * cc);
        float4 st = make_float4(0.f, 0.f, 0.f, 0.f);     // D of queries x .. x + 3
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          if ((x & 2) == 0) st = d4[x / 4];
          // (P = 0 where masked; dP is finite there: rows past the sequence end are cleared)
          const float d0 = pf[32 * c2 + x] * (__uint_as_float(dr[x]) - ((x & 2) ? st.z : st.x));
          const float d1 = pf[32 * c2 + x + 1] * (__uint_as_float(dr[x + 1]) - ((x & 2) ? st.w : st.y));
          dd[x / 2] = pack2<T>(d0, d1);
        }
        tmem_st16(tDP + lane_off + 64 * half + 16 * c2, dd);
        // dS^T also as row `row` of a [128 k][128 q] tile, two 64-column panels, 128-byte swizzle
        if (c2 == 0) mbar_wait(bar_pfree, it & 1, abort_flag);      // the tile is no longer being read out
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = 4 * c2 + ch;                       // 16-byte chunk of this half's 128-byte panel row
          const uint32_t off = half * L::kPanel + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
        }
      }
      tmem_wait_st();
      fence_proxy_async();       // generic-proxy writes -> visible to the tensor core's reads
      tc_fence_before();
      mbar_arrive(bar_pds);
      fetch_row_stats(it + 1);
      // dQ tile of this pair -> fp32 accumulator
      mbar_wait(bar_dq, it & 1, abort_flag);
      tc_fence_after();
      // scaled fp32 tile -> shared memory in the copy engine's 128-byte-swizzled layout
      // (one panel per 32 columns); the loader warp adds it to global memory
      uint8_t* sStage = sgen + (half == 0 ? L::kDS : ((it & 1) ? L::kQ1 : L::kQ));
#pragma unroll
      for (int c2 = 0; c2 < DP / 64; ++c2) {
        const int cc = (DP / 64) * half + c2;
        uint32_t qr[32];
        tmem_ld32(tDP + lane_off + 32 * cc, qr);
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint32_t off = c2 * L::kStagePanel + row * 128 + ((ch ^ (row & 7)) << 4);
          *reinterpret_cast<float4*>(sStage + off) =
              make_float4(__uint_as_float(qr[4 * ch]) * p.scale, __uint_as_float(qr[4 * ch + 1]) * p.scale,
                          __uint_as_float(qr[4 * ch + 2]) * p.scale, __uint_as_float(qr[4 * ch + 3]) * p.scale);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_free);
    }
    // ---- dK, dV of this key tile (every product has completed: the last bar_dq was waited).
    // A whole tile goes out as 16-bit through the dead K and V buffers (same swizzled layout as
    // the operands) and two copy-engine stores: written row by row from the threads, 16 bytes per
    // lane at a stride of a token, the 64 KB took ~8000 cycles per CTA.  A tile that the sequence
    // end cuts keeps the per-thread stores, which can leave the next sequence's rows alone.
    // (tcgen05.ld is warp-collective: every thread runs the loads, only the stores depend on
    // the row being a real key)
    const bool key_ok = kj < len;
    const bool whole = kv0 + kT <= len;
    const long long ktok = (long long)seq_start + (key_ok ? kj : 0);
    T* dkrow = (T*)p.dk + (p.cu_seqlens ? 0 : (long long)b * p.dk_sb) + ktok * p.dk_st + (long long)hk * p.dk_sh;
    T* dvrow = (T*)p.dv + (p.cu_seqlens ? 0 : (long long)b * p.dv_sb) + ktok * p.dv_st + (long long)hk * p.dv_sh;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const float sc = which ? 1.f : p.scale;
      T* dst = which ? dvrow : dkrow;
      uint8_t* sOut = sgen + (which ? L::kV : L::kK);
#pragma unroll
      for (int c2 = 0; c2 < DP / 64; ++c2) {
        const int cc = (DP / 64) * half + c2;
        uint32_t r[32];
        tmem_ld32((which ? tDV : tDK) + lane_off + 32 * cc, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; x += 8) {
          uint4 pk;
          pk.x = pack2<T>(__uint_as_float(r[x]) * sc, __uint_as_float(r[x + 1]) * sc);
          pk.y = pack2<T>(__uint_as_float(r[x + 2]) * sc, __uint_as_float(r[x + 3]) * sc);
          pk.z = pack2<T>(__uint_as_float(r[x + 4]) * sc, __uint_as_float(r[x + 5]) * sc);
          pk.w = pack2<T>(__uint_as_float(r[x + 6]) * sc, __uint_as_float(r[x + 7]) * sc);
          if (whole) {
            const int col = 32 * cc + x;                 // 16-byte chunk (col % 64) / 8 of panel col / 64
            *reinterpret_cast<uint4*>(sOut + (col >> 6) * L::kPanel + row * 128 + (((((col & 63) >> 3)) ^ (row & 7)) << 4)) = pk;
          } else if (key_ok && 32 * cc < p.head_dim) {
            *reinterpret_cast<uint4*>(dst + 32 * cc + x) = pk;
          }
        }
      }
    }
    if (whole) {
      fence_proxy_async();
      asm volatile("bar.sync 1, %0;" ::"n"(kBwdComputeThreads) : "memory");
      if (threadIdx.x == 0) {
        for (int pn = 0; pn < kPanels; ++pn) {
          tma_store_4d(&tmap_dk, sbase + L::kK + pn * L::kPanel, 64 * pn, seq_start + kv0, hk, bcoord);
          tma_store_4d(&tmap_dv, sbase + L::kV + pn * L::kPanel, 64 * pn, seq_start + kv0, hk, bcoord);
        }
        bulk_commit_group();
        bulk_wait_read_all();
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status_word) atomicExch(p.status_word, 1);
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


// D[t, h] = sum_d dO[t, h, d] * O[t, h, d], and the row's fp32 dQ accumulator cleared (saves a
// separate memset pass over it): eight lanes per (token, head) with 16-byte loads.
template <typename T>
__global__ void bwd_rowsum_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ dvec,
                                  float* __restrict__ dq_acc, long long o_sb, long long o_st, long long o_sh,
                                  long long do_sb, long long do_st, long long do_sh, int tokens_per_batch, int heads,
                                  int D, int DP, long long total) {
  const int sub = threadIdx.x & 7;
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  float s = 0.f;
  if (idx < total) {
    const int hq = (int)(idx % heads);
    const long long tl = idx / heads;
    const long long bb = tl / tokens_per_batch, tt = tl % tokens_per_batch;
    const T* orow = o + bb * o_sb + tt * o_st + (long long)hq * o_sh;
    const T* drow = d_o + bb * do_sb + tt * do_st + (long long)hq * do_sh;
    for (int c = 8 * sub; c < D; c += 64) {
      const uint4 ov = *reinterpret_cast<const uint4*>(orow + c);
      const uint4 dv = *reinterpret_cast<const uint4*>(drow + c);
      const T* oe = reinterpret_cast<const T*>(&ov);
      const T* de = reinterpret_cast<const T*>(&dv);
#pragma unroll
      for (int x = 0; x < 8; ++x) s = fmaf((float)oe[x], (float)de[x], s);
    }
    float4* acc = reinterpret_cast<float4*>(dq_acc + idx * DP);
    for (int c = sub; c < DP / 4; c += 8) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (idx < total && sub == 0) dvec[idx] = s;
}

// dq[t, h, :D] = T(dq_acc[t, h, :D])
template <typename T>
__global__ void bwd_convert_dq_kernel(const float* __restrict__ acc, T* __restrict__ dq, long long dq_sb,
                                      long long dq_st, long long dq_sh, int tokens_per_batch, int heads, int D,
                                      int DP, long long total_rows) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 8 elements
  const int per_row = DP / 8;
  const long long r = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  if (r >= total_rows || c >= D) return;
  const int hq = (int)(r % heads);
  const long long tl = r / heads;
  const long long bb = tl / tokens_per_batch, tt = tl % tokens_per_batch;
  const float4 a = *reinterpret_cast<const float4*>(acc + r * DP + c);
  const float4 bq = *reinterpret_cast<const float4*>(acc + r * DP + c + 4);
  uint4 pk;
  pk.x = pack2<T>(a.x, a.y); pk.y = pack2<T>(a.z, a.w);
  pk.z = pack2<T>(bq.x, bq.y); pk.w = pack2<T>(bq.z, bq.w);
  *reinterpret_cast<uint4*>(dq + bb * dq_sb + tt * dq_st + (long long)hq * dq_sh + c) = pk;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

bool make_tmap(CUtensorMap* m, int dtype, const void* base, int D, long long tokens, int heads, int batch,
               long long st, long long sh, long long sb) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)tokens, (cuuint64_t)heads, (cuuint64_t)batch};
  if (batch <= 1 || sb <= 0) sb = st * tokens;
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)kT, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, dtype == B200ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 [tokens, heads, DP] accumulator as [DP, tokens, heads], box = 32 x 128 x 1, 128B swizzle
bool make_dq_tmap(CUtensorMap* m, float* base, int DP, long long tokens, int heads) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)DP, (cuuint64_t)tokens, (cuuint64_t)heads};
  cuuint64_t strides[2] = {(cuuint64_t)heads * DP * 4, (cuuint64_t)DP * 4};
  cuuint32_t box[3] = {32, (cuuint32_t)kT, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int dpad(int d) { return d <= 64 ? 64 : 128; }

long long total_rows(const b200attn_prefill_bwd_args* a) {
  const long long tokens = a->cu_seqlens ? a->total_tokens : (long long)a->batch * a->seqlen;
  return tokens * a->heads_q;
}

int validate_bwd(const b200attn_prefill_bwd_args* a) {
  if (!a || !a->q || !a->k || !a->v || !a->o || !a->d_o || !a->lse || !a->dq || !a->dk || !a->dv)
    return B200ATTN_ERR_NULL;
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
  const void* ptrs[8] = {a->q, a->k, a->v, a->o, a->d_o, a->dq, a->dk, a->dv};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr & 15) return B200ATTN_ERR_ALIGN;
  const long long strides[24] = {
      a->q_stride_b, a->q_stride_t, a->q_stride_h, a->k_stride_b, a->k_stride_t, a->k_stride_h,
      a->v_stride_b, a->v_stride_t, a->v_stride_h, a->o_stride_b, a->o_stride_t, a->o_stride_h,
      a->do_stride_b, a->do_stride_t, a->do_stride_h, a->dq_stride_b, a->dq_stride_t, a->dq_stride_h,
      a->dk_stride_b, a->dk_stride_t, a->dk_stride_h, a->dv_stride_b, a->dv_stride_t, a->dv_stride_h};
  for (long long s : strides)
    if (s % 8 != 0 || s < 0) return B200ATTN_ERR_STRIDE;
  if (!(a->softmax_scale > 0.f)) return B200ATTN_ERR_SHAPE;
  if (a->heads_kv > 65535 || a->batch > 65535) return B200ATTN_ERR_TOO_LARGE;
  return B200ATTN_OK;
}

template <typename T, int DP>
int launch_bwd(const b200attn_prefill_bwd_args* a, const BwdParams& p, cudaStream_t stream) {
  using L = BwdSmem<DP>;
  const long long tokens = a->cu_seqlens ? a->total_tokens : a->seqlen;
  const int tb = a->cu_seqlens ? 1 : a->batch;
  CUtensorMap tq, tk, tv, tdo, tdk, tdv;
  if (!make_tmap(&tq, a->dtype, a->q, a->head_dim, tokens, a->heads_q, tb, a->q_stride_t, a->q_stride_h, a->q_stride_b) ||
      !make_tmap(&tk, a->dtype, a->k, a->head_dim, tokens, a->heads_kv, tb, a->k_stride_t, a->k_stride_h, a->k_stride_b) ||
      !make_tmap(&tv, a->dtype, a->v, a->head_dim, tokens, a->heads_kv, tb, a->v_stride_t, a->v_stride_h, a->v_stride_b) ||
      !make_tmap(&tdo, a->dtype, a->d_o, a->head_dim, tokens, a->heads_q, tb, a->do_stride_t, a->do_stride_h, a->do_stride_b) ||
      !make_tmap(&tdk, a->dtype, a->dk, a->head_dim, tokens, a->heads_kv, tb, a->dk_stride_t, a->dk_stride_h, a->dk_stride_b) ||
      !make_tmap(&tdv, a->dtype, a->dv, a->head_dim, tokens, a->heads_kv, tb, a->dv_stride_t, a->dv_stride_h, a->dv_stride_b))
    return B200ATTN_ERR_CUDA;
  auto kern = bwd_kernel<T, DP>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc) != cudaSuccess)
    return B200ATTN_ERR_CUDA;
  const long long rows = total_rows(a);
  CUtensorMap tdq;
  if (!make_dq_tmap(&tdq, p.dq_acc, DP, rows / a->heads_q, a->heads_q)) return B200ATTN_ERR_CUDA;
  const int tpb = a->cu_seqlens ? (int)a->total_tokens : a->seqlen;   // tokens per batch entry of the dense index
  // 1. D = rowsum(dO o O), and the dq accumulator cleared
  {
    const long long blocks = (rows * 8 + 255) / 256;
    bwd_rowsum_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
        (const T*)a->o, (const T*)a->d_o, const_cast<float*>(p.dvec), p.dq_acc, a->cu_seqlens ? 0 : a->o_stride_b,
        a->o_stride_t, a->o_stride_h, a->cu_seqlens ? 0 : a->do_stride_b, a->do_stride_t, a->do_stride_h, tpb,
        a->heads_q, a->head_dim, DP, rows);
  }
  // 2. main kernel (the dq accumulator was cleared by the row-sum kernel)
  const long long n_ctas = (long long)p.n_kvtiles * a->heads_kv * a->batch;
  if (n_ctas > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  dim3 grid((unsigned)n_ctas);
  kern<<<grid, kBwdThreads, L::kAlloc, stream>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  // 3. dq accumulator -> dq
  {
    const long long items = rows * (DP / 8);
    bwd_convert_dq_kernel<T><<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(
        p.dq_acc, (T*)a->dq, a->cu_seqlens ? 0 : a->dq_stride_b, a->dq_stride_t, a->dq_stride_h, tpb,
        a->heads_q, a->head_dim, DP, rows);
  }
  set_launch_count(3);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

}  // namespace

size_t prefill_bwd_workspace_bytes(const b200attn_prefill_bwd_args* a) {
  if (!a || a->heads_q <= 0) return 0;
  const long long rows = total_rows(a);
  if (rows <= 0) return 0;
  return (size_t)rows * dpad(a->head_dim) * 4 + (size_t)rows * 4;
}

int prefill_bwd(const b200attn_prefill_bwd_args* a, cudaStream_t stream) {
  int st = validate_bwd(a);
  if (st != B200ATTN_OK) return st;
  const size_t need = prefill_bwd_workspace_bytes(a);
  if (!a->workspace || a->workspace_bytes < need) return B200ATTN_ERR_WORKSPACE;
  if ((uintptr_t)a->workspace & 15) return B200ATTN_ERR_ALIGN;
  const DeviceInfo* di = nullptr;
  st = device_info(&di);
  if (st != B200ATTN_OK) return st;
  const long long rows = total_rows(a);
  const int DP = dpad(a->head_dim);
  BwdParams p;
  p.lse = a->lse;
  p.dq_acc = (float*)a->workspace;
  p.dvec = p.dq_acc + rows * DP;
  p.dk = a->dk; p.dv = a->dv;
  p.cu_seqlens = a->cu_seqlens;
  p.lse_sb = a->lse_stride_b; p.lse_st = a->lse_stride_t; p.lse_sh = a->lse_stride_h;
  p.dk_sb = a->dk_stride_b; p.dk_st = a->dk_stride_t; p.dk_sh = a->dk_stride_h;
  p.dv_sb = a->dv_stride_b; p.dv_st = a->dv_stride_t; p.dv_sh = a->dv_stride_h;
  p.batch = a->batch; p.heads_q = a->heads_q; p.heads_kv = a->heads_kv;
  p.group = a->heads_q / a->heads_kv; p.head_dim = a->head_dim;
  p.seqlen = a->seqlen;
  const int maxlen = a->cu_seqlens ? a->max_seqlen : a->seqlen;
  p.n_kvtiles = (maxlen + kT - 1) / kT;
  if (p.n_kvtiles <= 0) return B200ATTN_OK;
  p.causal = a->causal ? 1 : 0;
  p.scale = a->softmax_scale * (a->scale_has_log2e ? 0.6931471805599453f : 1.f);
  p.scale_log2 = a->softmax_scale * (a->scale_has_log2e ? 1.f : 1.4426950408889634f);
  p.lse_base2 = a->lse_base2;
  p.status_word = a->status_word;
  p.prefetch_ahead = di->sm_count;   // one CTA per SM
  const bool dp64 = DP == 64;
  if (a->dtype == B200ATTN_F16)
    return dp64 ? launch_bwd<__half, 64>(a, p, stream) : launch_bwd<__half, 128>(a, p, stream);
  return dp64 ? launch_bwd<__nv_bfloat16, 64>(a, p, stream) : launch_bwd<__nv_bfloat16, 128>(a, p, stream);
}

}  // namespace b200attn
