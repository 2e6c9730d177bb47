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
// with vector reductions and converted at the end.  All five products are
// tcgen05.mma: S and dP with both operands K-major from shared memory; P and
// dS are written by the softmax threads into 128-byte-swizzled shared memory
// once and read twice, as the MN-major A operand of dV / dK and as the K-major
// A operand of dQ.  TMEM columns: S [0,128), dP then dQ [128,256), dK
// [256,384), dV [384,512).  Pipelining across (query tile, key tile) pairs: the
// query tiles are double buffered and the next pair's S is issued right behind
// this pair's dQ; dO is refetched as soon as the dV product has read it (and asked
// into L2 a pair ahead); the fp32 dQ tile leaves through shared memory and a copy-
// engine reduce-add, which runs while the next pair is computed.
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {
using namespace sm100;

namespace {

constexpr int kBwdComputeWarps = 8;   // warps 0-7: two threads per row (64 columns each)
constexpr int kBwdCtrlWarp = kBwdComputeWarps;                // MMA issue, Q reloads, dQ reduce-adds
constexpr int kBwdLoadWarp = kBwdComputeWarps + 1;            // K, V, dO loads
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
  static constexpr int kPds = kT * kT * 2;           // P, dS tiles
  static constexpr int kK = 0, kV = kOperand, kQ = 2 * kOperand, kDO = 3 * kOperand;
  static constexpr int kP = 4 * kOperand, kDS = kP + kPds;
  static constexpr int kQ1 = kDS + kPds;             // second Q tile (query tiles are double buffered)
  // The fp32 dQ tile leaves through shared memory in panels of 32 columns (128 rows,
  // 128-byte swizzle): the first half of the panels in the P tile, the second half in
  // the pair's own Q buffer, both dead by the time dQ exists.
  static constexpr int kStagePanel = kT * 128;
  static_assert((DP / 64) * kStagePanel <= kPds && (DP / 64) * kStagePanel <= kOperand, "dQ staging fits");
  static constexpr int kBarOffset = kQ1 + kOperand;
  static constexpr int kNumBars = 10;
  static constexpr int kBytes = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kAlloc = kBytes + 1024;
};

template <typename T, int DP>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
           const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
           const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  using L = BwdSmem<DP>;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdSS = idesc_f16(kFmt, false, kT, kT);           // S, dP: A, B K-major
  constexpr uint32_t kIdTT = idesc_f16(kFmt, true, kT, DP, true);      // dV, dK: A, B MN-major
  constexpr uint32_t kIdDQ = idesc_f16(kFmt, true, kT, DP, false);     // dQ: A K-major, B MN-major
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
  const uint32_t bar_kv = bars, bar_q0 = bars + 8, bar_do = bars + 24, bar_sdp = bars + 32, bar_pds = bars + 40,
                 bar_dv = bars + 48, bar_dq = bars + 56, bar_free = bars + 64, bar_pfree = bars + 72;   // bar_q0 + 8: second Q buffer
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_q0, 1);
    mbar_init(bar_q0 + 8, 1);
    mbar_init(bar_do, 1);
    mbar_init(bar_dv, 1);
    mbar_init(bar_sdp, 1);
    mbar_init(bar_pfree, 1);
    mbar_init(bar_pds, kBwdComputeThreads);
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

  // query tile and head of pair `it`
  auto pair_of = [&](int it, int& i, int& hq) { i = i_first + it / p.group; hq = hk * p.group + it % p.group; };
  if (warp == kBwdLoadWarp) {
    // ============================================ loader warp: K, V, the first Q tiles, every dO tile
    // (dO has one buffer: pair it + 1's tile is fetched the moment the dV product of
    // pair it has read it, which must not wait for the MMA warp to finish issuing)
    if (elect_one()) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      mbar_expect_tx(bar_kv, 2 * L::kOperand);
      for (int pn = 0; pn < kPanels; ++pn) {
        tma_load_4d(sbase + L::kK + pn * L::kPanel, &tmap_k, bar_kv, 64 * pn, seq_start + kv0, hk, bcoord);
        tma_load_4d(sbase + L::kV + pn * L::kPanel, &tmap_v, bar_kv, 64 * pn, seq_start + kv0, hk, bcoord);
      }
      for (int it = 0; it < min(n_iter, 2); ++it) {
        int i, hq;
        pair_of(it, i, hq);
        const uint32_t dst = sbase + (it ? L::kQ1 : L::kQ), bar = bar_q0 + 8 * it;
        mbar_expect_tx(bar, L::kOperand);
        for (int pn = 0; pn < kPanels; ++pn)
          tma_load_4d(dst + pn * L::kPanel, &tmap_q, bar, 64 * pn, seq_start + i * kT, hq, bcoord);
      }
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
            tma_prefetch_4d(&tmap_v, 64 * pn, ss2 + nx.jt * kT, nx.hk, bc2);
            tma_prefetch_4d(&tmap_q, 64 * pn, ss2 + i2 * kT, hq2, bc2);
            tma_prefetch_4d(&tmap_do, 64 * pn, ss2 + i2 * kT, hq2, bc2);
          }
        }
      }
      for (int it = 0; it < n_iter; ++it) {
        int i, hq;
        pair_of(it, i, hq);
        if (it > 0) mbar_wait(bar_dv, (it - 1) & 1, abort_flag);
        mbar_expect_tx(bar_do, L::kOperand);
        for (int pn = 0; pn < kPanels; ++pn)
          tma_load_4d(sbase + L::kDO + pn * L::kPanel, &tmap_do, bar_do, 64 * pn, seq_start + i * kT, hq, bcoord);
        if (it + 1 < n_iter) {        // next pair's dO, and the Q tile after next, into L2
          int in, hqn;
          pair_of(it + 1, in, hqn);
          for (int pn = 0; pn < kPanels; ++pn) tma_prefetch_4d(&tmap_do, 64 * pn, seq_start + in * kT, hqn, bcoord);
          if (it + 2 < n_iter) {
            pair_of(it + 2, in, hqn);
            for (int pn = 0; pn < kPanels; ++pn) tma_prefetch_4d(&tmap_q, 64 * pn, seq_start + in * kT, hqn, bcoord);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kBwdCtrlWarp) {
    // ============================================ MMA warp: products, Q reloads, dQ reduce-adds
    const uint32_t issue = elect_one() ? 1u : 0u;
    const uint64_t d_k = smem_desc_sw128(sbase + L::kK, 16, 1024);
    const uint64_t d_v = smem_desc_sw128(sbase + L::kV, 16, 1024);
    const uint64_t d_do = smem_desc_sw128(sbase + L::kDO, 16, 1024);
    const uint64_t d_p_mn = smem_desc_sw128(sbase + L::kP, L::kPanel, 1024);     // [q][k] read with M = k
    const uint64_t d_ds_mn = smem_desc_sw128(sbase + L::kDS, L::kPanel, 1024);
    const uint64_t d_ds_k = smem_desc_sw128(sbase + L::kDS, 16, 1024);           // same bytes, M = q
    const uint64_t d_do_mn = smem_desc_sw128(sbase + L::kDO, L::kPanel, 1024);   // [q][d] read with K = q
    const uint64_t d_k_mn = smem_desc_sw128(sbase + L::kK, L::kPanel, 1024);     // [k][d] read with K = k
    auto issue_s = [&](int itx) {      // S = Q K^T of pair itx (its Q buffer must have landed)
      const uint64_t dq_x = smem_desc_sw128(sbase + ((itx & 1) ? L::kQ1 : L::kQ), 16, 1024);
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        const uint64_t off = (uint64_t)(((ks / 4) * L::kPanel + (ks % 4) * 32) >> 4);
        mma_ss(tS, dq_x + off, d_k + off, kIdSS, ks > 0, issue);
      }
    };
    for (int it = 0; it < n_iter; ++it) {
      int i, hq;
      pair_of(it, i, hq);
      const uint32_t q_off = (it & 1) ? L::kQ1 : L::kQ;
      const uint64_t d_q_mn = smem_desc_sw128(sbase + q_off, L::kPanel, 1024);
      // Operand rows past the sequence end belong to the next packed sequence (or to nobody).
      // P and dS are exact zeros there, but 0 * Inf/NaN would still poison the sums they are
      // contracted over (K rows feed dQ; Q and dO rows feed dK and dV), so those rows are
      // cleared, like the reference's zero-padded loads (flash_attn_triton.py:155-165).
      const bool q_ragged = (i + 1) * kT > len;
      if (it == 0) {
        mbar_wait(bar_kv, 0, abort_flag);
        mbar_wait(bar_q0, 0, abort_flag);
        if (kv0 + kT > len) zero_tile_rows(sgen + L::kK, kPanels, L::kPanel, len - kv0, kT, lane);
        if (q_ragged) zero_tile_rows(sgen + L::kQ, kPanels, L::kPanel, max(len - i * kT, 0), kT, lane);
        tc_fence_after();
        issue_s(0);
      }
      // (S of later pairs is issued at the end of the pair before, behind its dQ product)
      mbar_wait(bar_do, it & 1, abort_flag);
      if (q_ragged) zero_tile_rows(sgen + L::kDO, kPanels, L::kPanel, max(len - i * kT, 0), kT, lane);
      tc_fence_after();
      // dP = dO V^T
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        const uint64_t off = (uint64_t)(((ks / 4) * L::kPanel + (ks % 4) * 32) >> 4);
        mma_ss(tDP, d_do + off, d_v + off, kIdSS, ks > 0, issue);
      }
      mma_commit(bar_sdp, issue);
      // the first half of the previous pair's dQ tile must have left the P bytes before
      // they are rewritten (the second half sits in a Q buffer and may still be on its way);
      // told to the compute warps separately, so that they wait for it only when they are
      // about to store, after their exponentials
      if (issue) { bulk_wait_read_but_one(); mbar_arrive(bar_pfree); }
      __syncwarp();
      // wait for P and dS in shared memory
      mbar_wait(bar_pds, it & 1, abort_flag);
      tc_fence_after();
      const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {   // contraction over the 128 queries
        const uint64_t off = (uint64_t)((ks * 2048) >> 4);
        mma_ss(tDV, d_p_mn + off, d_do_mn + off, kIdTT, ks > 0 ? 1u : acc, issue);
      }
      mma_commit(bar_dv, issue);
      // (issued first and alone: the loader refetches dO the moment this product has read it, and
      // that fetch is the longest wait of a pair)
      // The Q buffer of pair it - 1 held the second half of its dQ tile; once that is
      // read it takes the query tile of pair it + 1 (in L2 by now).  Behind the dV issue: waiting
      // for the copy engine here must not delay the product that frees dO.
      if (it > 0 && it + 1 < n_iter) {
        int in, hqn;
        pair_of(it + 1, in, hqn);
        if (issue) {
          bulk_wait_read_all();
          const uint32_t dst = sbase + (((it + 1) & 1) ? L::kQ1 : L::kQ), bar = bar_q0 + 8 * ((it + 1) & 1);
          mbar_expect_tx(bar, L::kOperand);
          for (int pn = 0; pn < kPanels; ++pn)
            tma_load_4d(dst + pn * L::kPanel, &tmap_q, bar, 64 * pn, seq_start + in * kT, hqn, bcoord);
        }
        __syncwarp();
      }
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {
        const uint64_t off = (uint64_t)((ks * 2048) >> 4);
        mma_ss(tDK, d_ds_mn + off, d_q_mn + off, kIdTT, ks > 0 ? 1u : acc, issue);
      }
#pragma unroll
      for (int ks = 0; ks < kT / 16; ++ks) {   // contraction over the 128 keys
        const uint64_t offa = (uint64_t)(((ks / 4) * L::kPanel + (ks % 4) * 32) >> 4);
        const uint64_t offb = (uint64_t)((ks * 2048) >> 4);
        mma_ss(tDP, d_ds_k + offa, d_k_mn + offb, kIdDQ, ks > 0, issue);   // dQ takes the dP columns
      }
      mma_commit(bar_dq, issue);
      // the S columns were read before P and dS were written: start the next pair's scores
      // now, so they are computed while this pair's dQ tile is being moved out
      if (it + 1 < n_iter) {
        mbar_wait(bar_q0 + 8 * ((it + 1) & 1), ((it + 1) >> 1) & 1, abort_flag);
        int in, hqn;
        pair_of(it + 1, in, hqn);
        if ((in + 1) * kT > len)
          zero_tile_rows(sgen + (((it + 1) & 1) ? L::kQ1 : L::kQ), kPanels, L::kPanel, max(len - in * kT, 0), kT, lane);
        tc_fence_after();
        issue_s(it + 1);
      }
      // the compute warps have moved the scaled dQ tile into shared memory (first half of
      // the columns in the P tile, second half in this pair's Q buffer): add both to the
      // fp32 accumulator in global memory, one bulk group each.  Rows past the sequence
      // end hold exact zeros.
      mbar_wait(bar_free, it & 1, abort_flag);
      if (issue) {
        const int tl0 = (p.cu_seqlens ? seq_start : b * p.seqlen) + i * kT;
        for (int pn = 0; pn < DP / 64; ++pn)
          tma_reduce_add_3d(&tmap_dq, sbase + L::kP + pn * L::kStagePanel, 32 * pn, tl0, hq);
        bulk_commit_group();
        for (int pn = 0; pn < DP / 64; ++pn)
          tma_reduce_add_3d(&tmap_dq, sbase + q_off + pn * L::kStagePanel, 32 * (DP / 64 + pn), tl0, hq);
        bulk_commit_group();
      }
      __syncwarp();
    }
#ifdef B200ATTN_BWD_READ_WAIT
    if (issue) bulk_wait_read_all();
#else
    if (issue) bulk_wait_all();
#endif
    __syncwarp();
  } else if (warp < kBwdComputeWarps) {
    // ============================================ compute warps: two threads per row
    // Two threads per row: warps w and w + 4 share TMEM lanes 32 (w % 4) .., each takes half
    // of the columns, so every scheduler has two warps to switch between.
    const int row = threadIdx.x & (kT - 1);              // query row in the tile / key row in the epilogue
    const int half = threadIdx.x >> 7;                   // which half of the columns
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* sP = sgen + L::kP;
    uint8_t* sDS = sgen + L::kDS;
    // lse and D of a pair's rows are fetched a pair ahead (global loads take thousands of cycles
    // while the reduce-adds keep the L2 busy)
    float lse2_nx = 0.f, dsum_nx = 0.f;
    bool live_nx = false;
    auto fetch_row_stats = [&](int itx) {
      lse2_nx = 0.f; dsum_nx = 0.f; live_nx = false;
      if (itx >= n_iter) return;
      const int gx = itx % p.group, ix = i_first + itx / p.group;
      const int hqx = hk * p.group + gx, qix = ix * kT + row;
      if (qix < len) {
        const long long tokx = (long long)seq_start + qix;
        const float l = p.lse[(p.cu_seqlens ? 0 : (long long)b * p.lse_sb) + tokx * p.lse_st + (long long)hqx * p.lse_sh];
        lse2_nx = p.lse_base2 ? l : l * 1.4426950408889634f;
        live_nx = l != -INFINITY;
        const long long tl = p.cu_seqlens ? tokx : (long long)b * p.seqlen + qix;
        dsum_nx = p.dvec[tl * p.heads_q + hqx];
      }
    };
    fetch_row_stats(0);
    for (int it = 0; it < n_iter; ++it) {
      const int i = i_first + it / p.group;
      const int qi = i * kT + row;
      const float lse2 = lse2_nx, dsum = dsum_nx;
      const bool live = live_nx;
      mbar_wait(bar_sdp, it & 1, abort_flag);
      tc_fence_after();
      // visible keys of this row inside the tile: columns [0, lim)
      int lim = live ? min(kT, len - kv0) : 0;
      if (p.causal) lim = min(lim, qi - kv0 + 1);
      const bool masked = __any_sync(0xffffffffu, lim < kT);   // only diagonal and ragged tiles
#pragma unroll
      for (int c2 = 0; c2 < kT / 64; ++c2) {
        const int cc = 2 * half + c2;                    // 32-column group
        uint32_t sr[32], dr[32];
        tmem_ld32(tS + lane_off + 32 * cc, sr);
        tmem_ld32(tDP + lane_off + 32 * cc, dr);
        tmem_wait_ld();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          float p0 = ex2f(fmaf(__uint_as_float(sr[x]), p.scale_log2, -lse2));
          float p1 = ex2f(fmaf(__uint_as_float(sr[x + 1]), p.scale_log2, -lse2));
          float d0 = p0 * (__uint_as_float(dr[x]) - dsum);
          float d1 = p1 * (__uint_as_float(dr[x + 1]) - dsum);
          if (masked) {
            // masked entries are exact zeros whatever S and dP hold there
            if (32 * cc + x >= lim) { p0 = 0.f; d0 = 0.f; }
            if (32 * cc + x + 1 >= lim) { p1 = 0.f; d1 = 0.f; }
          }
          pp[x / 2] = pack2<T>(p0, p1);
          dd[x / 2] = pack2<T>(d0, d1);
        }
        // row `row` of a [128 q][128 k] tile, two 64-column panels, 128-byte swizzle
        if (c2 == 0) mbar_wait(bar_pfree, it & 1, abort_flag);      // the P tile is no longer being read out
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = 4 * cc + ch;                       // 16-byte chunk of the 256-byte row
          const uint32_t off = (chunk >> 3) * L::kPanel + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
          *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
        }
      }
      fence_proxy_async();       // generic-proxy writes -> visible to the tensor core's reads
      tc_fence_before();
      mbar_arrive(bar_pds);
      fetch_row_stats(it + 1);
      // dQ tile of this pair -> fp32 accumulator
      mbar_wait(bar_dq, it & 1, abort_flag);
      tc_fence_after();
      // scaled fp32 tile -> shared memory in the copy engine's 128-byte-swizzled layout
      // (one panel per 32 columns); the control warp adds it to global memory
      uint8_t* sStage = sgen + (half == 0 ? L::kP : ((it & 1) ? L::kQ1 : L::kQ));
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
    // ---- dK, dV of this key tile (every product has completed: the last bar_dq was waited)
    // (tcgen05.ld is warp-collective: every thread runs the loads, only the
    // stores depend on the row being a real key)
    const int kj = kv0 + row;
    const bool key_ok = kj < len;
    const long long ktok = (long long)seq_start + (key_ok ? kj : 0);
    T* dkrow = (T*)p.dk + (p.cu_seqlens ? 0 : (long long)b * p.dk_sb) + ktok * p.dk_st + (long long)hk * p.dk_sh;
    T* dvrow = (T*)p.dv + (p.cu_seqlens ? 0 : (long long)b * p.dv_sb) + ktok * p.dv_st + (long long)hk * p.dv_sh;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const float sc = which ? 1.f : p.scale;
      T* dst = which ? dvrow : dkrow;
#pragma unroll
      for (int c2 = 0; c2 < DP / 64; ++c2) {
        const int cc = (DP / 64) * half + c2;
        uint32_t r[32];
        tmem_ld32((which ? tDV : tDK) + lane_off + 32 * cc, r);
        tmem_wait_ld();
        if (key_ok && 32 * cc < p.head_dim) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 pk;
            pk.x = pack2<T>(__uint_as_float(r[x]) * sc, __uint_as_float(r[x + 1]) * sc);
            pk.y = pack2<T>(__uint_as_float(r[x + 2]) * sc, __uint_as_float(r[x + 3]) * sc);
            pk.z = pack2<T>(__uint_as_float(r[x + 4]) * sc, __uint_as_float(r[x + 5]) * sc);
            pk.w = pack2<T>(__uint_as_float(r[x + 6]) * sc, __uint_as_float(r[x + 7]) * sc);
            *reinterpret_cast<uint4*>(dst + 32 * cc + x) = pk;
          }
        }
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
  CUtensorMap tq, tk, tv, tdo;
  if (!make_tmap(&tq, a->dtype, a->q, a->head_dim, tokens, a->heads_q, tb, a->q_stride_t, a->q_stride_h, a->q_stride_b) ||
      !make_tmap(&tk, a->dtype, a->k, a->head_dim, tokens, a->heads_kv, tb, a->k_stride_t, a->k_stride_h, a->k_stride_b) ||
      !make_tmap(&tv, a->dtype, a->v, a->head_dim, tokens, a->heads_kv, tb, a->v_stride_t, a->v_stride_h, a->v_stride_b) ||
      !make_tmap(&tdo, a->dtype, a->d_o, a->head_dim, tokens, a->heads_q, tb, a->do_stride_t, a->do_stride_h, a->do_stride_b))
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
  kern<<<grid, kBwdThreads, L::kAlloc, stream>>>(tq, tk, tv, tdo, tdq, p);
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
