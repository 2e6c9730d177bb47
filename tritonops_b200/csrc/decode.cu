// Split-KV GQA decoding for sm_100a: one query token per sequence against a
// padded KV cache, dense / window-sparse / block-list-sparse, plus the
// log-sum-exp combine.  Stands in for flash_attn_decoding_kernel +
// flash_attn_decoding_correction_kernel (flash_attn_triton/flash_attn_decoding.py:9-210)
// and their sparse twins (flash_attn_triton/flash_attn_decoding_sparse.py:10-219).
//
// The path is HBM-bound (each K/V byte is used once), so the kernel is built
// around the memory system: every K and V element goes from global memory
// straight into registers with 128-bit loads, already in the operand layout
// of the m16n8k16 tensor-core instruction, so no shared-memory staging and no
// shuffles sit between the load and the math.  All query heads of one KV head
// (GQA group, up to 8 per pass) ride in one MMA tile, so the cache is read
// once per KV head instead of once per query head as the reference does
// (flash_attn_decoding.py:45).
//
//   S^T[g, t] = sum_d Q[g, d] K[t, d]      A = Q (16 x 16, rows >= 8 are zero)
//                                          B = K^T (16 x 8 tokens)
//   O^T[d, g] = sum_t V[t, d] P[g, t]      A = V^T (16 d x 16 tokens)
//                                          B = P^T (16 tokens x 8 heads)
//
// The contraction index of the first product (d) and the row index of the
// second (d again) may be permuted freely, which is what lets a thread feed
// 8 consecutive d of one token row (one 16-byte load) to the instruction:
// the C fragment of S^T is, register for register, the B fragment of P^T.
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kUnit = 16;  // tokens one warp handles per step
constexpr int kPaged = 3;  // internal key map: every key of the sequence, found through a page table

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* part_o;    // [B, Hq, max_chunks, D] fp32, normalised inside the chunk
  float* part_lse;  // [B, Hq, max_chunks] base-2 LSE of the prescaled scores
  const int32_t* cu_seqlens;
  const int32_t* seqlens;
  const int32_t* block_idx;
  const int32_t* block_cnt;
  long long q_sb, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, o_sb, o_sh;
  int batch, heads_q, heads_kv, group, ggroups;
  int chunk, max_chunks;
  int sparsity, win_global, win_local, block_size, max_sel;
  int head_dim_rt;
  int max_seqlen;     // lengths beyond it are cut there (the grid and the scratch are sized for it)
  int* status_word;   // nullable: set to 1 when a bounded wait of the split kernel gave up
  float scale_log2;
  long long map_keys;  // host only: key extent and batch extent of the cache's tensor maps
  int map_batch;
};

// How many keys sequence b / kv head hk attends to, and where they live.
// The visible keys are numbered 0..n-1 ("virtual" positions); to_token maps a
// virtual position to a row of the cache.
struct KeyMap {
  int n;       // number of visible keys
  int len;     // sequence length
  int mode;    // b200attn_sparsity, or kPaged
  int split;   // WINDOW: virtual positions >= split are shifted by `shift`
  int shift;
  int bshift;  // BLOCK_LIST: log2(block_size) when a power of two, else -1
  int bsize;
  const int32_t* blocks;
  __device__ __forceinline__ int to_token(int vpos) const {
    if (mode == 0) return vpos;
    if (mode == 1) return vpos < split ? vpos : vpos + shift;
    int bi = vpos / bsize;
    return blocks[bi] * bsize + (vpos - bi * bsize);
  }
};

__device__ __forceinline__ int seq_len_of(const DecodeParams& p, int b) {
  return p.seqlens ? p.seqlens[b] : p.cu_seqlens[b + 1] - p.cu_seqlens[b];
}

__device__ __forceinline__ KeyMap make_keymap(const DecodeParams& p, int b, int hk) {
  KeyMap m;
  m.len = min(max(seq_len_of(p, b), 0), p.max_seqlen);
  m.mode = p.sparsity;
  m.split = 0; m.shift = 0; m.bsize = 1; m.bshift = 0; m.blocks = nullptr;
  if (p.sparsity == 0) {
    m.n = m.len;
  } else if (p.sparsity == 1) {
    // keys j < G or j >= len - L  (flash_attn_decoding_sparse.py:82-85)
    int g = min(p.win_global, m.len);
    int start2 = max(m.len - p.win_local, g);
    m.split = g;
    m.shift = start2 - g;
    m.n = g + (m.len - start2);
  } else if (p.sparsity == kPaged) {
    // key t lives in row page_table[b][t / page] * page + t % page of the pool
    m.bsize = p.block_size;
    m.blocks = p.block_idx + (long long)b * p.max_sel;
    m.n = min(m.len, p.max_sel * p.block_size);
  } else {
    m.bsize = p.block_size;
    m.blocks = p.block_idx + ((long long)b * p.heads_kv + hk) * p.max_sel;
    int cnt = p.block_cnt ? min(p.block_cnt[b * p.heads_kv + hk], p.max_sel) : p.max_sel;
    // trailing -1 entries are padding
    while (cnt > 0 && m.blocks[cnt - 1] < 0) --cnt;
    m.n = cnt * p.block_size;
  }
  return m;
}

template <int D>
struct UnitRegs {
  static constexpr int KC = D / 32;        // 16-byte chunks of a K row per thread
  static constexpr int DH = (D + 63) / 64;  // 64-wide d groups of a V row
  uint4 k[2][KC];  // [8-token tile][chunk]
  uint4 v[4][DH];  // [token slot][d group]
  unsigned valid;  // bit nt*2+i: key (8nt + 2tig + i) is a real key
};

template <typename T, int D>
__device__ __forceinline__ void load_unit(UnitRegs<D>& r, const T* __restrict__ kbase,
                                          const T* __restrict__ vbase, long long k_st,
                                          long long v_st, const KeyMap& km, int v0, int v_end,
                                          int gid, int tig) {
  constexpr int KC = UnitRegs<D>::KC, DH = UnitRegs<D>::DH;
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    int vp = v0 + 8 * nt + gid;
    bool ok = vp < v_end;
    int tok = ok ? km.to_token(vp) : 0;
    ok = ok && tok >= 0 && tok < km.len;
    const T* row = kbase + (long long)tok * k_st + 8 * tig;
#pragma unroll
    for (int c = 0; c < KC; ++c) r.k[nt][c] = ok ? ld_nc_16(row + 32 * c) : zero;
  }
  unsigned valid = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // token slots 2tig, 2tig+1, 2tig+8, 2tig+9 of the 16-token unit
    int slot = 2 * tig + (j & 1) + 8 * (j >> 1);
    int vp = v0 + slot;
    bool ok = vp < v_end;
    int tok = ok ? km.to_token(vp) : 0;
    ok = ok && tok >= 0 && tok < km.len;
    valid |= ok ? (1u << j) : 0u;
    const T* row = vbase + (long long)tok * v_st + 8 * gid;
#pragma unroll
    for (int h = 0; h < DH; ++h) {
      bool dok = ok && (64 * h + 8 * gid < D);
      r.v[j][h] = dok ? ld_nc_16(row + 64 * h) : zero;
    }
  }
  r.valid = valid;
}

#ifndef B200ATTN_DECODE_CTAS
#define B200ATTN_DECODE_CTAS 4
#endif
// Resident CTAs per SM the register budget is sized for.  Four (16 warps)
// rather than two with a software-pipelined second register buffer: each CTA
// has a fixed start-up and combine cost of a few microseconds during which it
// moves no data, and more resident CTAs keep the memory system busy meanwhile.
constexpr int kDecodeCtasPerSm = B200ATTN_DECODE_CTAS;

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, kDecodeCtasPerSm)
decode_split_kernel(const DecodeParams p) {
  constexpr int KC = UnitRegs<D>::KC, DH = UnitRegs<D>::DH;
  constexpr int NMT = 4 * DH;  // 16-row d tiles of O^T
  // KV heads vary fastest in launch order: the CTAs resident together then read
  // neighbouring 256-byte pieces of the same token rows (same DRAM pages)
  const int hk = blockIdx.x / p.ggroups;
  const int gg = blockIdx.x % p.ggroups;
  const int chunk_id = blockIdx.y;
  const int b = blockIdx.z;
  const KeyMap km = make_keymap(p, b, hk);
  const int c_begin = chunk_id * p.chunk;
  if (c_begin >= km.n) return;
  const int c_end = min(km.n, c_begin + p.chunk);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int g_row = gg * 8 + gid;               // query head inside the GQA group owned by this lane's row
  const bool g_ok = g_row < p.group;

  const T* qrow = (const T*)p.q + (long long)b * p.q_sb + (long long)(hk * p.group + (g_ok ? g_row : 0)) * p.q_sh;
  const T* kbase = (const T*)p.k + (long long)b * p.k_sb + (long long)hk * p.k_sh;
  const T* vbase = (const T*)p.v + (long long)b * p.v_sb + (long long)hk * p.v_sh;

  // Q fragments: chunk c holds d = 32c + 8tig .. +8 of head g_row
  uint4 qf[KC];
#pragma unroll
  for (int c = 0; c < KC; ++c)
    qf[c] = g_ok ? ld_nc_16(qrow + 32 * c + 8 * tig) : make_uint4(0, 0, 0, 0);

  float acc[NMT][4];
#pragma unroll
  for (int i = 0; i < NMT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run = -INFINITY;  // running max of row gid (base-2 domain), uniform across the quad
  float l_run = 0.f;        // this thread's share of the row sum

  auto compute = [&](const UnitRegs<D>& r, int v0) {
    // ---- scores S^T for two 8-token tiles
    float s[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < KC; ++ch) {
        mma_16816<T>(c, qf[ch].x, 0u, qf[ch].y, 0u, r.k[nt][ch].x, r.k[nt][ch].y);
        mma_16816<T>(c, qf[ch].z, 0u, qf[ch].w, 0u, r.k[nt][ch].z, r.k[nt][ch].w);
      }
      s[nt][0] = c[0] * p.scale_log2;
      s[nt][1] = c[1] * p.scale_log2;
    }
    // this thread's score columns are token slots 8nt + 2tig + {0,1} == V slots j = 2nt + i
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (!((r.valid >> (2 * nt + i)) & 1u)) s[nt][i] = -INFINITY;
    float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_use);   // m_run = -inf -> 0
    m_run = m_new;
    float pr[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 2; ++i) pr[nt][i] = exp2f(s[nt][i] - m_use);
    l_run = l_run * alpha + (pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1]);
    // accumulator columns of this thread are heads 2tig, 2tig+1 -> fetch their factors
    const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * tig) * 4);
    const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * tig + 1) * 4);
    const unsigned pb0 = pack2<T>(pr[0][0], pr[0][1]);
    const unsigned pb1 = pack2<T>(pr[1][0], pr[1][1]);
    // ---- O^T += V^T P^T
#pragma unroll
    for (int h = 0; h < DH; ++h) {
      const unsigned* t0 = reinterpret_cast<const unsigned*>(&r.v[0][h]);
      const unsigned* t1 = reinterpret_cast<const unsigned*>(&r.v[1][h]);
      const unsigned* t2 = reinterpret_cast<const unsigned*>(&r.v[2][h]);
      const unsigned* t3 = reinterpret_cast<const unsigned*>(&r.v[3][h]);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        float* c = acc[h * 4 + w];
        c[0] *= a0; c[1] *= a1; c[2] *= a0; c[3] *= a1;
        const unsigned ra0 = __byte_perm(t0[w], t1[w], 0x5410);  // d = 8gid+2w,   tokens 2tig, 2tig+1
        const unsigned ra1 = __byte_perm(t0[w], t1[w], 0x7632);  // d = 8gid+2w+1
        const unsigned ra2 = __byte_perm(t2[w], t3[w], 0x5410);  // tokens 2tig+8, 2tig+9
        const unsigned ra3 = __byte_perm(t2[w], t3[w], 0x7632);
        mma_16816<T>(c, ra0, ra1, ra2, ra3, pb0, pb1);
      }
    }
    (void)v0;
  };

  // ---- stream the chunk: warps take 16-token units round-robin, loads for
  // the next unit are in flight while the current one is computed
  const int stride = kDecodeWarps * kUnit;
  if (kDecodeCtasPerSm <= 2) {
    // two register buffers: loads of the next unit in flight during the math
    UnitRegs<D> ra, rb;
    int u = c_begin + warp * kUnit;
    if (u < c_end) load_unit<T, D>(ra, kbase, vbase, p.k_st, p.v_st, km, u, c_end, gid, tig);
    for (; u < c_end; u += 2 * stride) {
      const bool has_b = u + stride < c_end;
      if (has_b) load_unit<T, D>(rb, kbase, vbase, p.k_st, p.v_st, km, u + stride, c_end, gid, tig);
      compute(ra, u);
      if (u + 2 * stride < c_end)
        load_unit<T, D>(ra, kbase, vbase, p.k_st, p.v_st, km, u + 2 * stride, c_end, gid, tig);
      if (has_b) compute(rb, u + stride);
    }
  } else {
    // one register buffer, more warps per SM: the other warps' loads cover this
    // warp's math
    UnitRegs<D> ra;
    for (int u = c_begin + warp * kUnit; u < c_end; u += stride) {
      load_unit<T, D>(ra, kbase, vbase, p.k_st, p.v_st, km, u, c_end, gid, tig);
      compute(ra, u);
    }
  }

  // ---- combine the four warps, then write the chunk partial
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __shared__ float sm_m[kDecodeWarps][8];
  __shared__ float sm_l[kDecodeWarps][8];
  __shared__ float sm_o[kDecodeWarps][NMT * 16][8 + 1];
  if (tig == 0) { sm_m[warp][gid] = m_run; sm_l[warp][gid] = l_run; }
#pragma unroll
  for (int mt = 0; mt < NMT; ++mt) {
    // row index inside the tile list: d = 64h + 8gid + 2w + {0,1}
    const int h = mt >> 2, w = mt & 3;
    const int d0 = 64 * h + 8 * gid + 2 * w;
    sm_o[warp][d0][2 * tig] = acc[mt][0];
    sm_o[warp][d0][2 * tig + 1] = acc[mt][1];
    sm_o[warp][d0 + 1][2 * tig] = acc[mt][2];
    sm_o[warp][d0 + 1][2 * tig + 1] = acc[mt][3];
  }
  __syncthreads();
  const int heads_here = min(8, p.group - gg * 8);
  for (int idx = threadIdx.x; idx < heads_here * D; idx += kDecodeThreads) {
    const int g = idx / D, d = idx - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, sm_m[w][g]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float f = exp2f(sm_m[w][g] - Ms);
      L += sm_l[w][g] * f;
      O += sm_o[w][d][g] * f;
    }
    const int hq = hk * p.group + gg * 8 + g;
    const long long row = ((long long)b * p.heads_q + hq) * p.max_chunks + chunk_id;
    p.part_o[row * D + d] = L > 0.f ? O / L : 0.f;
    if (d == 0) p.part_lse[row] = L > 0.f ? Ms + log2f(L) : -INFINITY;
  }
}

// --------------------------------------------------------------------------
// TMA variant of phase 1.  Same work split (one CTA per sequence, KV-head
// group and 512-key chunk) and the same partials, but K and V reach the SM as
// bulk tensor copies: a producer warp streams 64-key stages (four 16-key boxes
// per operand and 64-column panel, 128-byte swizzle) through a shared-memory
// ring guarded by full / empty mbarriers, so the bytes in flight per SM are set
// by the ring depth rather than by the load/store unit's outstanding requests,
// and four consumer warps read their 16 keys of each stage with ldmatrix.
// Up to 16 query heads of a GQA group ride in one MMA tile (M = 16).
// --------------------------------------------------------------------------
constexpr int kStageTok = 64;   // keys per ring stage
constexpr int kBoxTok = 16;     // keys per TMA box (window / block gathers are 16-key aligned)

template <int DP>
struct DecodeTmaSmem {
  static constexpr int kPanels = DP / 64;
  static constexpr int kPanelBytes = kStageTok * 128;
  static constexpr int kTileBytes = kPanels * kPanelBytes;   // K or V of one stage
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kStages = DP == 128 ? 3 : 5;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kBytes = kBarOffset + 2 * kStages * 8 + 16;
  static constexpr int kAlloc = kBytes + 1024;
  static constexpr int kCombinePitch = DP + 1;                // floats per (warp, head) row of the combine buffer
  static_assert(4 * 16 * kCombinePitch * 4 + 2 * 4 * 16 * 4 <= kStages * kStageBytes, "combine buffer aliases the ring");
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T, int DP>
__global__ void __launch_bounds__(160, 2)
decode_split_tma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const DecodeParams p) {
  using L = DecodeTmaSmem<DP>;
  using namespace sm100;
  constexpr int NKT = DP / 16;   // 16-wide d steps of the score product
  constexpr int NDT = DP / 8;    // 8-wide d tiles of the output
  const int hk = blockIdx.x / p.ggroups;
  const int gg = blockIdx.x % p.ggroups;   // group of 16 query heads inside the GQA group
  const int chunk_id = blockIdx.y;
  const int b = blockIdx.z;
  const KeyMap km = make_keymap(p, b, hk);
  const int c_begin = chunk_id * p.chunk;
  if (c_begin >= km.n) return;
  const int c_end = min(km.n, c_begin + p.chunk);
  const int map_b = km.mode == kPaged ? 0 : b;   // a page pool has no batch axis
  const int n_tiles = (c_end - c_begin + kStageTok - 1) / kStageTok;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bars = sbase + L::kBarOffset;
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (L::kStages + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kBarOffset + 2 * L::kStages * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < L::kStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 4); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == 4) {
    // ================================================================ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      int issued = 0;
      // Block lists and page tables: the block holding a stage's first key is looked up one
      // stage ahead (the load is in flight during the wait for the stage to become free), and
      // boxes of the stage that lie in the same block reuse it.
      const bool listed = km.mode >= 2;
      int nxt_blk = (listed && n_tiles > 0) ? km.blocks[c_begin / km.bsize] : 0;
      for (int tile = 0; tile < n_tiles; ++tile, ++issued) {
        const int s = tile % L::kStages;
        const int v0 = c_begin + tile * kStageTok;
        const int cur_blk = nxt_blk;
        const int cur_idx = listed ? v0 / km.bsize : 0;
        const int cur_off = listed ? v0 - cur_idx * km.bsize : 0;
        if (listed && tile + 1 < n_tiles) nxt_blk = km.blocks[(v0 + kStageTok) / km.bsize];
        if (!mbar_wait(empty(s), ((tile / L::kStages) & 1) ^ 1, abort_flag)) break;
        const int nbox = min(kStageTok / kBoxTok, (c_end - v0 + kBoxTok - 1) / kBoxTok);
        mbar_expect_tx(full(s), nbox * 2 * L::kPanels * kBoxTok * 128);
        const uint32_t kdst = sbase + s * L::kStageBytes, vdst = kdst + L::kTileBytes;
        for (int i = 0; i < nbox; ++i) {
          // 16 consecutive cache rows (rows past the end are masked)
          const int tok = (listed && cur_off + kBoxTok * i < km.bsize) ? cur_blk * km.bsize + cur_off + kBoxTok * i
                                                                       : km.to_token(v0 + kBoxTok * i);
          for (int pn = 0; pn < L::kPanels; ++pn) {
            const uint32_t off = pn * L::kPanelBytes + i * kBoxTok * 128;
            tma_load_4d(kdst + off, &tmap_k, full(s), 64 * pn, tok, hk, map_b);
            tma_load_4d(vdst + off, &tmap_v, full(s), 64 * pn, tok, hk, map_b);
          }
        }
      }
      // A wait gave up somewhere in the CTA: the consumers no longer wait for the stages, so
      // the copies still in flight are waited for here before the CTA may exit.
      if (*abort_flag)
        for (int tile = max(issued - L::kStages, 0); tile < issued; ++tile)
          mbar_drain(full(tile % L::kStages), (tile / L::kStages) & 1);
    }
    return;
  }

  // ================================================================== consumers
  const int gid = lane >> 2, tig = lane & 3;
  const int g0 = gg * 16 + gid, g1 = g0 + 8;          // query heads of this lane's two MMA rows
  const T* qbase = (const T*)p.q + (long long)b * p.q_sb + (long long)(hk * p.group) * p.q_sh;
  unsigned qa[NKT][4];
#pragma unroll
  for (int kt = 0; kt < NKT; ++kt) {
    const int d = 16 * kt + 2 * tig;
    const bool dok0 = d < p.head_dim_rt, dok1 = d + 8 < p.head_dim_rt;
    qa[kt][0] = (g0 < p.group && dok0) ? *reinterpret_cast<const unsigned*>(qbase + (long long)g0 * p.q_sh + d) : 0u;
    qa[kt][1] = (g1 < p.group && dok0) ? *reinterpret_cast<const unsigned*>(qbase + (long long)g1 * p.q_sh + d) : 0u;
    qa[kt][2] = (g0 < p.group && dok1) ? *reinterpret_cast<const unsigned*>(qbase + (long long)g0 * p.q_sh + d + 8) : 0u;
    qa[kt][3] = (g1 < p.group && dok1) ? *reinterpret_cast<const unsigned*>(qbase + (long long)g1 * p.q_sh + d + 8) : 0u;
  }
  float acc[NDT][4];
#pragma unroll
  for (int i = 0; i < NDT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % L::kStages;
    if (!mbar_wait(full(s), (tile / L::kStages) & 1, abort_flag)) break;   // reported below
    const int v0 = c_begin + tile * kStageTok + 16 * warp;   // this warp's 16 keys of the stage
    if (v0 < c_end) {
      const uint32_t ktile = sbase + s * L::kStageBytes, vtile = ktile + L::kTileBytes;
      // which of the 16 keys are real (inside the chunk and inside the sequence)
      bool ok = false;
      if (lane < 16) {
        const int vp = v0 + lane;
        if (vp < c_end) {
          if (km.mode == kPaged) {
            ok = true;                       // every key below the length is real, wherever its page lies
          } else {
            const int tok = km.to_token(v0 & ~(kBoxTok - 1)) + (lane & (kBoxTok - 1));
            ok = tok >= 0 && tok < km.len;
          }
        }
      }
      const unsigned vmask = __ballot_sync(0xffffffffu, ok) & 0xffffu;
      if (vmask != 0xffffu) {
        // rows of V that are not real keys may hold anything (cache padding): P = 0
        // times NaN would poison O, so they are cleared in shared memory first
        uint8_t* vgen = sgen + (vtile - sbase);
        for (int r = 0; r < 16; ++r) {
          if ((vmask >> r) & 1u) continue;
          const int row = 16 * warp + r;
          for (int i = lane; i < L::kPanels * 8; i += 32)
            *reinterpret_cast<uint4*>(vgen + (i >> 3) * L::kPanelBytes + row * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();   // these plain stores precede the copy engine's next write to the stage
        __syncwarp();
      }
      // ---- S[g, key] = Q K^T for two 8-key tiles
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const int mi = lane >> 3, r = lane & 7;
        const int row = 16 * warp + 8 * (mi >> 1) + r;
#pragma unroll
        for (int kt = 0; kt < NKT; ++kt) {
          const int c16 = 2 * kt + (mi & 1);
          const uint32_t addr = ktile + (c16 >> 3) * L::kPanelBytes + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(addr, b0, b1, b2, b3);
          mma_16816<T>(c0, qa[kt][0], qa[kt][1], qa[kt][2], qa[kt][3], b0, b1);
          mma_16816<T>(c1, qa[kt][0], qa[kt][1], qa[kt][2], qa[kt][3], b2, b3);
        }
      }
      // columns of this thread: keys 2tig, 2tig+1 (c0) and 8+2tig, 9+2tig (c1); rows gid (x0,x1) and gid+8 (x2,x3)
      float sc[2][4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sc[r][0] = ((vmask >> (2 * tig)) & 1u) ? c0[2 * r] * p.scale_log2 : -INFINITY;
        sc[r][1] = ((vmask >> (2 * tig + 1)) & 1u) ? c0[2 * r + 1] * p.scale_log2 : -INFINITY;
        sc[r][2] = ((vmask >> (8 + 2 * tig)) & 1u) ? c1[2 * r] * p.scale_log2 : -INFINITY;
        sc[r][3] = ((vmask >> (9 + 2 * tig)) & 1u) ? c1[2 * r + 1] * p.scale_log2 : -INFINITY;
      }
      float alpha[2];
      unsigned pa[4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = fmaxf(fmaxf(sc[r][0], sc[r][1]), fmaxf(sc[r][2], sc[r][3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use);
        m_run[r] = m_new;
        const float p0 = exp2f(sc[r][0] - m_use), p1 = exp2f(sc[r][1] - m_use);
        const float p2 = exp2f(sc[r][2] - m_use), p3 = exp2f(sc[r][3] - m_use);
        l_run[r] = l_run[r] * alpha[r] + ((p0 + p1) + (p2 + p3));
        pa[r] = pack2<T>(p0, p1);        // A fragment: row gid (+8), keys 2tig, 2tig+1
        pa[2 + r] = pack2<T>(p2, p3);    //             row gid (+8), keys 8+2tig, 9+2tig
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < NDT; ++i) {
          acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
          acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
        }
      }
      // ---- O[g, d] += P V
      {
        const int mi = lane >> 3, r = lane & 7;
        const int row = 16 * warp + 8 * (mi & 1) + r;
#pragma unroll
        for (int dp = 0; dp < NDT / 2; ++dp) {
          const int c16 = 2 * dp + (mi >> 1);
          const uint32_t addr = vtile + (c16 >> 3) * L::kPanelBytes + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(addr, b0, b1, b2, b3);
          mma_16816<T>(acc[2 * dp], pa[0], pa[1], pa[2], pa[3], b0, b1);
          mma_16816<T>(acc[2 * dp + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty(s));
  }

  // ---- combine the four warps (the ring is free now: every stage was consumed)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  const int heads_here = min(16, p.group - gg * 16);
  const int D = p.head_dim_rt;
  if (*abort_flag) {
    // A bounded wait gave up (flash_attn_decoding.py has no counterpart: its loads cannot
    // stall).  The ring may still be receiving copies, so it is not reused as the combine
    // buffer: the chunk is reported as empty and the caller is told through the status word.
    for (int idx = threadIdx.x; idx < heads_here * D; idx += 128) {
      const int g = idx / D, d = idx - g * D;
      const long long row = ((long long)b * p.heads_q + hk * p.group + gg * 16 + g) * p.max_chunks + chunk_id;
      p.part_o[row * D + d] = 0.f;
      if (d == 0) p.part_lse[row] = -INFINITY;
    }
    if (threadIdx.x == 0 && p.status_word) atomicExch(p.status_word, 1);
    return;
  }
  float* sm_o = reinterpret_cast<float*>(sgen);                       // [4][16][DP + 1]
  float* sm_m = sm_o + 4 * 16 * L::kCombinePitch;                      // [4][16]
  float* sm_l = sm_m + 4 * 16;
  if (tig == 0) {
    sm_m[warp * 16 + gid] = m_run[0]; sm_m[warp * 16 + gid + 8] = m_run[1];
    sm_l[warp * 16 + gid] = l_run[0]; sm_l[warp * 16 + gid + 8] = l_run[1];
  }
#pragma unroll
  for (int i = 0; i < NDT; ++i) {
    float* r0 = sm_o + (warp * 16 + gid) * L::kCombinePitch + 8 * i + 2 * tig;
    float* r1 = sm_o + (warp * 16 + gid + 8) * L::kCombinePitch + 8 * i + 2 * tig;
    r0[0] = acc[i][0]; r0[1] = acc[i][1];
    r1[0] = acc[i][2]; r1[1] = acc[i][3];
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  for (int idx = threadIdx.x; idx < heads_here * D; idx += 128) {
    const int g = idx / D, d = idx - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + g]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_m[w * 16 + g] - Ms);
      Lsum += sm_l[w * 16 + g] * f;
      O += sm_o[(w * 16 + g) * L::kCombinePitch + d] * f;
    }
    const int hq = hk * p.group + gg * 16 + g;
    const long long row = ((long long)b * p.heads_q + hq) * p.max_chunks + chunk_id;
    p.part_o[row * D + d] = Lsum > 0.f ? O / Lsum : 0.f;
    if (d == 0) p.part_lse[row] = Lsum > 0.f ? Ms + log2f(Lsum) : -INFINITY;
  }
}

// Phase 2: O = sum_c o_c * 2^(lse_c - lse), lse = log2 sum_c 2^lse_c
// (flash_attn_decoding.py:173-208).  Sequences without visible keys give 0.
template <typename T, int D>
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecodeParams p) {
  // Launched with programmatic stream serialisation: its CTAs may be set up while phase 1 is
  // still draining, and wait here until that whole grid has finished and its partials are
  // visible (a no-op when launched the ordinary way).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int hq = blockIdx.x, b = blockIdx.y;
  const KeyMap km = make_keymap(p, b, hq / p.group);
  const int nchunk = (km.n + p.chunk - 1) / p.chunk;
  const long long row0 = ((long long)b * p.heads_q + hq) * p.max_chunks;
  float M = -INFINITY;
  for (int c = 0; c < nchunk; ++c) M = fmaxf(M, p.part_lse[row0 + c]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f;
  for (int c = 0; c < nchunk; ++c) L += exp2f(p.part_lse[row0 + c] - Ms);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  T* orow = (T*)p.o + (long long)b * p.o_sb + (long long)hq * p.o_sh;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < nchunk; ++c)
      acc += p.part_o[(row0 + c) * D + d] * (exp2f(p.part_lse[row0 + c] - Ms) * inv);
    orow[d] = from_float<T>(acc);
  }
}

// --------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------
static int decode_max_visible(const b200attn_decode_args* a) {
  if (a->sparsity == B200ATTN_WINDOW) {
    long long w = (long long)a->window_global + a->window_local;
    return (int)(w < a->max_seqlen ? w : a->max_seqlen);
  }
  if (a->sparsity == B200ATTN_BLOCK_LIST) return a->max_sel * a->block_size;
  if (a->sparsity == kPaged) {
    long long w = (long long)a->max_sel * a->block_size;
    return (int)(w < a->max_seqlen ? w : a->max_seqlen);
  }
  return a->max_seqlen;
}

// Split size.  A CTA has a fixed cost (length lookup, Q load, pipeline fill, cross-warp
// combine: ~2.8 us), so longer chunks move more bytes per CTA, but the launch still has
// to fill the machine and ragged batches need several CTAs per slot to balance.  Measured
// on B200 (bf16, D = 128, GB/s of KV):
//   many units (batch x KV heads x 16-query-head groups >= 256): 2048 keys is best or within
//     1 % of best (config 3, ragged: 6290 at 2048, 6120 at 4096, 5560 at 8192; config 5: 6110
//     at 2048, 5600 at 4096);
//   few units: the longest power-of-two chunk that still gives one CTA per SM (batch 8 x 32768
//     keys: 6630 at 8192, 5870 at 1024; batch 1 x 131072: 5900 at 4096, 3270 at 512; batch 4, 128
//     query heads: 4650 at 2048, 2140 at 256; batch 3 x 20000: 4980 at 2048, 4310 at 1024).
//     Chunks cut to fill exactly one wave of 296 CTAs (e.g. 3584 keys) measured 4-7 % slower
//     than the neighbouring power of two.
static int decode_chunk(const b200attn_decode_args* a) {
  if (a->chunk_tokens > 0) return a->chunk_tokens;
  const long long group = a->heads_kv > 0 ? a->heads_q / a->heads_kv : 1;
  const long long units = (long long)a->batch * a->heads_kv * ((group + 15) / 16);
  const long long visible = decode_max_visible(a);
  if (units >= 256) return 2048;
  const int sizes[7] = {8192, 4096, 2048, 1024, 512, 256, 128};
  for (int c : sizes)
    if (units * ((visible + c - 1) / c) >= 148) return c;   // at least one CTA per SM
  return 128;
}

size_t decode_workspace_bytes(const b200attn_decode_args* a) {
  if (!a || a->batch <= 0 || a->heads_q <= 0 || a->head_dim <= 0) return 0;
  int chunk = decode_chunk(a);
  long long chunks = (decode_max_visible(a) + chunk - 1) / chunk;
  if (chunks < 1) chunks = 1;
  long long rows = (long long)a->batch * a->heads_q * chunks;
  return (size_t)(rows * a->head_dim * 4 + rows * 4);
}

static int validate_decode(const b200attn_decode_args* a, bool sparse, bool paged) {
  if (!a || !a->q || !a->k_cache || !a->v_cache || !a->o) return B200ATTN_ERR_NULL;
  if (!a->cu_seqlens == !a->seqlens) return B200ATTN_ERR_NULL;  // exactly one of the two
  if (a->dtype != B200ATTN_F16 && a->dtype != B200ATTN_BF16) return B200ATTN_ERR_DTYPE;
  if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 96 && a->head_dim != 128)
    return B200ATTN_ERR_HEAD_DIM;
  if (a->batch <= 0 || a->heads_q <= 0 || a->heads_kv <= 0 || a->max_seqlen < 0)
    return B200ATTN_ERR_SHAPE;
  if (a->batch > 65535) return B200ATTN_ERR_TOO_LARGE;
  if (a->heads_q % a->heads_kv != 0) return B200ATTN_ERR_GQA;
  const void* ptrs[3] = {a->q, a->k_cache, a->v_cache};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr & 15) return B200ATTN_ERR_ALIGN;
  if ((uintptr_t)a->o & 1) return B200ATTN_ERR_ALIGN;
  const long long strides[8] = {a->q_stride_b, a->q_stride_h, a->k_stride_b, a->k_stride_t,
                                a->k_stride_h, a->v_stride_b, a->v_stride_t, a->v_stride_h};
  for (long long s : strides)
    if (s % 8 != 0) return B200ATTN_ERR_STRIDE;
  int chunk = decode_chunk(a);
  if (chunk % 64 != 0 || chunk <= 0) return B200ATTN_ERR_SHAPE;
  int mode = sparse ? a->sparsity : B200ATTN_DENSE;
  if (mode == B200ATTN_WINDOW) {
    if (a->window_global < 0 || a->window_local < 0) return B200ATTN_ERR_MODE;
  } else if (mode == B200ATTN_BLOCK_LIST || (paged && mode == kPaged)) {
    if (!a->block_idx) return B200ATTN_ERR_NULL;
    if (a->block_size <= 0 || a->block_size % 16 != 0 || a->max_sel <= 0) return B200ATTN_ERR_MODE;
  } else if (mode != B200ATTN_DENSE) {
    return B200ATTN_ERR_MODE;
  }
  return B200ATTN_OK;
}

// Phase 2 right behind phase 1 on the stream, allowed to start its launch before phase 1 has
// fully drained (the kernel itself waits for phase 1's results): saves most of a launch gap,
// which counts when the whole decoding step is a few tens of microseconds.
template <typename T, int D>
static cudaError_t launch_combine(const DecodeParams& p, dim3 g2, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = g2;
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_combine_kernel<T, D>, p);
}

template <typename T, int D>
static int launch_decode_t(const DecodeParams& p, dim3 g1, dim3 g2, cudaStream_t stream) {
  decode_split_kernel<T, D><<<g1, kDecodeThreads, 0, stream>>>(p);
  if (launch_combine<T, D>(p, g2, stream) != cudaSuccess) return B200ATTN_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

template <typename T>
static int launch_decode_d(int D, const DecodeParams& p, dim3 g1, dim3 g2, cudaStream_t s) {
  switch (D) {
    case 32: return launch_decode_t<T, 32>(p, g1, g2, s);
    case 64: return launch_decode_t<T, 64>(p, g1, g2, s);
    case 96: return launch_decode_t<T, 96>(p, g1, g2, s);
    default: return launch_decode_t<T, 128>(p, g1, g2, s);
  }
}


// ---- host side of the TMA variant
typedef CUresult (*DecEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static DecEncodeFn dec_encode_fn() {
  static DecEncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (DecEncodeFn)f;
  }();
  return fn;
}
// [D, keys, kv heads, batch] view of a cache, box = 64 x 16 x 1 x 1, 128-byte swizzle
static bool make_cache_tmap(CUtensorMap* m, int dtype, const void* base, int D, long long keys, int heads, int batch,
                            long long st, long long sh, long long sb) {
  DecEncodeFn enc = dec_encode_fn();
  if (!enc) return false;
  if (batch <= 1 || sb <= 0) sb = st * keys;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)keys, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)kBoxTok, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, dtype == B200ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int DP>
static int launch_decode_tma_d(const b200attn_decode_args* a, const DecodeParams& p, dim3 g1, dim3 g2,
                               cudaStream_t stream) {
  using L = DecodeTmaSmem<DP>;
  CUtensorMap tk, tv;
  if (!make_cache_tmap(&tk, a->dtype, a->k_cache, a->head_dim, p.map_keys, a->heads_kv, p.map_batch,
                       a->k_stride_t, a->k_stride_h, a->k_stride_b) ||
      !make_cache_tmap(&tv, a->dtype, a->v_cache, a->head_dim, p.map_keys, a->heads_kv, p.map_batch,
                       a->v_stride_t, a->v_stride_h, a->v_stride_b))
    return B200ATTN_ERR_CUDA;
  auto kern = decode_split_tma_kernel<T, DP>;
  // per device and cheap, so set on every call rather than remembered
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc) != cudaSuccess)
    return B200ATTN_ERR_CUDA;
  kern<<<g1, 160, L::kAlloc, stream>>>(tk, tv, p);
  cudaError_t e;
  switch (a->head_dim) {
    case 32: e = launch_combine<T, 32>(p, g2, stream); break;
    case 64: e = launch_combine<T, 64>(p, g2, stream); break;
    case 96: e = launch_combine<T, 96>(p, g2, stream); break;
    default: e = launch_combine<T, 128>(p, g2, stream); break;
  }
  if (e != cudaSuccess) return B200ATTN_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

template <typename T>
static int launch_decode_tma(const b200attn_decode_args* a, const DecodeParams& p, dim3 g1, dim3 g2,
                             cudaStream_t stream) {
  return a->head_dim <= 64 ? launch_decode_tma_d<T, 64>(a, p, g1, g2, stream)
                           : launch_decode_tma_d<T, 128>(a, p, g1, g2, stream);
}

// scratch == nullptr: use the caller's workspace from the args.
// pool_keys > 0: the caches are page pools of that many rows and a->sparsity is kPaged.
static int decode_fwd_impl(const b200attn_decode_args* a, bool sparse, long long pool_keys, void* scratch,
                           size_t scratch_bytes, cudaStream_t stream) {
  int st = validate_decode(a, sparse, pool_keys > 0);
  if (st != B200ATTN_OK) return st;
  b200attn_decode_args eff = *a;
  if (!sparse) eff.sparsity = B200ATTN_DENSE;
  void* ws = scratch ? scratch : a->workspace;
  size_t ws_bytes = scratch ? scratch_bytes : a->workspace_bytes;
  size_t need = decode_workspace_bytes(&eff);
  if (!ws || ws_bytes < need) return scratch ? B200ATTN_ERR_TOO_LARGE : B200ATTN_ERR_WORKSPACE;
  if ((uintptr_t)ws & 15) return B200ATTN_ERR_ALIGN;
  st = device_info(nullptr);
  if (st != B200ATTN_OK) return st;

  DecodeParams p;
  p.q = a->q; p.k = a->k_cache; p.v = a->v_cache; p.o = a->o;
  p.cu_seqlens = a->cu_seqlens; p.seqlens = a->seqlens;
  p.block_idx = a->block_idx; p.block_cnt = a->block_cnt;
  p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
  p.k_sb = a->k_stride_b; p.k_st = a->k_stride_t; p.k_sh = a->k_stride_h;
  p.v_sb = a->v_stride_b; p.v_st = a->v_stride_t; p.v_sh = a->v_stride_h;
  p.o_sb = a->o_stride_b; p.o_sh = a->o_stride_h;
  p.batch = a->batch; p.heads_q = a->heads_q; p.heads_kv = a->heads_kv;
  p.group = a->heads_q / a->heads_kv;
  p.ggroups = (p.group + 7) / 8;
  p.chunk = decode_chunk(&eff);
  p.max_chunks = (decode_max_visible(&eff) + p.chunk - 1) / p.chunk;
  if (p.max_chunks < 1) p.max_chunks = 1;
  p.sparsity = eff.sparsity;
  p.win_global = a->window_global; p.win_local = a->window_local;
  p.block_size = a->block_size; p.max_sel = a->max_sel;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.head_dim_rt = a->head_dim;
  p.max_seqlen = a->max_seqlen;
  p.status_word = a->status_word;
  // keys beyond max_seqlen are never visible; the copy engine zero-fills past the extent
  p.map_keys = pool_keys > 0 ? pool_keys : a->max_seqlen;
  p.map_batch = pool_keys > 0 ? 1 : a->batch;
  long long rows = (long long)a->batch * a->heads_q * p.max_chunks;
  p.part_o = (float*)ws;
  p.part_lse = p.part_o + rows * a->head_dim;
  if (p.max_chunks > 65535) return B200ATTN_ERR_TOO_LARGE;

  dim3 g2(a->heads_q, a->batch);
  set_launch_count(2);
  // bulk-copy path unless a window edge is not 16-key aligned (a box must not straddle it)
  const bool tma_ok = !(eff.sparsity == B200ATTN_WINDOW && (a->window_global % kBoxTok) != 0) &&
                      a->max_seqlen > 0;
  if (tma_ok) {
    p.ggroups = (p.group + 15) / 16;
    dim3 g1t(a->heads_kv * p.ggroups, p.max_chunks, a->batch);
    return a->dtype == B200ATTN_F16 ? launch_decode_tma<__half>(a, p, g1t, g2, stream)
                                    : launch_decode_tma<__nv_bfloat16>(a, p, g1t, g2, stream);
  }
  dim3 g1(a->heads_kv * p.ggroups, p.max_chunks, a->batch);
  return a->dtype == B200ATTN_F16 ? launch_decode_d<__half>(a->head_dim, p, g1, g2, stream)
                                  : launch_decode_d<__nv_bfloat16>(a->head_dim, p, g1, g2, stream);
}

int decode_fwd(const b200attn_decode_args* a, bool sparse, void* scratch, size_t scratch_bytes,
               cudaStream_t stream) {
  if (a && sparse && a->sparsity == kPaged) return B200ATTN_ERR_MODE;   // only reachable through paged_decode_fwd
  return decode_fwd_impl(a, sparse, 0, scratch, scratch_bytes, stream);
}

// --------------------------------------------------------------------------
// Paged KV: the caches are pools [num_pages, page_size, heads_kv, head_dim] and a
// page table says where the pages of each sequence are.  Page p of the pool is
// rows p * page_size .. of a flat [num_pages * page_size] key axis, so a page
// table is a block list over that axis that covers every key of the sequence.
// --------------------------------------------------------------------------
static int paged_as_decode_args(const b200attn_paged_decode_args* g, b200attn_decode_args* a) {
  if (!g) return B200ATTN_ERR_NULL;
  if (!g->page_table || !g->seqlens) return B200ATTN_ERR_NULL;
  if (g->page_size <= 0 || g->page_size % 16 != 0 || g->num_pages <= 0 || g->max_pages_per_seq <= 0)
    return B200ATTN_ERR_MODE;
  if (g->k_stride_page != (int64_t)g->page_size * g->k_stride_t ||
      g->v_stride_page != (int64_t)g->page_size * g->v_stride_t)
    return B200ATTN_ERR_STRIDE;   // pages must follow one another on the key axis
  *a = b200attn_decode_args{};
  a->q = g->q; a->k_cache = g->k_pages; a->v_cache = g->v_pages; a->o = g->o;
  a->dtype = g->dtype;
  a->batch = g->batch; a->heads_q = g->heads_q; a->heads_kv = g->heads_kv; a->head_dim = g->head_dim;
  a->max_seqlen = g->max_seqlen;
  a->seqlens = g->seqlens;
  a->q_stride_b = g->q_stride_b; a->q_stride_h = g->q_stride_h;
  a->k_stride_b = 0; a->k_stride_t = g->k_stride_t; a->k_stride_h = g->k_stride_h;
  a->v_stride_b = 0; a->v_stride_t = g->v_stride_t; a->v_stride_h = g->v_stride_h;
  a->o_stride_b = g->o_stride_b; a->o_stride_h = g->o_stride_h;
  a->softmax_scale = g->softmax_scale;
  a->chunk_tokens = g->chunk_tokens;
  a->sparsity = kPaged;
  a->block_idx = g->page_table;
  a->block_size = g->page_size;
  a->max_sel = g->max_pages_per_seq;
  a->workspace = g->workspace; a->workspace_bytes = g->workspace_bytes;
  a->status_word = g->status_word;
  return B200ATTN_OK;
}

size_t paged_decode_workspace_bytes(const b200attn_paged_decode_args* g) {
  b200attn_decode_args a;
  if (paged_as_decode_args(g, &a) != B200ATTN_OK) return 0;
  return decode_workspace_bytes(&a);
}

int paged_decode_fwd(const b200attn_paged_decode_args* g, cudaStream_t stream) {
  b200attn_decode_args a;
  int st = paged_as_decode_args(g, &a);
  if (st != B200ATTN_OK) return st;
  return decode_fwd_impl(&a, true, (long long)g->num_pages * g->page_size, nullptr, 0, stream);
}

// --------------------------------------------------------------------------
// Decoding without any allocation by anyone: the split-KV partials live in a
// fixed array that is part of the loaded module instead of a caller workspace.
// --------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = (size_t)B200ATTN_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int decode_fwd_noalloc(const b200attn_decode_args* a, cudaStream_t stream) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* dev_ptr[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200ATTN_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      // In host code the array's name only stands for the symbol; the address
      // the kernels may use has to be asked for, once per device, while that
      // device is current.
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return B200ATTN_ERR_CUDA;
      dev_ptr[dev] = ptr;
    }
    scratch = dev_ptr[dev];
  }
  return decode_fwd(a, false, scratch, kStaticScratchBytes, stream);
}

}  // namespace b200attn
