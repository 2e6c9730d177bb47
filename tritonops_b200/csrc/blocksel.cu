// Block selection: device-side builders of the sorted KV-block lists that the
// block-list prefill and decoding kernels take.
//
//  * window covers: the blocks touched by the reference's "local window +
//    global prefix" pattern (flash_attn_sparse_attn_triton.py:125-129,178-183
//    for prefill, flash_attn_decoding_sparse.py:52-58,82-85 for decoding);
//  * top-k: the k best-scoring blocks per row by a radix select, written in
//    ascending block order.
//
// All of it is integer work on a few KB per row; the kernels are launch-latency
// bound and exist so that no host round trip sits between the pattern's
// producer and the attention launch.
#include "common.cuh"

namespace b200attn {

// ---------------------------------------------------------------- window cover, prefill
// Query block i sees KV block j <= i iff some (q in i, k in j) has k <= q and
// (q - k < L or k < G).  Closest pair of blocks j < i: q - k = (i-j-1)*bs + 1.
struct WindowCover {
  int a_end;   // blocks [0, a_end): global prefix
  int b_lo;    // blocks [b_lo, b_hi): local band
  int b_hi;
  __host__ __device__ int count() const {
    if (b_lo >= b_hi) return a_end;
    return b_lo <= a_end ? (b_hi > a_end ? b_hi : a_end) : a_end + (b_hi - b_lo);
  }
  // n-th selected block, n < count()
  __host__ __device__ int at(int n) const {
    if (b_lo >= b_hi || b_lo <= a_end) return n;
    return n < a_end ? n : b_lo + (n - a_end);
  }
};

__host__ __device__ inline WindowCover prefill_cover(int i, int bs, int L, int G) {
  WindowCover c;
  const long long gb = G > 0 ? ((long long)G + bs - 1) / bs : 0;
  c.a_end = (int)(gb < i + 1 ? gb : i + 1);
  c.b_hi = i + 1;
  if (L <= 0) c.b_lo = c.b_hi;                       // no local part at all
  else if (L == 1) c.b_lo = i;                       // only q == k
  else {
    long long lo = (long long)i - 1 - (L - 2) / bs;
    c.b_lo = (int)(lo > 0 ? lo : 0);
  }
  return c;
}

__global__ void __launch_bounds__(128) window_blocks_prefill_kernel(b200attn_window_blocks_prefill_args a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + warp;
  const long long rows = (long long)a.batch * a.heads * a.n_qblocks;
  if (row >= rows) return;
  const int i = (int)(row % a.n_qblocks);
  const WindowCover c = prefill_cover(i, a.block_size, a.window_local, a.window_global);
  const int cnt = min(c.count(), a.max_nnz);
  int32_t* out = a.block_idx + row * a.max_nnz;
  for (int n = lane; n < a.max_nnz; n += 32) out[n] = n < cnt ? c.at(n) : -1;
  if (lane == 0) a.block_cnt[row] = cnt;
}

int32_t window_blocks_prefill_max_nnz(int32_t bs, int32_t L, int32_t G, int32_t n_qblocks) {
  if (bs <= 0 || n_qblocks <= 0) return 0;
  int best = 0;
  // the count grows with i until both ranges are fully inside; the last row has the most
  for (int i = n_qblocks - 1; i >= 0 && i >= n_qblocks - 2; --i) {
    int c = prefill_cover(i, bs, L, G).count();
    if (c > best) best = c;
  }
  return best;
}

int window_blocks_prefill(const b200attn_window_blocks_prefill_args* a, cudaStream_t stream) {
  if (!a || !a->block_idx || !a->block_cnt) return B200ATTN_ERR_NULL;
  if (a->batch <= 0 || a->heads <= 0 || a->n_qblocks <= 0 || a->max_nnz <= 0 || a->block_size <= 0)
    return B200ATTN_ERR_SHAPE;
  if (a->window_local < 0 || a->window_global < 0) return B200ATTN_ERR_MODE;
  if (a->max_nnz < window_blocks_prefill_max_nnz(a->block_size, a->window_local, a->window_global, a->n_qblocks))
    return B200ATTN_ERR_TOO_LARGE;
  const long long rows = (long long)a->batch * a->heads * a->n_qblocks;
  const long long ctas = (rows + 3) / 4;
  if (ctas > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  if (int dst = device_info(nullptr)) return dst;
  set_launch_count(1);
  window_blocks_prefill_kernel<<<(unsigned)ctas, 128, 0, stream>>>(*a);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

// ---------------------------------------------------------------- window cover, decoding
__global__ void __launch_bounds__(128) window_blocks_decode_kernel(b200attn_window_blocks_decode_args a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + warp;
  const long long rows = (long long)a.batch * a.heads_kv;
  if (row >= rows) return;
  const int b = (int)(row / a.heads_kv);
  const int len = max(a.seqlens ? a.seqlens[b] : a.cu_seqlens[b + 1] - a.cu_seqlens[b], 0);
  const int bs = a.block_size;
  // keys j < g, and keys start2 <= j < len  (flash_attn_decoding_sparse.py:82-85)
  const int g = min(a.window_global, len);
  const int start2 = max(len - a.window_local, g);
  WindowCover c;
  c.a_end = (g + bs - 1) / bs;
  c.b_lo = start2 / bs;
  c.b_hi = start2 < len ? (len + bs - 1) / bs : c.b_lo;
  const int cnt = min(c.count(), a.max_sel);
  int32_t* out = a.block_idx + row * a.max_sel;
  for (int n = lane; n < a.max_sel; n += 32) out[n] = n < cnt ? c.at(n) : -1;
  if (lane == 0) a.block_cnt[row] = cnt;
}

int window_blocks_decode(const b200attn_window_blocks_decode_args* a, cudaStream_t stream) {
  if (!a || !a->block_idx || !a->block_cnt) return B200ATTN_ERR_NULL;
  if (!a->cu_seqlens == !a->seqlens) return B200ATTN_ERR_NULL;
  if (a->batch <= 0 || a->heads_kv <= 0 || a->max_sel <= 0 || a->block_size <= 0) return B200ATTN_ERR_SHAPE;
  if (a->window_local < 0 || a->window_global < 0) return B200ATTN_ERR_MODE;
  const long long rows = (long long)a->batch * a->heads_kv;
  if (int dst = device_info(nullptr)) return dst;
  set_launch_count(1);
  window_blocks_decode_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, stream>>>(*a);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

// ---------------------------------------------------------------- top-k
constexpr int kTopkThreads = 256;
constexpr int kTopkMaxBlocks = 8192;

// Monotone map fp32 -> uint32: larger score, larger key; NaN -> 0 (below -inf,
// whose key is 0x007fffff); -0 counts as +0.
__device__ __forceinline__ uint32_t score_key(float x) {
  if (x != x) return 0u;
  uint32_t u = __float_as_uint(x + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix sum of one int per thread over the CTA; `total` gets the sum
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();   // warp_sums may still be read from a previous scan
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kTopkThreads / 32; ++w) {
    const int s = warp_sums[w];
    if (w < warp) base += s;
    tot += s;
  }
  total = tot;
  return base + inc - v;
}

__global__ void __launch_bounds__(kTopkThreads) topk_blocks_kernel(b200attn_topk_blocks_args a) {
  extern __shared__ uint32_t keys[];   // [n_blocks]
  __shared__ int hist[256];
  __shared__ int warp_sums[kTopkThreads / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  int nv = a.n_valid ? a.n_valid[row] : a.n_blocks;
  nv = max(0, min(nv, a.n_blocks));
  const int k = min(a.top_k, nv);
  const float* srow = a.scores + (long long)row * a.score_stride_row;
  for (int j = tid; j < nv; j += kTopkThreads) {
    const bool forced = j < a.force_first || j >= nv - a.force_last;
    keys[j] = forced ? 0xffffffffu : score_key(srow[j]);
  }
  if (tid == 0) { s_prefix = 0u; s_remaining = k; }
  __syncthreads();

  // radix select, most significant byte first: after the four passes s_prefix is
  // the k-th largest key T and s_remaining how many keys equal to T belong to the top k
  uint32_t mask = 0u;
  if (k < nv) {
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      for (int j = tid; j < nv; j += kTopkThreads) {
        const uint32_t key = keys[j];
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int remaining = s_remaining, cum = 0, d = 255;
        for (; d > 0; --d) {
          if (cum + hist[d] >= remaining) break;
          cum += hist[d];
        }
        s_remaining = remaining - cum;
        s_prefix = prefix | ((uint32_t)d << shift);
      }
      mask |= 255u << shift;
      __syncthreads();
    }
  }
  const uint32_t T = k < nv ? s_prefix : 0u;
  const int take_eq = k < nv ? s_remaining : nv;   // k == nv: every candidate (all keys >= 0)

  // each thread owns a contiguous run of blocks so that output order is block order
  const int per = (nv + kTopkThreads - 1) / kTopkThreads;
  const int j0 = min(tid * per, nv), j1 = min(j0 + per, nv);
  int n_eq = 0;
  for (int j = j0; j < j1; ++j) n_eq += keys[j] == T;
  int total;
  int eq_rank = block_exclusive_scan(n_eq, warp_sums, total);
  int n_sel = 0;
  {
    int e = eq_rank;
    for (int j = j0; j < j1; ++j) {
      const uint32_t key = keys[j];
      if (key > T) ++n_sel;
      else if (key == T) { n_sel += e < take_eq; ++e; }
    }
  }
  int pos = block_exclusive_scan(n_sel, warp_sums, total);
  int32_t* out = a.block_idx + (long long)row * a.top_k;
  {
    int e = eq_rank;
    for (int j = j0; j < j1; ++j) {
      const uint32_t key = keys[j];
      bool sel = key > T;
      if (key == T) { sel = e < take_eq; ++e; }
      if (sel && pos < a.top_k) out[pos++] = j;
    }
  }
  for (int n = k + tid; n < a.top_k; n += kTopkThreads) out[n] = -1;
  if (tid == 0) a.block_cnt[row] = k;
}

int topk_blocks(const b200attn_topk_blocks_args* a, cudaStream_t stream) {
  if (!a || !a->scores || !a->block_idx || !a->block_cnt) return B200ATTN_ERR_NULL;
  if (a->rows <= 0 || a->n_blocks <= 0 || a->top_k <= 0 || a->score_stride_row < a->n_blocks)
    return B200ATTN_ERR_SHAPE;
  if (a->force_first < 0 || a->force_last < 0) return B200ATTN_ERR_MODE;
  if (a->n_blocks > kTopkMaxBlocks) return B200ATTN_ERR_TOO_LARGE;
  if (int dst = device_info(nullptr)) return dst;
  set_launch_count(1);
  topk_blocks_kernel<<<a->rows, kTopkThreads, (size_t)a->n_blocks * 4, stream>>>(*a);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

}  // namespace b200attn
