// KV-cache glue for sm_100a: packed varlen rows -> zero-padded cache, and the
// append of one new token per sequence.  These are the steps either side of
// decoding that the reference's tests do with Python loops
// (flash_attn_triton/flash_attn_decoding.py:404-425,
// flash_attn_triton/flash_attn_decoding_sparse.py:445-466).  Pure byte moves:
// 16-byte vector copies, one warp per (token, head) row, bound by HBM.
#include "common.cuh"

namespace b200attn {
namespace {

// cache[b, t, h, :] = t < len_b ? packed[cu[b] + t, h, :] : 0   for t < capacity
__global__ void pack_to_cache_kernel(const uint4* __restrict__ packed, uint4* __restrict__ cache,
                                     const int32_t* __restrict__ cu, long long p_st, long long p_sh,
                                     long long c_sb, long long c_st, long long c_sh, int batch, int capacity,
                                     int heads, int vec_per_row, int zero_pad) {
  // one warp per (b, t, h) row; strides are in 16-byte units
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)batch * capacity * heads;
  if (row >= total) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(row % heads);
  const long long bt = row / heads;
  const int t = (int)(bt % capacity), b = (int)(bt / capacity);
  const int s0 = cu[b], len = cu[b + 1] - s0;
  uint4* dst = cache + b * c_sb + t * c_st + h * c_sh;
  if (t < len) {
    const uint4* src = packed + (long long)(s0 + t) * p_st + h * p_sh;
    for (int i = lane; i < vec_per_row; i += 32) dst[i] = src[i];
  } else if (zero_pad) {
    for (int i = lane; i < vec_per_row; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
  }
}

// cache[b, len_b, h, :] = new_rows[b, h, :]   (rows with len_b >= capacity are skipped)
__global__ void append_kernel(const uint4* __restrict__ new_k, const uint4* __restrict__ new_v,
                              uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                              const int32_t* __restrict__ seqlens, long long n_sb, long long n_sh,
                              long long c_sb, long long c_st, long long c_sh, int batch, int capacity,
                              int heads, int vec_per_row) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long long)batch * heads) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(row % heads), b = (int)(row / heads);
  const int pos = seqlens[b];
  if (pos < 0 || pos >= capacity) return;
  const long long src = b * n_sb + h * n_sh, dst = b * c_sb + (long long)pos * c_st + h * c_sh;
  for (int i = lane; i < vec_per_row; i += 32) {
    k_cache[dst + i] = new_k[src + i];
    v_cache[dst + i] = new_v[src + i];
  }
}

}  // namespace

int kv_pack_to_cache(const b200attn_kv_pack_args* a, cudaStream_t stream) {
  if (!a || !a->packed || !a->cache || !a->cu_seqlens) return B200ATTN_ERR_NULL;
  if (a->batch <= 0 || a->heads <= 0 || a->capacity <= 0) return B200ATTN_ERR_SHAPE;
  if (a->head_dim <= 0 || a->head_dim % 8 != 0) return B200ATTN_ERR_HEAD_DIM;
  if (((uintptr_t)a->packed | (uintptr_t)a->cache) & 15) return B200ATTN_ERR_ALIGN;
  const long long strides[5] = {a->packed_stride_t, a->packed_stride_h, a->cache_stride_b,
                                a->cache_stride_t, a->cache_stride_h};
  for (long long s : strides)
    if (s % 8 != 0 || s < 0) return B200ATTN_ERR_STRIDE;
  const long long rows = (long long)a->batch * a->capacity * a->heads;
  const int wpb = 8;
  const long long blocks = (rows + wpb - 1) / wpb;
  if (blocks > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  if (int dst = device_info(nullptr)) return dst;
  pack_to_cache_kernel<<<(unsigned)blocks, wpb * 32, 0, stream>>>(
      (const uint4*)a->packed, (uint4*)a->cache, a->cu_seqlens, a->packed_stride_t / 8, a->packed_stride_h / 8,
      a->cache_stride_b / 8, a->cache_stride_t / 8, a->cache_stride_h / 8, a->batch, a->capacity, a->heads,
      a->head_dim / 8, a->zero_pad);
  set_launch_count(1);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

int kv_append(const b200attn_kv_append_args* a, cudaStream_t stream) {
  if (!a || !a->new_k || !a->new_v || !a->k_cache || !a->v_cache || !a->seqlens) return B200ATTN_ERR_NULL;
  if (a->batch <= 0 || a->heads <= 0 || a->capacity <= 0) return B200ATTN_ERR_SHAPE;
  if (a->head_dim <= 0 || a->head_dim % 8 != 0) return B200ATTN_ERR_HEAD_DIM;
  if (((uintptr_t)a->new_k | (uintptr_t)a->new_v | (uintptr_t)a->k_cache | (uintptr_t)a->v_cache) & 15)
    return B200ATTN_ERR_ALIGN;
  const long long strides[5] = {a->new_stride_b, a->new_stride_h, a->cache_stride_b, a->cache_stride_t,
                                a->cache_stride_h};
  for (long long s : strides)
    if (s % 8 != 0 || s < 0) return B200ATTN_ERR_STRIDE;
  const long long rows = (long long)a->batch * a->heads;
  const int wpb = 8;
  if (int dst = device_info(nullptr)) return dst;
  append_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
      (const uint4*)a->new_k, (const uint4*)a->new_v, (uint4*)a->k_cache, (uint4*)a->v_cache, a->seqlens,
      a->new_stride_b / 8, a->new_stride_h / 8, a->cache_stride_b / 8, a->cache_stride_t / 8,
      a->cache_stride_h / 8, a->batch, a->capacity, a->heads, a->head_dim / 8);
  set_launch_count(1);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

}  // namespace b200attn
