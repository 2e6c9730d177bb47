// RMSNorm forward and backward for sm_100a (HBM-bound row reductions).
// Stands in for rmsnorm_fwd_kernel / rmsnorm_bwd_kernel and their autograd function
// (common/rms.py:9-88, :91-218, :221-355 of the reference).
//
//   r_t  = (mean_d x_td^2 + eps)^-1/2          y_td = x_td r_t w_d
//   dx_td = r_t (w_d dy_td - x_td r_t^2 mean_d'(dy_td' w_d' x_td'))
//   dw_d  = sum_t dy_td x_td r_t
//
// Forward: one warp per row, two passes over the row (the second one hits L1), 16-byte
// loads when the row is aligned for them.  Backward: a fixed number of CTAs each walk
// rows c, c + G, ...; the per-column dw sums stay in registers for the whole walk and
// are written as one partial row per CTA, which a second kernel adds up in a fixed
// order (the reference uses fp32 atomics, :217; this is deterministic).  All arithmetic
// is fp32 whatever the storage type.
#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {
namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kFwdWarps = 4;

template <typename T>
struct __align__(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

// N consecutive weights starting at column c (c a multiple of N, w 16-byte aligned) as floats,
// fetched with 16-byte loads
template <typename WT, int N>
__device__ __forceinline__ void load_weights(const WT* __restrict__ w, int c, float (&out)[N]) {
  constexpr int PER = 16 / sizeof(WT);          // weights per 16-byte load
  static_assert(N % PER == 0, "chunk of weights is a whole number of 16-byte loads");
#pragma unroll
  for (int j = 0; j < N / PER; ++j) {
    const Vec16<WT> v = *reinterpret_cast<const Vec16<WT>*>(w + c + PER * j);
#pragma unroll
    for (int i = 0; i < PER; ++i) out[PER * j + i] = to_f(v.v[i]);
  }
}

template <typename XT, typename WT, bool VECTOR>
__global__ void __launch_bounds__(32 * kFwdWarps)
rmsnorm_fwd_kernel(const XT* __restrict__ x, const WT* __restrict__ w, XT* __restrict__ y, float* __restrict__ rstd,
                   long long rows, int D, long long xs, long long ys, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kFwdWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const XT* xr = x + row * xs;
  XT* yr = y + row * ys;
  constexpr int N = Vec16<XT>::N;
  float ss = 0.f;
  if (VECTOR) {
    for (int c = lane * N; c < D; c += 32 * N) {
      const Vec16<XT> v = *reinterpret_cast<const Vec16<XT>*>(xr + c);
#pragma unroll
      for (int i = 0; i < N; ++i) { const float f = to_f(v.v[i]); ss = fmaf(f, f, ss); }
    }
  } else {
    for (int c = lane; c < D; c += 32) { const float f = to_f(xr[c]); ss = fmaf(f, f, ss); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = 1.f / sqrtf(eps + ss / (float)D);   // the reference's form (common/rms.py:68)
  if (VECTOR) {
    for (int c = lane * N; c < D; c += 32 * N) {
      const Vec16<XT> v = *reinterpret_cast<const Vec16<XT>*>(xr + c);
      float wf[N];
      load_weights<WT, N>(w, c, wf);
      Vec16<XT> o;
#pragma unroll
      for (int i = 0; i < N; ++i) o.v[i] = from_f<XT>(to_f(v.v[i]) * r * wf[i]);
      *reinterpret_cast<Vec16<XT>*>(yr + c) = o;
    }
  } else {
    for (int c = lane; c < D; c += 32) yr[c] = from_f<XT>(to_f(xr[c]) * r * to_f(w[c]));
  }
  if (lane == 0 && rstd) rstd[row] = r;
}

// Rows that fit in registers (CH 16-byte chunks per lane, dim <= 32 * N * CH): one pass.
template <typename XT, typename WT, int CH>
__global__ void __launch_bounds__(32 * kFwdWarps)
rmsnorm_fwd_reg_kernel(const XT* __restrict__ x, const WT* __restrict__ w, XT* __restrict__ y,
                       float* __restrict__ rstd, long long rows, int D, long long xs, long long ys, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kFwdWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const XT* xr = x + row * xs;
  XT* yr = y + row * ys;
  constexpr int N = Vec16<XT>::N;
  Vec16<XT> v[CH];
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = (lane + 32 * k) * N;
    if (c < D) v[k] = *reinterpret_cast<const Vec16<XT>*>(xr + c);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    if ((lane + 32 * k) * N < D) {
#pragma unroll
      for (int i = 0; i < N; ++i) { const float f = to_f(v[k].v[i]); ss = fmaf(f, f, ss); }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = 1.f / sqrtf(eps + ss / (float)D);
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = (lane + 32 * k) * N;
    if (c < D) {
      float wf[N];
      load_weights<WT, N>(w, c, wf);
      Vec16<XT> o;
#pragma unroll
      for (int i = 0; i < N; ++i) o.v[i] = from_f<XT>(to_f(v[k].v[i]) * r * wf[i]);
      *reinterpret_cast<Vec16<XT>*>(yr + c) = o;
    }
  }
  if (lane == 0 && rstd) rstd[row] = r;
}

// ---------------------------------------------------------------------------
// Streaming forward for rows of 2 .. 16 KB: one persistent CTA per SM; a producer warp brings
// groups of rows into a three-stage ring of 64 KB stages with untiled bulk copies, so the bytes
// in flight per SM are set by the ring (up to 192 KB) instead of by how many loads the resident
// warps have outstanding, and eight consumer warps take one row each: sum of squares from
// shared memory, then scale and store with 16-byte stores.  The weights sit in shared memory as
// fp32 for the whole kernel.
// ---------------------------------------------------------------------------
constexpr int kStreamConsumers = 8;
constexpr int kStreamThreads = 32 * (kStreamConsumers + 1);
constexpr int kStreamStages = 3;
constexpr int kStreamStageBytes = 64 * 1024;

struct StreamSmem {
  static constexpr int kWeights = kStreamStages * kStreamStageBytes;       // fp32 [D]
  static int bars(int D) { return kWeights + ((D * 4 + 127) & ~127); }
  static int bytes(int D) { return bars(D) + 2 * kStreamStages * 8 + 16 + 128; }   // + slack to align the base
};

template <typename XT, typename WT>
__global__ void __launch_bounds__(kStreamThreads, 1)
rmsnorm_fwd_stream_kernel(const XT* __restrict__ x, const WT* __restrict__ w, XT* __restrict__ y,
                          float* __restrict__ rstd, long long rows, int D, long long xs, long long ys, float eps,
                          int rows_per_stage, int* status_word) {
  using namespace sm100;
  constexpr int N = Vec16<XT>::N;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  float* sw = reinterpret_cast<float*>(sgen + StreamSmem::kWeights);
  const int bar_off = StreamSmem::kWeights + ((D * 4 + 127) & ~127);
  const uint32_t bars = sbase + bar_off;
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (kStreamStages + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + bar_off + 2 * kStreamStages * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)D * sizeof(XT);
  const long long n_groups = (rows + rows_per_stage - 1) / rows_per_stage;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStreamStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), kStreamConsumers); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == kStreamConsumers) {
    // ================================================================ producer
    if (lane == 0) {
      int it = 0, issued = 0;
      for (long long g = blockIdx.x; g < n_groups; g += gridDim.x, ++it, ++issued) {
        const int s = it % kStreamStages;
        if (!mbar_wait(empty(s), ((it / kStreamStages) & 1) ^ 1, abort_flag)) break;
        const long long r0 = g * rows_per_stage;
        const int n = (int)min((long long)rows_per_stage, rows - r0);
        mbar_expect_tx(full(s), (uint32_t)n * row_bytes);
        for (int r = 0; r < n; ++r)
          bulk_load_1d(sbase + s * kStreamStageBytes + r * row_bytes, x + (r0 + r) * xs, row_bytes, full(s));
      }
      if (*abort_flag)      // the consumers no longer wait for the stages: no copy may outlive the CTA
        for (int i = max(issued - kStreamStages, 0); i < issued; ++i)
          mbar_drain(full(i % kStreamStages), (i / kStreamStages) & 1);
    }
    return;
  }

  // ==================================================================== consumers
  for (int c = threadIdx.x; c < D; c += 32 * kStreamConsumers) sw[c] = to_f(w[c]);
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kStreamConsumers) : "memory");
  const float inv_d = 1.f / (float)D;
  const int chunks = D / N;
  int it = 0;
  for (long long g = blockIdx.x; g < n_groups; g += gridDim.x, ++it) {
    const int s = it % kStreamStages;
    if (!mbar_wait(full(s), (it / kStreamStages) & 1, abort_flag)) break;
    const long long r0 = g * rows_per_stage;
    const int n = (int)min((long long)rows_per_stage, rows - r0);
    for (int r = warp; r < n; r += kStreamConsumers) {
      const uint8_t* srow = sgen + s * kStreamStageBytes + (size_t)r * row_bytes;
      float ss0 = 0.f, ss1 = 0.f;
#pragma unroll 4
      for (int c = lane; c < chunks; c += 32) {
        const Vec16<XT> v = *reinterpret_cast<const Vec16<XT>*>(srow + 16 * c);
#pragma unroll
        for (int i = 0; i < N; i += 2) {
          const float f0 = to_f(v.v[i]), f1 = to_f(v.v[i + 1]);
          ss0 = fmaf(f0, f0, ss0);
          ss1 = fmaf(f1, f1, ss1);
        }
      }
      float ss = ss0 + ss1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rr = 1.f / sqrtf(eps + ss * inv_d);   // the reference's form (common/rms.py:68)
      XT* yr = y + (r0 + r) * ys;
#pragma unroll 4
      for (int c = lane; c < chunks; c += 32) {
        const Vec16<XT> v = *reinterpret_cast<const Vec16<XT>*>(srow + 16 * c);
        Vec16<XT> o;
#pragma unroll
        for (int i = 0; i < N; i += 4) {
          const float4 wf = *reinterpret_cast<const float4*>(sw + c * N + i);
          o.v[i] = from_f<XT>(to_f(v.v[i]) * rr * wf.x);
          o.v[i + 1] = from_f<XT>(to_f(v.v[i + 1]) * rr * wf.y);
          o.v[i + 2] = from_f<XT>(to_f(v.v[i + 2]) * rr * wf.z);
          o.v[i + 3] = from_f<XT>(to_f(v.v[i + 3]) * rr * wf.w);
        }
        *reinterpret_cast<Vec16<XT>*>(yr + c * N) = o;
      }
      if (lane == 0 && rstd) rstd[r0 + r] = rr;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty(s));
  }
  if (threadIdx.x == 0 && *abort_flag && status_word) atomicExch(status_word, 1);
}

// ---------------------------------------------------------------------------
// Streaming backward, rows of at least 2 KB and at most 4096 columns: one persistent CTA per SM.
// The ring holds (x row, dy row) pairs in slots of 16 KB filled by the producer warp in row
// order; consumer warp i takes the CTA's rows i, i + 8, ...: pass 1 sums dy w x over the row,
// pass 2 writes dx and adds dy x r into per-column dw sums that stay in the lane's registers
// for the whole kernel (CH 16-byte chunks per lane).  At the end the eight warps' dw rows are
// added in a fixed order through the (by then idle) ring and leave as one partial row per CTA.
// ---------------------------------------------------------------------------
constexpr int kBwdSlotBytes = 16 * 1024;
// seven consumer warps and the producer: 256 threads, so a consumer lane may hold the 128 dw sums
// of its columns and its working set in registers (nine warps would cap it at 168)
constexpr int kBwdStreamConsumers = 7;
constexpr int kBwdStreamThreads = 32 * (kBwdStreamConsumers + 1);
constexpr int kBwdSlots = kStreamStages * kStreamStageBytes / kBwdSlotBytes;   // 12

struct StreamBwdSmem {
  static constexpr int kWeights = kBwdSlots * kBwdSlotBytes;
  static int bars(int D) { return kWeights + ((D * 4 + 127) & ~127); }
  static int bytes(int D) { return bars(D) + 2 * kBwdSlots * 8 + 16 + 128; }
};

template <typename XT, typename WT, int CH>
__global__ void __launch_bounds__(kBwdStreamThreads, 1)
rmsnorm_bwd_stream_kernel(const XT* __restrict__ dy, const XT* __restrict__ x, const WT* __restrict__ w,
                          const float* __restrict__ rstd, XT* __restrict__ dx, float* __restrict__ partial,
                          long long rows, int D, long long dys, long long xs, long long dxs) {
  using namespace sm100;
  constexpr int N = Vec16<XT>::N;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  float* sw = reinterpret_cast<float*>(sgen + StreamBwdSmem::kWeights);
  const int bar_off = StreamBwdSmem::kWeights + ((D * 4 + 127) & ~127);
  const uint32_t bars = sbase + bar_off;
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (kBwdSlots + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + bar_off + 2 * kBwdSlots * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)D * sizeof(XT);
  // this CTA's rows: blockIdx.x, blockIdx.x + gridDim.x, ...
  const long long my_rows = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kBwdSlots; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == kBwdStreamConsumers) {
    // ================================================================ producer
    if (lane == 0) {
      long long issued = 0;
      for (long long it = 0; it < my_rows; ++it, ++issued) {
        const int s = (int)(it % kBwdSlots);
        if (!mbar_wait(empty(s), (uint32_t)((it / kBwdSlots) & 1) ^ 1u, abort_flag)) break;
        const long long row = blockIdx.x + it * gridDim.x;
        mbar_expect_tx(full(s), 2 * row_bytes);
        bulk_load_1d(sbase + s * kBwdSlotBytes, x + row * xs, row_bytes, full(s));
        bulk_load_1d(sbase + s * kBwdSlotBytes + kBwdSlotBytes / 2, dy + row * dys, row_bytes, full(s));
      }
      if (*abort_flag)
        for (long long i = issued > kBwdSlots ? issued - kBwdSlots : 0; i < issued; ++i)
          mbar_drain(full((int)(i % kBwdSlots)), (uint32_t)((i / kBwdSlots) & 1));
    }
  } else {
    // ================================================================== consumers
    for (int c = threadIdx.x; c < D; c += 32 * kBwdStreamConsumers) sw[c] = to_f(w[c]);
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
    const float inv_d = 1.f / (float)D;
    const int chunks = D / N;
    float dwv[CH][N];
#pragma unroll
    for (int k = 0; k < CH; ++k)
#pragma unroll
      for (int i = 0; i < N; ++i) dwv[k][i] = 0.f;
    for (long long it = warp; it < my_rows; it += kBwdStreamConsumers) {
      const int s = (int)(it % kBwdSlots);
      if (!mbar_wait(full(s), (uint32_t)((it / kBwdSlots) & 1), abort_flag)) break;
      const long long row = blockIdx.x + it * gridDim.x;
      const uint8_t* sx = sgen + s * kBwdSlotBytes;
      const uint8_t* sg = sx + kBwdSlotBytes / 2;
      const float r = rstd[row];
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = lane + 32 * k;
        if (c < chunks) {
          const Vec16<XT> xv = *reinterpret_cast<const Vec16<XT>*>(sx + 16 * c);
          const Vec16<XT> gv = *reinterpret_cast<const Vec16<XT>*>(sg + 16 * c);
#pragma unroll
          for (int i = 0; i < N; i += 4) {
            const float4 wf = *reinterpret_cast<const float4*>(sw + c * N + i);
            t0 = fmaf(to_f(gv.v[i]) * wf.x, to_f(xv.v[i]), t0);
            t1 = fmaf(to_f(gv.v[i + 1]) * wf.y, to_f(xv.v[i + 1]), t1);
            t0 = fmaf(to_f(gv.v[i + 2]) * wf.z, to_f(xv.v[i + 2]), t0);
            t1 = fmaf(to_f(gv.v[i + 3]) * wf.w, to_f(xv.v[i + 3]), t1);
          }
        }
      }
      float tot = t0 + t1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
      const float coef = tot * r * r * inv_d;
      XT* dr = dx + row * dxs;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = lane + 32 * k;
        if (c < chunks) {
          const Vec16<XT> xv = *reinterpret_cast<const Vec16<XT>*>(sx + 16 * c);
          const Vec16<XT> gv = *reinterpret_cast<const Vec16<XT>*>(sg + 16 * c);
          Vec16<XT> o;
#pragma unroll
          for (int i = 0; i < N; i += 4) {
            const float4 wf = *reinterpret_cast<const float4*>(sw + c * N + i);
            const float wv[4] = {wf.x, wf.y, wf.z, wf.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float xf = to_f(xv.v[i + j]), gf = to_f(gv.v[i + j]);
              o.v[i + j] = from_f<XT>(r * (wv[j] * gf - xf * coef));
              dwv[k][i + j] = fmaf(gf * xf, r, dwv[k][i + j]);
            }
          }
          *reinterpret_cast<Vec16<XT>*>(dr + c * N) = o;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(s));
    }
    // ---- the seven dw rows -> one partial row per CTA, added in warp order.  Every slot has
    // been consumed (or the CTA is aborting and the producer drains): the ring is free.
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
    if (!*abort_flag) {
      float* red = reinterpret_cast<float*>(sgen);     // [7][D] fp32 <= 112 KB of the 192 KB ring
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = lane + 32 * k;
        if (c < chunks) {
#pragma unroll
          for (int i = 0; i < N; i += 4)
            *reinterpret_cast<float4*>(red + (size_t)warp * D + c * N + i) =
                make_float4(dwv[k][i], dwv[k][i + 1], dwv[k][i + 2], dwv[k][i + 3]);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
      for (int c = threadIdx.x; c < D; c += 32 * kBwdStreamConsumers) {
        float sum = 0.f;
#pragma unroll
        for (int wq = 0; wq < kBwdStreamConsumers; ++wq) sum += red[(size_t)wq * D + c];
        partial[(long long)blockIdx.x * D + c] = sum;
      }
    }
  }
}

constexpr int kBwdThreadsRms = 256;
constexpr int kBwdMaxCols = 64;          // columns per thread: dim <= 256 * 64
constexpr int kBwdCtas = 148 * 4;

// KC: columns per thread (dim <= 256 * KC)
template <typename XT, typename WT, int KC>
__global__ void __launch_bounds__(kBwdThreadsRms)
rmsnorm_bwd_kernel(const XT* __restrict__ dy, const XT* __restrict__ x, const WT* __restrict__ w,
                   const float* __restrict__ rstd, XT* __restrict__ dx, float* __restrict__ partial, long long rows,
                   int D, long long dys, long long xs, long long dxs) {
  __shared__ float red[kBwdThreadsRms / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float wv[KC], dwv[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    const int c = tid + kBwdThreadsRms * k;
    wv[k] = c < D ? to_f(w[c]) : 0.f;
    dwv[k] = 0.f;
  }
  const float inv_d = 1.f / (float)D;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const XT* xr = x + row * xs;
    const XT* gr = dy + row * dys;
    XT* dr = dx + row * dxs;
    const float r = rstd[row];
    float xv[KC], gv[KC];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = tid + kBwdThreadsRms * k;
      xv[k] = c < D ? to_f(xr[c]) : 0.f;
      gv[k] = c < D ? to_f(gr[c]) : 0.f;
      s = fmaf(gv[k] * wv[k], xv[k], s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();            // `red` of the previous row has been read by everyone
    if (lane == 0) red[warp] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kBwdThreadsRms / 32; ++i) tot += red[i];
    const float coef = tot * r * r * inv_d;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = tid + kBwdThreadsRms * k;
      if (c < D) {
        dr[c] = from_f<XT>(r * (wv[k] * gv[k] - xv[k] * coef));
        dwv[k] = fmaf(gv[k] * xv[k], r, dwv[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    const int c = tid + kBwdThreadsRms * k;
    if (c < D) partial[(long long)blockIdx.x * D + c] = dwv[k];
  }
}

// Vector form: thread t owns the 16-byte chunks t, t + 256, ... (KC of them) of every row,
// dim <= 256 * N * KC, rows 16-byte aligned.
template <typename XT, typename WT, int KC>
__global__ void __launch_bounds__(kBwdThreadsRms)
rmsnorm_bwd_vec_kernel(const XT* __restrict__ dy, const XT* __restrict__ x, const WT* __restrict__ w,
                       const float* __restrict__ rstd, XT* __restrict__ dx, float* __restrict__ partial,
                       long long rows, int D, long long dys, long long xs, long long dxs) {
  __shared__ float red[kBwdThreadsRms / 32];
  constexpr int N = Vec16<XT>::N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float wv[KC][N], dwv[KC][N];
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    const int c = (tid + kBwdThreadsRms * k) * N;
#pragma unroll
    for (int i = 0; i < N; ++i) { wv[k][i] = c < D ? to_f(w[c + i]) : 0.f; dwv[k][i] = 0.f; }
  }
  const float inv_d = 1.f / (float)D;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const XT* xr = x + row * xs;
    const XT* gr = dy + row * dys;
    XT* dr = dx + row * dxs;
    Vec16<XT> xv[KC], gv[KC];
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = (tid + kBwdThreadsRms * k) * N;
      if (c < D) {
        xv[k] = *reinterpret_cast<const Vec16<XT>*>(xr + c);
        gv[k] = *reinterpret_cast<const Vec16<XT>*>(gr + c);
      }
    }
    const float r = rstd[row];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      if ((tid + kBwdThreadsRms * k) * N < D) {
#pragma unroll
        for (int i = 0; i < N; ++i) s = fmaf(to_f(gv[k].v[i]) * wv[k][i], to_f(xv[k].v[i]), s);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();            // `red` of the previous row has been read by everyone
    if (lane == 0) red[warp] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kBwdThreadsRms / 32; ++i) tot += red[i];
    const float coef = tot * r * r * inv_d;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = (tid + kBwdThreadsRms * k) * N;
      if (c < D) {
        Vec16<XT> o;
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float xf = to_f(xv[k].v[i]), gf = to_f(gv[k].v[i]);
          o.v[i] = from_f<XT>(r * (wv[k][i] * gf - xf * coef));
          dwv[k][i] = fmaf(gf * xf, r, dwv[k][i]);
        }
        *reinterpret_cast<Vec16<XT>*>(dr + c) = o;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    const int c = (tid + kBwdThreadsRms * k) * N;
    if (c < D) {
#pragma unroll
      for (int i = 0; i < N; ++i) partial[(long long)blockIdx.x * D + c + i] = dwv[k][i];
    }
  }
}

template <typename WT>
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, WT* __restrict__ dw, int D, int n_partial) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int i = 0; i < n_partial; ++i) s += partial[(long long)i * D + c];
  dw[c] = from_f<WT>(s);
}

bool valid_dtypes(int xd, int wd) {
  if (xd != B200ATTN_F16 && xd != B200ATTN_BF16 && xd != B200ATTN_F32) return false;
  return wd == xd || wd == B200ATTN_F32;
}
int elem_size(int d) { return d == B200ATTN_F32 ? 4 : 2; }

int bwd_ctas(long long rows) { return (int)(rows < kBwdCtas ? rows : kBwdCtas); }

template <typename XT, typename WT>
int launch_fwd(const b200attn_rmsnorm_fwd_args* a, cudaStream_t stream) {
  constexpr int N = Vec16<XT>::N;
  const bool vec = a->dim % N == 0 && a->x_stride_row % N == 0 && a->y_stride_row % N == 0 &&
                   ((uintptr_t)a->x & 15) == 0 && ((uintptr_t)a->y & 15) == 0 && ((uintptr_t)a->weight & 15) == 0;
  const long long ctas = (a->rows + kFwdWarps - 1) / kFwdWarps;
  if (ctas > 0x7fffffffLL) return B200ATTN_ERR_TOO_LARGE;
  // rows of 2 .. 16 KB, enough of them to fill the machine: the streaming kernel
  const long long row_bytes = (long long)a->dim * (long long)sizeof(XT);
  if (vec && row_bytes >= 2048 && row_bytes <= 16384 && a->dim * 4 <= 32768 && a->rows >= 1024) {
    const DeviceInfo* di = nullptr;
    if (int st = device_info(&di)) return st;
    int per_stage = (int)(kStreamStageBytes / row_bytes);
    if (per_stage > kStreamConsumers) per_stage = kStreamConsumers;
    const long long groups = (a->rows + per_stage - 1) / per_stage;
    const int grid = (int)(groups < di->sm_count ? groups : di->sm_count);
    auto kern = rmsnorm_fwd_stream_kernel<XT, WT>;
    const int smem = StreamSmem::bytes(a->dim);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return B200ATTN_ERR_CUDA;
    kern<<<grid, kStreamThreads, smem, stream>>>((const XT*)a->x, (const WT*)a->weight, (XT*)a->y, a->rstd, a->rows,
                                               a->dim, a->x_stride_row, a->y_stride_row, a->eps, per_stage, nullptr);
    set_launch_count(1);
    return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
  }
#define B200ATTN_RMS_FWD_REG(CH)                                                                          \
  rmsnorm_fwd_reg_kernel<XT, WT, CH><<<(unsigned)ctas, 32 * kFwdWarps, 0, stream>>>(                        \
      (const XT*)a->x, (const WT*)a->weight, (XT*)a->y, a->rstd, a->rows, a->dim, a->x_stride_row, a->y_stride_row, a->eps)
  if (vec && a->dim <= 32 * N * 4) B200ATTN_RMS_FWD_REG(4);
  else if (vec && a->dim <= 32 * N * 8) B200ATTN_RMS_FWD_REG(8);
  else if (vec && a->dim <= 32 * N * 16) B200ATTN_RMS_FWD_REG(16);
#undef B200ATTN_RMS_FWD_REG
  else if (vec)
    rmsnorm_fwd_kernel<XT, WT, true><<<(unsigned)ctas, 32 * kFwdWarps, 0, stream>>>(
        (const XT*)a->x, (const WT*)a->weight, (XT*)a->y, a->rstd, a->rows, a->dim, a->x_stride_row, a->y_stride_row, a->eps);
  else
    rmsnorm_fwd_kernel<XT, WT, false><<<(unsigned)ctas, 32 * kFwdWarps, 0, stream>>>(
        (const XT*)a->x, (const WT*)a->weight, (XT*)a->y, a->rstd, a->rows, a->dim, a->x_stride_row, a->y_stride_row, a->eps);
  set_launch_count(1);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

template <typename XT, typename WT>
int launch_bwd_rms(const b200attn_rmsnorm_bwd_args* a, cudaStream_t stream) {
  const int g = bwd_ctas(a->rows);
  float* partial = (float*)a->workspace;
  const XT *dy = (const XT*)a->dy, *x = (const XT*)a->x;
  const WT* w = (const WT*)a->weight;
  XT* dx = (XT*)a->dx;
  constexpr int N = Vec16<XT>::N;
  const bool vec = a->dim % N == 0 && a->x_stride_row % N == 0 && a->dy_stride_row % N == 0 &&
                   a->dx_stride_row % N == 0 && (((uintptr_t)a->x | (uintptr_t)a->dy | (uintptr_t)a->dx) & 15) == 0;
  // rows of at least 2 KB, at most 4096 columns (the dw sums of a row live in one warp's registers)
  const long long row_bytes = (long long)a->dim * (long long)sizeof(XT);
  if (vec && ((uintptr_t)a->weight & 15) == 0 && row_bytes >= 2048 && row_bytes <= kBwdSlotBytes / 2 && a->dim <= 4096 &&
      a->rows >= 1024) {
    const DeviceInfo* di = nullptr;
    if (int st = device_info(&di)) return st;
    const int grid = di->sm_count < g ? di->sm_count : g;     // partial rows: the workspace holds g of them
    const int smem = StreamBwdSmem::bytes(a->dim);
    const int ch = (a->dim / N + 31) / 32;                    // 16-byte chunks per lane
#define B200ATTN_RMS_BWD_STREAM(CH)                                                                               \
  {                                                                                                               \
    auto kern = rmsnorm_bwd_stream_kernel<XT, WT, CH>;                                                            \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)             \
      return B200ATTN_ERR_CUDA;                                                                                   \
    kern<<<grid, kBwdStreamThreads, smem, stream>>>(dy, x, w, a->rstd, dx, partial, a->rows, a->dim, a->dy_stride_row, \
                                                 a->x_stride_row, a->dx_stride_row);                              \
  }
    if (ch <= 4) B200ATTN_RMS_BWD_STREAM(4)
    else if (ch <= 8) B200ATTN_RMS_BWD_STREAM(8)
    else if (ch <= 16) B200ATTN_RMS_BWD_STREAM(16)
    else if constexpr (N == 4) B200ATTN_RMS_BWD_STREAM(32)     // (fp32 rows: 4 columns per chunk)
#undef B200ATTN_RMS_BWD_STREAM
    rmsnorm_dw_reduce_kernel<WT><<<(a->dim + 255) / 256, 256, 0, stream>>>(partial, (WT*)a->dweight, a->dim, grid);
    set_launch_count(2);
    return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
  }
  if (vec && a->dim <= kBwdThreadsRms * 16)
    rmsnorm_bwd_vec_kernel<XT, WT, 16 / N><<<g, kBwdThreadsRms, 0, stream>>>(
        dy, x, w, a->rstd, dx, partial, a->rows, a->dim, a->dy_stride_row, a->x_stride_row, a->dx_stride_row);
  else if (vec && a->dim <= kBwdThreadsRms * 32)
    rmsnorm_bwd_vec_kernel<XT, WT, 32 / N><<<g, kBwdThreadsRms, 0, stream>>>(
        dy, x, w, a->rstd, dx, partial, a->rows, a->dim, a->dy_stride_row, a->x_stride_row, a->dx_stride_row);
  else if (a->dim <= kBwdThreadsRms * 4)
    rmsnorm_bwd_kernel<XT, WT, 4><<<g, kBwdThreadsRms, 0, stream>>>(dy, x, w, a->rstd, dx, partial, a->rows, a->dim,
                                                                 a->dy_stride_row, a->x_stride_row, a->dx_stride_row);
  else if (a->dim <= kBwdThreadsRms * 16)
    rmsnorm_bwd_kernel<XT, WT, 16><<<g, kBwdThreadsRms, 0, stream>>>(dy, x, w, a->rstd, dx, partial, a->rows, a->dim,
                                                                  a->dy_stride_row, a->x_stride_row, a->dx_stride_row);
  else
    rmsnorm_bwd_kernel<XT, WT, kBwdMaxCols><<<g, kBwdThreadsRms, 0, stream>>>(
        dy, x, w, a->rstd, dx, partial, a->rows, a->dim, a->dy_stride_row, a->x_stride_row, a->dx_stride_row);
  rmsnorm_dw_reduce_kernel<WT><<<(a->dim + 255) / 256, 256, 0, stream>>>(partial, (WT*)a->dweight, a->dim, g);
  set_launch_count(2);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

}  // namespace

int rmsnorm_fwd(const b200attn_rmsnorm_fwd_args* a, cudaStream_t stream) {
  if (!a || !a->x || !a->weight || !a->y) return B200ATTN_ERR_NULL;
  if (!valid_dtypes(a->x_dtype, a->w_dtype)) return B200ATTN_ERR_DTYPE;
  if (a->rows < 0 || a->dim <= 0 || a->x_stride_row < a->dim || a->y_stride_row < a->dim) return B200ATTN_ERR_SHAPE;
  if (((uintptr_t)a->x | (uintptr_t)a->y) & (elem_size(a->x_dtype) - 1)) return B200ATTN_ERR_ALIGN;
  if (a->rows == 0) { set_launch_count(0); return B200ATTN_OK; }
  if (int dst = device_info(nullptr)) return dst;
  const bool wf = a->w_dtype == B200ATTN_F32;
  switch (a->x_dtype) {
    case B200ATTN_F32: return launch_fwd<float, float>(a, stream);
    case B200ATTN_F16: return wf ? launch_fwd<__half, float>(a, stream) : launch_fwd<__half, __half>(a, stream);
    default: return wf ? launch_fwd<__nv_bfloat16, float>(a, stream) : launch_fwd<__nv_bfloat16, __nv_bfloat16>(a, stream);
  }
}

size_t rmsnorm_bwd_workspace_bytes(const b200attn_rmsnorm_bwd_args* a) {
  if (!a || a->rows <= 0 || a->dim <= 0) return 0;
  return (size_t)bwd_ctas(a->rows) * a->dim * 4;
}

int rmsnorm_bwd(const b200attn_rmsnorm_bwd_args* a, cudaStream_t stream) {
  if (!a || !a->dy || !a->x || !a->weight || !a->rstd || !a->dx || !a->dweight) return B200ATTN_ERR_NULL;
  if (!valid_dtypes(a->x_dtype, a->w_dtype)) return B200ATTN_ERR_DTYPE;
  if (a->rows <= 0 || a->dim <= 0 || a->x_stride_row < a->dim || a->dy_stride_row < a->dim || a->dx_stride_row < a->dim)
    return B200ATTN_ERR_SHAPE;
  if (a->dim > kBwdThreadsRms * kBwdMaxCols) return B200ATTN_ERR_TOO_LARGE;
  if (!a->workspace || a->workspace_bytes < rmsnorm_bwd_workspace_bytes(a)) return B200ATTN_ERR_WORKSPACE;
  if ((uintptr_t)a->workspace & 3) return B200ATTN_ERR_ALIGN;
  if (int dst = device_info(nullptr)) return dst;
  const bool wf = a->w_dtype == B200ATTN_F32;
  switch (a->x_dtype) {
    case B200ATTN_F32: return launch_bwd_rms<float, float>(a, stream);
    case B200ATTN_F16: return wf ? launch_bwd_rms<__half, float>(a, stream) : launch_bwd_rms<__half, __half>(a, stream);
    default:
      return wf ? launch_bwd_rms<__nv_bfloat16, float>(a, stream) : launch_bwd_rms<__nv_bfloat16, __nv_bfloat16>(a, stream);
  }
}

}  // namespace b200attn
