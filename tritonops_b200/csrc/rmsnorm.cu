// RMSNorm forward and backward for sm_100a (HBM-bound row reductions).
// Stands in for rmsnorm_fwd_kernel / rmsnorm_bwd_kernel and their autograd function
// (common/rms.py:9-88, :91-218, :221-355 of the reference).
//
//   r_t  = (mean_d x_td^2 + eps)^-1/2          y_td = x_td r_t w_d
//   dx_td = r_t (w_d dy_td - x_td r_t^2 mean_d'(dy_td' w_d' x_td'))
//   dw_d  = sum_t dy_td x_td r_t
//
// Large inputs (1024 rows or more of 2 .. 12 KB) take the streaming kernels: persistent CTAs
// whose producer warp feeds a shared-memory ring with bulk copies.  Otherwise -- forward: one
// warp per row, two passes over the row (the second one hits L1), 16-byte loads when the row
// is aligned for them; backward: a fixed number of CTAs each walk rows c, c + G, ....  In every
// backward form the per-column dw sums stay in registers for the whole walk and leave as one
// partial row per CTA, which a second kernel adds up in a fixed order (the reference uses fp32
// atomics, :217; this is deterministic).  All arithmetic is fp32 whatever the storage type.
#include "common.cuh"
#include "sm100.cuh"

// Rows are read once: their bulk copies carry an L2 evict-first hint, which leaves L2 to the
// output lines that are still collecting writes (forward, bf16 65536 x 4096: 5.50 -> 5.66 TB/s;
// the same hint on the output stores changed nothing).
#ifndef B200ATTN_RMS_LOAD_HINT
#define B200ATTN_RMS_LOAD_HINT 1
#endif

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
// Streaming kernels for rows of 2 .. 12 KB (forward) / 2 .. 13.5 KB (backward): one persistent CTA per SM.  A producer warp brings
// the CTA's rows (blockIdx.x, blockIdx.x + gridDim.x, ...) one per slot into a 192 KB ring with
// untiled bulk copies, so the bytes in flight per SM are set by the ring instead of by how many
// loads the resident warps have outstanding; consumer warps take the rows in turn from shared
// memory.  The weights sit in shared memory as fp32 for the whole kernel.  The consumers'
// instruction streams are chains of dependent operations, so the kernels need many of them:
// with 8 consumer warps both were bound by issue latency (1.4 .. 1.8 instructions per clock
// per SM at 2 warps per scheduler), hence 16 / 14.
// Row `it` of the CTA lives in slot it % n_slots, whoever consumes it.  A slot's barriers are
// therefore read by different consumers in turn, and a phase parity alone cannot tell "my row
// has landed" from "the row before the previous one had landed" (bulk copies may complete out
// of order, so the row in between, another consumer's, may still be in flight).  Hence a
// consumer first waits until the slot's previous row has been released (the same wait the
// producer does before refilling it) and only then for its own row: from that point the only
// phase the slot's full barrier can complete is this row's.  (That first wait is itself free of
// aliasing because the producer issues rows in order and the ring has at least as many slots as
// there are consumers: a consumer's previous row having landed implies that the row before this
// one in the slot had been issued, hence that the one before that had been released.)
// ---------------------------------------------------------------------------
constexpr int kRingBytes = 192 * 1024;
constexpr int kMaxSlots = 96;

struct StreamSmem {
  static constexpr int kWeights = kRingBytes;                                  // fp32 [D]
  __host__ __device__ static int bars(int D) { return kWeights + ((D * 4 + 127) & ~127); }
  static int bytes(int D) { return bars(D) + 2 * kMaxSlots * 8 + 16 + 128; }   // + slack to align the base
};

// ---- forward: a row per consumer warp: sum of squares, then y = x r w written over the row in
// its slot and sent out as one bulk store.
constexpr int kFwdStreamConsumers = 16;
constexpr int kFwdStreamThreads = 32 * (kFwdStreamConsumers + 1);

template <typename XT, typename WT>
__global__ void __launch_bounds__(kFwdStreamThreads, 1)
rmsnorm_fwd_stream_kernel(const XT* __restrict__ x, const WT* __restrict__ w, XT* __restrict__ y,
                          float* __restrict__ rstd, long long rows, int D, long long xs, long long ys, float eps,
                          int slot_bytes, int n_slots) {
  using namespace sm100;
  constexpr int N = Vec16<XT>::N;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  float* sw = reinterpret_cast<float*>(sgen + StreamSmem::kWeights);
  const int bar_off = StreamSmem::bars(D);
  const uint32_t bars = sbase + bar_off;
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (kMaxSlots + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + bar_off + 2 * kMaxSlots * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)D * sizeof(XT);
  const long long my_rows = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < n_slots; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  auto slot_of = [&](long long it) { return (int)(it % n_slots); };
  auto use_of = [&](long long it) { return (uint32_t)((it / n_slots) & 1); };      // phase parity of row `it` in its slot

  if (warp == kFwdStreamConsumers) {
    // ================================================================ producer
    if (lane == 0) {
      long long issued = 0;
#if B200ATTN_RMS_LOAD_HINT
      const uint64_t pol = l2_policy_evict_first();
#endif
      for (long long it = 0; it < my_rows; ++it, ++issued) {
        const int s = slot_of(it);
        if (!mbar_wait(empty(s), use_of(it) ^ 1u, abort_flag)) break;
        mbar_expect_tx(full(s), row_bytes);
#if B200ATTN_RMS_LOAD_HINT
        bulk_load_1d_hint(sbase + s * slot_bytes, x + (blockIdx.x + it * gridDim.x) * xs, row_bytes, full(s), pol);
#else
        bulk_load_1d(sbase + s * slot_bytes, x + (blockIdx.x + it * gridDim.x) * xs, row_bytes, full(s));
#endif
      }
      if (*abort_flag) {    // the consumers no longer wait for the slots: no copy may outlive the CTA
        for (long long i = issued > n_slots ? issued - n_slots : 0; i < issued; ++i) mbar_drain(full(slot_of(i)), use_of(i));
      }
    }
    return;
  }

  // ==================================================================== consumers
  for (int c = threadIdx.x; c < D; c += 32 * kFwdStreamConsumers) sw[c] = to_f(w[c]);
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kFwdStreamConsumers) : "memory");
  const float inv_d = 1.f / (float)D;
  const int chunks = D / N;
  for (long long it = warp; it < my_rows; it += kFwdStreamConsumers) {
    const int s = slot_of(it);
    if (!mbar_wait(empty(s), use_of(it) ^ 1u, abort_flag)) break;     // the slot's previous row has been released ...
    if (!mbar_wait(full(s), use_of(it), abort_flag)) break;           // ... so this can only be row `it` landing
    const long long row = blockIdx.x + it * gridDim.x;
    uint8_t* srow = sgen + (size_t)s * slot_bytes;
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
      *reinterpret_cast<Vec16<XT>*>(srow + 16 * c) = o;     // each lane rewrites the chunks it read
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      bulk_store_1d(y + row * ys, sbase + s * slot_bytes, row_bytes);
      bulk_commit_group();
      if (rstd) rstd[row] = rr;
      bulk_wait_read_all();          // the slot may be refilled once the store has read it
      mbar_arrive(empty(s));
    }
    __syncwarp();
  }
  if (lane == 0) bulk_wait_all();     // no store of this thread may outlive the CTA
}

// ---- backward, at most 4096 columns: a row (x and dy) per PAIR of consumer warps, each warp
// half of the row's 16-byte chunks.  Pass 1 sums dy w x over the row (the two halves meet in
// shared memory, added in a fixed order), pass 2 writes dx over x in the slot (one bulk store
// per row) and adds dy x r into per-column dw sums that stay in the lane's registers for the
// whole kernel (CH chunks per lane).  At the end the pairs' dw rows are added in pair order
// through the (by then idle) ring and leave as one partial row per CTA.
constexpr int kBwdPairs = 7;
constexpr int kBwdStreamConsumers = 2 * kBwdPairs;
constexpr int kBwdStreamThreads = 32 * (kBwdStreamConsumers + 1);

template <typename XT, typename WT, int CH>
__global__ void __launch_bounds__(kBwdStreamThreads, 1)
rmsnorm_bwd_stream_kernel(const XT* __restrict__ dy, const XT* __restrict__ x, const WT* __restrict__ w,
                          const float* __restrict__ rstd, XT* __restrict__ dx, float* __restrict__ partial,
                          long long rows, int D, long long dys, long long xs, long long dxs, int slot_bytes,
                          int n_slots) {
  using namespace sm100;
  constexpr int N = Vec16<XT>::N;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  float* sw = reinterpret_cast<float*>(sgen + StreamSmem::kWeights);
  const int bar_off = StreamSmem::bars(D);
  const uint32_t bars = sbase + bar_off;
  auto full = [&](int s) { return bars + 8 * s; };
  auto empty = [&](int s) { return bars + 8 * (kMaxSlots + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + bar_off + 2 * kMaxSlots * 8);
  __shared__ float pair_sum[kBwdPairs][2][2];     // [pair][row parity][half]
  __shared__ int pair_ok[kBwdPairs][2][2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)D * sizeof(XT);
  const long long my_rows = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < n_slots; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 2); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  auto slot_of = [&](long long it) { return (int)(it % n_slots); };
  auto use_of = [&](long long it) { return (uint32_t)((it / n_slots) & 1); };      // phase parity of row `it` in its slot

  if (warp == kBwdStreamConsumers) {
    // ================================================================ producer
    if (lane == 0) {
      long long issued = 0;
#if B200ATTN_RMS_LOAD_HINT
      const uint64_t pol = l2_policy_evict_first();
#endif
      for (long long it = 0; it < my_rows; ++it, ++issued) {
        const int s = slot_of(it);
        if (!mbar_wait(empty(s), use_of(it) ^ 1u, abort_flag)) break;
        const long long row = blockIdx.x + it * gridDim.x;
        mbar_expect_tx(full(s), 2 * row_bytes);
#if B200ATTN_RMS_LOAD_HINT
        bulk_load_1d_hint(sbase + s * slot_bytes, x + row * xs, row_bytes, full(s), pol);
        bulk_load_1d_hint(sbase + s * slot_bytes + slot_bytes / 2, dy + row * dys, row_bytes, full(s), pol);
#else
        bulk_load_1d(sbase + s * slot_bytes, x + row * xs, row_bytes, full(s));
        bulk_load_1d(sbase + s * slot_bytes + slot_bytes / 2, dy + row * dys, row_bytes, full(s));
#endif
      }
      if (*abort_flag) {
        for (long long i = issued > n_slots ? issued - n_slots : 0; i < issued; ++i) mbar_drain(full(slot_of(i)), use_of(i));
      }
    }
    return;
  }

  // ==================================================================== consumers
  for (int c = threadIdx.x; c < D; c += 32 * kBwdStreamConsumers) sw[c] = to_f(w[c]);
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
  const int pair = warp >> 1, half = warp & 1;
  const float inv_d = 1.f / (float)D;
  const int chunks = D / N;
  // this lane's chunks: (2 k + half) * 32 + lane, k < CH
  float dwv[CH][N];
#pragma unroll
  for (int k = 0; k < CH; ++k)
#pragma unroll
    for (int i = 0; i < N; ++i) dwv[k][i] = 0.f;
  long long n_done = 0;
  for (long long it = pair; it < my_rows; it += kBwdPairs, ++n_done) {
    const int s = slot_of(it);
    // (a wait that gave up is carried to the pair's barrier below, so that both warps of the
    // pair leave the loop together and neither waits for the other for ever)
    // first "the slot's previous row has been released", then "this row has landed" (see above)
    const bool landed = mbar_wait(empty(s), use_of(it) ^ 1u, abort_flag) && mbar_wait(full(s), use_of(it), abort_flag);
    const long long row = blockIdx.x + it * gridDim.x;
    uint8_t* sx = sgen + (size_t)s * slot_bytes;
    const uint8_t* sg = sx + slot_bytes / 2;
    const float r = rstd[row];
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = (2 * k + half) * 32 + lane;
      if (landed && c < chunks) {
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
    // meet the other half of the row (a slot of pair_sum per row parity: the barrier keeps the
    // two warps of a pair within one row of each other)
    const int par = (int)(n_done & 1);
    if (lane == 0) { pair_sum[pair][par][half] = tot; pair_ok[pair][par][half] = landed ? 1 : 0; }
    asm volatile("bar.sync %0, 64;" ::"r"(2 + pair) : "memory");
    if (!(pair_ok[pair][par][0] && pair_ok[pair][par][1])) break;
    tot = pair_sum[pair][par][0] + pair_sum[pair][par][1];
    const float coef = tot * r * r * inv_d;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = (2 * k + half) * 32 + lane;
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
        *reinterpret_cast<Vec16<XT>*>(sx + 16 * c) = o;      // dx over x: each lane rewrites the chunks it read
      }
    }
    fence_proxy_async();
    asm volatile("bar.sync %0, 64;" ::"r"(2 + pair) : "memory");   // both halves of dx are in the slot
    if (lane == 0) {
      if (half == 0) {
        bulk_store_1d(dx + row * dxs, sbase + s * slot_bytes, row_bytes);
        bulk_commit_group();
        bulk_wait_read_all();        // the slot may be refilled once the store has read it
      }
      mbar_arrive(empty(s));
    }
    __syncwarp();
  }
  if (lane == 0) bulk_wait_all();     // no store of this thread may outlive the CTA
  // ---- the pairs' dw rows -> one partial row per CTA, added in pair order.  Every slot has been
  // consumed (or the CTA is aborting and the producer drains): the ring is free.
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
  if (!*abort_flag) {
    float* red = reinterpret_cast<float*>(sgen);     // [kBwdPairs][D] fp32 <= 112 KB of the ring
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = (2 * k + half) * 32 + lane;
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < N; i += 4)
          *reinterpret_cast<float4*>(red + (size_t)pair * D + c * N + i) =
              make_float4(dwv[k][i], dwv[k][i + 1], dwv[k][i + 2], dwv[k][i + 3]);
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kBwdStreamConsumers) : "memory");
    for (int c = threadIdx.x; c < D; c += 32 * kBwdStreamConsumers) {
      float sum = 0.f;
#pragma unroll
      for (int p = 0; p < kBwdPairs; ++p) sum += red[(size_t)p * D + c];
      partial[(long long)blockIdx.x * D + c] = sum;
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
  // rows of 2 .. 12 KB, enough of them to fill the machine: the streaming kernel
  const long long row_bytes = (long long)a->dim * (long long)sizeof(XT);
  // (the ring must have a slot per consumer warp at least: the release-then-landing wait of the
  // consumers is only free of phase aliasing if the producer, which works in row order, cannot be
  // a whole ring behind a consumer's previous row)
  if (vec && row_bytes >= 2048 && kRingBytes / ((row_bytes + 127) & ~127LL) >= kFwdStreamConsumers &&
      a->dim * 4 <= 32768 && a->rows >= 1024) {
    const DeviceInfo* di = nullptr;
    if (int st = device_info(&di)) return st;
    const int slot = (int)((row_bytes + 127) & ~127LL);
    int n_slots = kRingBytes / slot;
    if (n_slots > kMaxSlots) n_slots = kMaxSlots;
    const int grid = (int)(a->rows < di->sm_count ? a->rows : di->sm_count);
    auto kern = rmsnorm_fwd_stream_kernel<XT, WT>;
    const int smem = StreamSmem::bytes(a->dim);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return B200ATTN_ERR_CUDA;
    kern<<<grid, kFwdStreamThreads, smem, stream>>>((const XT*)a->x, (const WT*)a->weight, (XT*)a->y, a->rstd, a->rows,
                                                  a->dim, a->x_stride_row, a->y_stride_row, a->eps, slot, n_slots);
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
  const int ch = (a->dim / N + 63) / 64;                      // 16-byte chunks per lane (two warps share a row)
  // (and a ring slot per pair of consumer warps at least, see the forward)
  if (vec && ((uintptr_t)a->weight & 15) == 0 && row_bytes >= 2048 &&
      kRingBytes / (2 * ((row_bytes + 127) & ~127LL)) >= kBwdPairs && a->dim <= 4096 && ch <= (N == 4 ? 16 : 8) &&
      a->rows >= 1024) {
    const DeviceInfo* di = nullptr;
    if (int st = device_info(&di)) return st;
    const int grid = di->sm_count < g ? di->sm_count : g;     // partial rows: the workspace holds g of them
    const int smem = StreamSmem::bytes(a->dim);
    const int slot = 2 * (int)((row_bytes + 127) & ~127LL);   // x row, dy row
    int n_slots = kRingBytes / slot;
    if (n_slots > kMaxSlots) n_slots = kMaxSlots;
#define B200ATTN_RMS_BWD_STREAM(CH)                                                                               \
  {                                                                                                               \
    auto kern = rmsnorm_bwd_stream_kernel<XT, WT, CH>;                                                            \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)             \
      return B200ATTN_ERR_CUDA;                                                                                   \
    kern<<<grid, kBwdStreamThreads, smem, stream>>>(dy, x, w, a->rstd, dx, partial, a->rows, a->dim, a->dy_stride_row, \
                                                 a->x_stride_row, a->dx_stride_row, slot, n_slots);               \
  }
    if (ch <= 2) B200ATTN_RMS_BWD_STREAM(2)
    else if (ch <= 4) B200ATTN_RMS_BWD_STREAM(4)
    else if (ch <= 8) B200ATTN_RMS_BWD_STREAM(8)
    else if constexpr (N == 4) B200ATTN_RMS_BWD_STREAM(16)     // (fp32 rows: 4 columns per chunk)
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
