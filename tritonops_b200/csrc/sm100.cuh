// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the prefill
// kernel uses: mbarrier, TMA tiled loads, tensor memory (TMEM) and tcgen05 MMA.
// Every spin on an mbarrier is bounded: after a cycle budget it records the
// failure and reports it, so a protocol bug can never hang the GPU.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace b200attn {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a converged warp (the lowest) gets true.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Cycle budget of one wait (~2 s at 2 GHz).  Legitimate waits last micro- to
// milliseconds.
constexpr long long kWaitBudgetCycles = 4000000000LL;

// Bounded wait.  `abort_flag` lives in shared memory: once any role gave up,
// every later wait in the CTA returns at once so all roles drain and exit.
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                              long long budget_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  int polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait_for(bar, parity, abort_flag, kWaitBudgetCycles);
}

// Wait, with a budget of its own, for a copy this CTA issued itself: used on the way out after
// a wait has given up (the abort flag is up, so mbar_wait would return at once), because a CTA
// must not exit while bulk copies into its shared memory are still in flight.
constexpr long long kDrainBudgetCycles = 400000000LL;   // ~0.2 s
__device__ __forceinline__ bool mbar_drain(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int polls = 0;
  while (!mbar_try_wait(bar, parity))
    if ((++polls & 255) == 0 && clock64() - t0 > kDrainBudgetCycles) return false;
  return true;
}

// Clear rows [row0, row1) of a 16-bit operand tile laid out as `panels` 64-column panels of
// 128-byte rows (`panel_bytes` apart), by the 32 lanes of one warp.  The 128-byte swizzle only
// permutes 16-byte chunks inside a row, so whole rows can be cleared without knowing it.  Ends
// with the fence that orders these generic-proxy stores before the tensor core's reads.
__device__ __forceinline__ void zero_tile_rows(uint8_t* tile, int panels, int panel_bytes, int row0, int row1,
                                               int lane) {
  const int per_row = panels * 8;
  for (int i = lane; i < (row1 - row0) * per_row; i += 32) {
    const int r = row0 + i / per_row, c = i % per_row;
    *reinterpret_cast<uint4*>(tile + (c >> 3) * panel_bytes + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
}

// ----------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tiled load global -> shared, completion counted in bytes on `bar`.
// c0 (innermost, elements) must be a multiple of 8 for 16-bit types.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared of `bytes` (a multiple of 16; both addresses 16-byte
// aligned), completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

// The same with an L2 eviction-priority hint (a policy made by l2_policy_evict_first()): for data
// that is read once, so that it does not push lines that will be reused, or dirty lines that
// are still collecting writes, out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_load_1d_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

// Untiled bulk copy shared -> global (both addresses 16-byte aligned, `bytes` a multiple of 16),
// tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes)
               : "memory");
}

// Ask for a tile to be brought into L2 (no destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* m, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// Tile of shared memory added (fp32) into a 3-D tensor in global memory by the copy
// engine; completion is tracked by the issuing thread's bulk group.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Tile of shared memory written to a 4-D tensor in global memory by the copy engine (the part of
// the box outside the tensor is not written); completion is tracked by the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every committed group of this thread has finished READING its shared-memory source
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the newest committed group of this thread have finished reading their source
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// every committed group of this thread is complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane -> registers.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// registers -> 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ----------------------------------------------------------------------- MMA
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), version 1.
// Addresses and offsets are encoded in 16-byte units.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// 16 consecutive 32-bit columns of this thread's TMEM lane <- registers.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}

// Instruction descriptor for kind::f16: fp32 accumulate, A and B both `fmt`
// (0 = f16, 1 = bf16), A K-major, B K-major or MN-major, M x N tile.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t fmt, bool b_mn_major, uint32_t M,
                                                 uint32_t N, bool a_mn_major = false) {
  return (1u << 4)                          // D format: f32
         | (fmt << 7) | (fmt << 10)         // A, B formats
         | ((a_mn_major ? 1u : 0u) << 15)   // A major
         | ((b_mn_major ? 1u : 0u) << 16)   // B major
         | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// The MMA wrappers below are executed by every lane of a converged warp and
// take an `issue` flag that is true in exactly one (always the same) lane: the
// instruction itself is predicated, so the surrounding code has no divergent
// branch and its addresses and descriptors can stay in uniform registers.

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
// 8 back-to-back SS products (one 128-wide contraction in steps of 16): D = A B, the
// first step overwrites D.  Descriptors are given as (low, high) words; a step only adds to
// the address field in the low word.
__device__ __forceinline__ void mma_ss_x8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred pi, pt, pf;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
      "setp.ne.b32 pi, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tsetp.ne.b32 pf, 0, 0;\n\t"
      "add.u32 la, %1, 0;\n\tadd.u32 lb, %3, 0;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pf;\n\t"
      "add.u32 la, %1, 2;\n\tadd.u32 lb, %3, 2;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 4;\n\tadd.u32 lb, %3, 4;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 6;\n\tadd.u32 lb, %3, 6;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 1024;\n\tadd.u32 lb, %3, 1024;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 1026;\n\tadd.u32 lb, %3, 1026;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 1028;\n\tadd.u32 lb, %3, 1028;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 1030;\n\tadd.u32 lb, %3, 1030;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(issue)
      : "memory");
}
// 4 back-to-back SS products (one 128-wide contraction in steps of 16): D = A B, the
// first step overwrites D.  Descriptors are given as (low, high) words; a step only adds to
// the address field in the low word.
__device__ __forceinline__ void mma_ss_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred pi, pt, pf;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
      "setp.ne.b32 pi, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tsetp.ne.b32 pf, 0, 0;\n\t"
      "add.u32 la, %1, 0;\n\tadd.u32 lb, %3, 0;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pf;\n\t"
      "add.u32 la, %1, 2;\n\tadd.u32 lb, %3, 2;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 4;\n\tadd.u32 lb, %3, 4;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "add.u32 la, %1, 6;\n\tadd.u32 lb, %3, 6;\n\tmov.b64 da, {la, %2};\n\tmov.b64 db, {lb, %4};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(issue)
      : "memory");
}
// 8 back-to-back TS products over 128 keys: D (+)= A[tmem] B[smem]; A advances by 8 TMEM
// columns per step, B by 2048 bytes; the first step accumulates only if `accumulate`.
__device__ __forceinline__ void mma_ts_x8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred pi, pt, pa;\n\t.reg .b64 db;\n\t.reg .b32 ta, lb;\n\t"
      "setp.ne.b32 pi, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\tsetp.ne.b32 pa, %5, 0;\n\t"
      "add.u32 ta, %1, 0;\n\tadd.u32 lb, %2, 0;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pa;\n\t"
      "add.u32 ta, %1, 8;\n\tadd.u32 lb, %2, 128;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 16;\n\tadd.u32 lb, %2, 256;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 24;\n\tadd.u32 lb, %2, 384;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 32;\n\tadd.u32 lb, %2, 512;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 40;\n\tadd.u32 lb, %2, 640;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 48;\n\tadd.u32 lb, %2, 768;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 56;\n\tadd.u32 lb, %2, 896;\n\tmov.b64 db, {lb, %3};\n\t"
      "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
// Arrive once on `bar` when every tcgen05 operation the issuing lane started so far is done.
__device__ __forceinline__ void mma_commit(uint32_t bar, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(issue)
      : "memory");
}

}  // namespace sm100
}  // namespace b200attn
