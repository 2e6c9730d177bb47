// Shared device / host helpers of the b200attn kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/b200attn.h"

namespace b200attn {

void set_launch_count(int n);

// Facts about the current device, looked up once per device (std::call_once) and read-only
// afterwards: launchers are re-entrant and keep no other global state.
struct DeviceInfo {
  int status;    // B200ATTN_OK, or B200ATTN_ERR_DEVICE when the device is not compute capability 10.x
  int sm_count;
};
// B200ATTN_OK and *info, B200ATTN_ERR_DEVICE (wrong architecture: the kernels are sm_100a only, the
// counterpart of the reference's arch probe, utils/utils.py:19-24) or B200ATTN_ERR_CUDA (no device).
int device_info(const DeviceInfo** info);

// implemented in decode.cu / prefill.cu, called by api.cu
size_t decode_workspace_bytes(const b200attn_decode_args* a);
int decode_fwd(const b200attn_decode_args* a, bool sparse, void* scratch, size_t scratch_bytes,
               cudaStream_t stream);
// row_begin / row_end: the query rows of every sequence to compute (0, INT_MAX = all)
int prefill_fwd(const b200attn_prefill_args* a, bool sparse, cudaStream_t stream, int row_begin = 0, int row_end = 0x7fffffff);
int decode_fwd_noalloc(const b200attn_decode_args* a, cudaStream_t stream);
size_t prefill_bwd_workspace_bytes(const b200attn_prefill_bwd_args* a);
int prefill_bwd(const b200attn_prefill_bwd_args* a, cudaStream_t stream);
int kv_pack_to_cache(const b200attn_kv_pack_args* a, cudaStream_t stream);
int kv_append(const b200attn_kv_append_args* a, cudaStream_t stream);
size_t paged_decode_workspace_bytes(const b200attn_paged_decode_args* a);
int paged_decode_fwd(const b200attn_paged_decode_args* a, cudaStream_t stream);
int32_t window_blocks_prefill_max_nnz(int32_t block_size, int32_t window_local, int32_t window_global,
                                      int32_t n_qblocks);
int window_blocks_prefill(const b200attn_window_blocks_prefill_args* a, cudaStream_t stream);
int window_blocks_decode(const b200attn_window_blocks_decode_args* a, cudaStream_t stream);
int topk_blocks(const b200attn_topk_blocks_args* a, cudaStream_t stream);
int selftest_bounded_wait(int32_t* status_word, long long budget_cycles, long long* waited_cycles, cudaStream_t stream);
int rmsnorm_fwd(const b200attn_rmsnorm_fwd_args* a, cudaStream_t stream);
size_t rmsnorm_bwd_workspace_bytes(const b200attn_rmsnorm_bwd_args* a);
int rmsnorm_bwd(const b200attn_rmsnorm_bwd_args* a, cudaStream_t stream);

// 16-byte read-only load that does not pollute L1 (data is used once).
template <typename T>
__device__ __forceinline__ uint4 ld_nc_16(const T* ptr) {
  uint4 r;
#ifndef B200ATTN_LD_HINT
#define B200ATTN_LD_HINT ".L2::256B"
#endif
  asm volatile("ld.global.nc.L1::no_allocate" B200ATTN_LD_HINT ".v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(ptr));
  return r;
}

// D(16x8,f32) += A(16x16) * B(16x8), A row-major fragments a0..a3, B column fragments b0,b1.
template <typename T>
__device__ __forceinline__ void mma_16816(float* c, unsigned a0, unsigned a1, unsigned a2,
                                          unsigned a3, unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float* c, unsigned a0, unsigned a1, unsigned a2,
                                                  unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float* c, unsigned a0, unsigned a1,
                                                         unsigned a2, unsigned a3, unsigned b0,
                                                         unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two floats -> one packed 16-bit pair, `lo` in the low half
template <typename T>
__device__ __forceinline__ unsigned pack2(float lo, float hi);
template <>
__device__ __forceinline__ unsigned pack2<__half>(float lo, float hi) {
  unsigned r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <>
__device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float lo, float hi) {
  unsigned r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

}  // namespace b200attn
