// extern "C" surface of libb200attn.so; declarations and the reference
// interfaces they replace are in include/b200attn.h.
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace b200attn {
static thread_local int g_launch_count = 0;
void set_launch_count(int n) { g_launch_count = n; }

int device_info(const DeviceInfo** info) {
  constexpr int kMaxDevices = 64;
  static std::once_flag once[kMaxDevices];
  static DeviceInfo infos[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200ATTN_ERR_CUDA;
  std::call_once(once[dev], [dev] {
    int major = 0, sms = 0;
    DeviceInfo& d = infos[dev];
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      d.status = B200ATTN_ERR_CUDA;
      return;
    }
    // B200ATTN_ASSUME_CC_MAJOR=<n> stands in for the probed value: the only way to see the
    // refusal path on a machine whose GPUs are all sm_100
    if (const char* e = getenv("B200ATTN_ASSUME_CC_MAJOR")) major = atoi(e);
    d.sm_count = sms;
    d.status = major == 10 ? B200ATTN_OK : B200ATTN_ERR_DEVICE;
  });
  if (infos[dev].status != B200ATTN_OK) return infos[dev].status;
  if (info) *info = &infos[dev];
  return B200ATTN_OK;
}
}  // namespace b200attn

using namespace b200attn;

extern "C" {

int b200attn_abi_version(void) { return B200ATTN_ABI_VERSION; }

int b200attn_last_launch_count(void) { return g_launch_count; }

const char* b200attn_strerror(int status) {
  switch (status) {
    case B200ATTN_OK: return "ok";
    case B200ATTN_ERR_NULL: return "a required pointer is NULL (or both / neither of cu_seqlens and seqlens given)";
    case B200ATTN_ERR_DTYPE: return "dtype must be fp16 or bf16";
    case B200ATTN_ERR_HEAD_DIM: return "head_dim must be 32, 64, 96 or 128";
    case B200ATTN_ERR_GQA: return "heads_q must be a positive multiple of heads_kv";
    case B200ATTN_ERR_ALIGN: return "base pointer is not 16-byte aligned";
    case B200ATTN_ERR_STRIDE: return "stride is not a multiple of 8 elements";
    case B200ATTN_ERR_SHAPE: return "invalid or inconsistent sizes";
    case B200ATTN_ERR_WORKSPACE: return "workspace missing or too small";
    case B200ATTN_ERR_MODE: return "bad sparsity mode, window or block-list parameters";
    case B200ATTN_ERR_CUDA: return "a CUDA call failed";
    case B200ATTN_ERR_TOO_LARGE: return "problem exceeds a built-in limit";
    case B200ATTN_ERR_DEVICE: return "device is not compute capability 10.x";
    default: return "unknown b200attn status";
  }
}

size_t b200attn_decode_workspace_bytes(const b200attn_decode_args* args) {
  return decode_workspace_bytes(args);
}

int b200attn_decode_fwd(const b200attn_decode_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return decode_fwd(args, false, nullptr, 0, (cudaStream_t)stream);
}

int b200attn_sparse_decode_fwd(const b200attn_decode_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return decode_fwd(args, true, nullptr, 0, (cudaStream_t)stream);
}

int b200attn_decode_fwd_noalloc(const b200attn_decode_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return decode_fwd_noalloc(args, (cudaStream_t)stream);
}

size_t b200attn_prefill_bwd_workspace_bytes(const b200attn_prefill_bwd_args* args) {
  return prefill_bwd_workspace_bytes(args);
}

int b200attn_prefill_bwd(const b200attn_prefill_bwd_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return prefill_bwd(args, (cudaStream_t)stream);
}

int b200attn_kv_pack_to_cache(const b200attn_kv_pack_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return kv_pack_to_cache(args, (cudaStream_t)stream);
}

int b200attn_kv_append(const b200attn_kv_append_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return kv_append(args, (cudaStream_t)stream);
}

size_t b200attn_paged_decode_workspace_bytes(const b200attn_paged_decode_args* args) {
  return paged_decode_workspace_bytes(args);
}

int b200attn_paged_decode_fwd(const b200attn_paged_decode_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return paged_decode_fwd(args, (cudaStream_t)stream);
}

int32_t b200attn_window_blocks_prefill_max_nnz(int32_t block_size, int32_t window_local, int32_t window_global,
                                               int32_t n_qblocks) {
  return window_blocks_prefill_max_nnz(block_size, window_local, window_global, n_qblocks);
}

int b200attn_window_blocks_prefill(const b200attn_window_blocks_prefill_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return window_blocks_prefill(args, (cudaStream_t)stream);
}

int b200attn_window_blocks_decode(const b200attn_window_blocks_decode_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return window_blocks_decode(args, (cudaStream_t)stream);
}

int b200attn_topk_blocks(const b200attn_topk_blocks_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return topk_blocks(args, (cudaStream_t)stream);
}

int b200attn_rmsnorm_fwd(const b200attn_rmsnorm_fwd_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return rmsnorm_fwd(args, (cudaStream_t)stream);
}

size_t b200attn_rmsnorm_bwd_workspace_bytes(const b200attn_rmsnorm_bwd_args* args) {
  return rmsnorm_bwd_workspace_bytes(args);
}

int b200attn_rmsnorm_bwd(const b200attn_rmsnorm_bwd_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return rmsnorm_bwd(args, (cudaStream_t)stream);
}

int b200attn_selftest_bounded_wait(int32_t* status_word, int64_t budget_cycles, int64_t* waited_cycles,
                                   b200attn_stream_t stream) {
  set_launch_count(0);
  return selftest_bounded_wait(status_word, (long long)budget_cycles, (long long*)waited_cycles, (cudaStream_t)stream);
}

size_t b200attn_prefill_workspace_bytes(const b200attn_prefill_args*) { return 0; }

int b200attn_prefill_fwd(const b200attn_prefill_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return prefill_fwd(args, false, (cudaStream_t)stream);
}

int b200attn_prefill_fwd_rows(const b200attn_prefill_args* args, int32_t row_begin, int32_t row_end,
                              b200attn_stream_t stream) {
  set_launch_count(0);
  if (row_begin == 0 && row_end == 0x7fffffff) row_end -= 1;   // (that pair means "all rows" internally)
  return prefill_fwd(args, false, (cudaStream_t)stream, row_begin, row_end);
}

int b200attn_sparse_prefill_fwd(const b200attn_prefill_args* args, b200attn_stream_t stream) {
  set_launch_count(0);
  return prefill_fwd(args, true, (cudaStream_t)stream);
}

}  // extern "C"
