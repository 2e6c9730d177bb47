// Self-test of the bounded device-side wait every kernel of the library uses: a wait on
// an mbarrier that nothing ever completes must give up after its cycle budget, raise the
// CTA's abort flag and let the kernel return normally with the status word set.
#include "common.cuh"
#include "sm100.cuh"

namespace b200attn {
namespace {

__global__ void bounded_wait_probe_kernel(int32_t* status_word, long long budget_cycles, long long* waited_cycles) {
  using namespace sm100;
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);      // one arrival expected; nobody arrives
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = mbar_wait_for(smem_u32(&bar), 0, &abort_flag, budget_cycles);
    if (waited_cycles) *waited_cycles = clock64() - t0;
    if (!ok && status_word) atomicExch(status_word, 1);
  }
  __syncthreads();
  // every other wait of the CTA now returns at once
  if (threadIdx.x == 1 && !mbar_wait_for(smem_u32(&bar), 0, &abort_flag, budget_cycles) && status_word)
    atomicAdd(status_word, 2);
}

}  // namespace

int selftest_bounded_wait(int32_t* status_word, long long budget_cycles, long long* waited_cycles, cudaStream_t stream) {
  if (!status_word) return B200ATTN_ERR_NULL;
  // the probe is meant to give up quickly: refuse budgets beyond ~50 ms
  if (budget_cycles <= 0 || budget_cycles > 100000000LL) return B200ATTN_ERR_SHAPE;
  if (int dst = device_info(nullptr)) return dst;
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status_word, budget_cycles, waited_cycles);
  set_launch_count(1);
  return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ERR_CUDA;
}

}  // namespace b200attn
