// A kernel whose bounded wait runs out on purpose, for testing the give-up path of the
// mbarrier waits every tcgen05 kernel of this library uses: one warp initialises a barrier that
// nobody ever arrives at, calls the same mbar_wait as the attention kernels with a short
// limit, and ORs the reason into the per-device status word when the wait returns false.
// No copy, no MMA and no tensor memory is in flight when it leaves; nothing traps or faults.
#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

__global__ void __launch_bounds__(32) stalled_wait_kernel(long long limit_cycles, int* status) {
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ WaitCtl wait_ctl;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    wait_ctl.abort = 0;
    wait_ctl.limit = limit_cycles;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(bar, 0, &wait_ctl);  // phase 0 never completes
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && threadIdx.x == 0) atomicOr(status, wait_ctl.abort);
}

}  // namespace

int launch_stalled_wait(long long limit_cycles, int* status, cudaStream_t st) {
  stalled_wait_kernel<<<1, 32, 0, st>>>(limit_cycles, status);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr
