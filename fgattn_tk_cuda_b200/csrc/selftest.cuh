// Self-test of the bounded wait that every kernel of this library uses on its mbarriers.
#pragma once
#include "sm100_ptx.cuh"

namespace fg {

// One warp waits on an mbarrier that nobody ever arrives at, with a budget of `budget_cycles`.  The wait
// gives up when the budget is spent, records code 9001 in the error word and the kernel returns
// normally -- the path a production kernel takes when a copy or a peer never shows up.
__global__ void __launch_bounds__(32) bounded_wait_probe_kernel(int* err, long long budget_cycles) {
  __shared__ __align__(8) uint64_t barrier_word;
  __shared__ AbortState abort_state;
  const uint32_t bar = smem_u32(&barrier_word);
  if (threadIdx.x == 0) {
    abort_state.flag = 0;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const bool ok = mbar_wait_budget(bar, 0, &abort_state, err, 9001, budget_cycles);
  // every lane must have given up (the first one to run out of budget raises the shared abort flag)
  if (ok && err) atomicCAS(err, 0, 9002);
}

}  // namespace fg
