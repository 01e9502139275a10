// A kernel whose only job is to let one bounded wait run out, so that the path a
// stuck pipeline would take (abort flag, status word, unwinding, normal return,
// TSM100_ERR_TIMEOUT on the host) can be exercised without anything being stuck.
// Nothing here faults, traps or spins without a limit.
#pragma once

#include "ptx.cuh"

namespace tsm100 {
namespace selftest {

constexpr uint32_t kSite = 63;  // the site id this kernel reports: 0x1000 | 63

// One CTA of 64 threads.  The mbarrier expects one arrival that nobody makes.  Thread 0
// waits on it with the caller's limit: the wait gives up, raises the CTA's abort flag and
// records kStatusWaitTimeout | kSite.  Thread 32 (another warp, as the consumer role of a
// real kernel would be) waits with the library's normal 2 s limit and must leave through
// the abort flag long before that.  observed[0] counts waits that returned false,
// observed[1] is the time thread 0 spent waiting, in microseconds.
__global__ void __launch_bounds__(64) wait_timeout_kernel(uint32_t* status, unsigned long long limit_ns, uint32_t* observed) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  volatile uint32_t* abort = &abort_flag;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    const bool ok = ptx::mbar_wait_for(&bar, 0, abort, status, kSite, limit_ns);
    const unsigned long long dt = ptx::globaltimer_ns() - t0;
    if (!ok) atomicAdd(&observed[0], 1u);
    observed[1] = static_cast<uint32_t>(dt / 1000ull);
  } else if (threadIdx.x == 32) {
    const bool ok = ptx::mbar_wait(&bar, 0, abort, status, kSite + 1);
    if (!ok) atomicAdd(&observed[0], 1u);
  }
  __syncthreads();  // every thread arrives: the kernel ends normally
}

}  // namespace selftest
}  // namespace tsm100
