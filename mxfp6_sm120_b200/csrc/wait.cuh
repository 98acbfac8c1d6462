// Bounded mbarrier waits shared by the GEMM kernels.  No wait in the library spins
// forever: after about two seconds the waiting thread raises the CTA's abort flag,
// records a code in the device status word and returns false; the kernel then lets
// its copies drain, frees tensor memory and exits.
#pragma once

#include "ptx.cuh"

namespace mx {

constexpr long long kWaitCycles = 4000000000ll;  // about two seconds of clock64

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort,
                                             int* status, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 63u) {
      if (*abort != 0) return false;
      if (clock64() - start > kWaitCycles) {
        *abort = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// The same with cluster-scope acquire: the barrier is completed by arrivals of peer CTAs
// whose shared-memory writes must be visible afterwards.
__device__ __forceinline__ bool bounded_wait_cluster(uint32_t bar, uint32_t parity,
                                                     volatile int* abort, int* status, int code) {
  if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 63u) == 63u) {
      if (*abort != 0) return false;
      if (clock64() - start > kWaitCycles) {
        *abort = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

}  // namespace mx
