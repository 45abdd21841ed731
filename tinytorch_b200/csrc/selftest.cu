// Self-test of the bounded-wait helper every tensor-core kernel of this library relies on.
//
// One CTA waits on an mbarrier that nothing ever arrives on, with a caller-chosen limit.  The
// wait must give up when the limit has passed, the kernel must set kStatusWaitExpired in the
// status word and return normally, and the context must stay usable.  Nothing here faults or
// spins without a bound; it is how the expiry path can be exercised on a GPU at all, since a
// healthy kernel never loses a signal.  The reference has no counterpart (its kernels have no
// device-side waits); what it maps to on the host is the LOGE + ASSERT convention of
// src/Utils/Macros.h:34-43, which a caller applies to the status word.
#include "common.cuh"
#include "ptx.cuh"

namespace ttattn {
namespace {

__global__ void wait_expiry_kernel(int32_t* status, uint64_t limit_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  const uint64_t t0 = ptx::globaltimer_ns();
  // every thread of the CTA waits, as the warps of the real kernels do; the first one whose
  // limit passes raises the flag that cuts the others short
  const bool ok = ptx::mbar_wait(&bar, 0, &abort_flag, limit_ns);
  const uint64_t t1 = ptx::globaltimer_ns();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok || abort_flag) atomicOr(status, kStatusWaitExpired);
    if (waited_ns) *waited_ns = t1 - t0;
    ptx::mbar_inval(&bar);
  }
}

}  // namespace

cudaError_t launch_wait_expiry(int32_t* status, uint64_t limit_ns, unsigned long long* waited_ns, cudaStream_t stream) {
  wait_expiry_kernel<<<1, 128, 0, stream>>>(status, limit_ns, waited_ns);
  return cudaGetLastError();
}

}  // namespace ttattn
