// Self-test of the bounded wait every mbarrier wait of the attention kernel goes through.
//
// A wait on a barrier that nothing ever arrives on must give up when its limit has passed, set the CTA's
// abort flag and let the kernel return with SA_DEV_WAIT_EXPIRED in the caller's status word.  The probe
// kernel does exactly that with a caller-chosen (short) limit: one CTA, one barrier with an arrival count
// of 1 and no arriver; thread 0 waits through ptx::mbar_wait_slow, the other threads wait for thread 0 at
// a __syncthreads.  Nothing spins without a limit.
#include "ptx_sm100.cuh"
#include "sa_common.cuh"

namespace sa {
namespace {

__global__ void __launch_bounds__(64)
bounded_wait_probe_kernel(const unsigned long long limit_ns, int32_t* dev_status, unsigned long long* waited_ns) {
  __shared__ __align__(8) unsigned long long barrier;
  __shared__ int abort_flag;
  const uint32_t bar = ptx::smem_u32(&barrier);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(bar, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = ptx::global_timer_ns();
    const bool ok = ptx::mbar_wait_slow(bar, 0, &abort_flag, limit_ns);      // phase 0 never completes
    if (waited_ns != nullptr) *waited_ns = ptx::global_timer_ns() - t0;
    if (ok) abort_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag != 0 && dev_status != nullptr) atomicMax(dev_status, SA_DEV_WAIT_EXPIRED);
}

}  // namespace

cudaError_t launch_bounded_wait_probe(unsigned long long limit_ns, int32_t* dev_status, unsigned long long* waited_ns,
                                      cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 64, 0, stream>>>(limit_ns, dev_status, waited_ns);
  return cudaGetLastError();
}

}  // namespace sa
