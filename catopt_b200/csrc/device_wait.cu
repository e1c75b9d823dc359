// cb2_wait_for_flag: the bounded hand-off wait of the segmented kernels as a launch of its own.
// One thread polls a device flag with `wait_flag_abortable` (acquire loads, a budget counted in SM cycles and polls);
// when the flag is non-zero the kernel simply ends, when the budget runs out it stores
// CB2_WAIT_TIMEOUT into the caller's status word and ends as well.  Nothing is in flight when
// it gives up (no copies, no tensor memory), so the context stays usable and the next launch
// on the stream runs normally.  Callers use it to order a stream behind a flag that a kernel
// on another stream sets; the tests use it to drive the timeout route
// (status word -> host check -> error) without faulting or hanging anything.
#include "common.cuh"

namespace cb2 {
namespace {

__global__ void wait_flag_kernel(const int* __restrict__ flag, unsigned long long budget_ns, int* dev_status) {
  __shared__ int s_abort;
  s_abort = 0;
  if (!wait_flag_abortable(flag, &s_abort, budget_ns) && dev_status) *dev_status = CB2_WAIT_TIMEOUT;
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_wait_for_flag(const int* flag, unsigned budget_us, int* dev_status, void* stream) {
  if (!flag) return CB2_NULL_PTR;
  if (budget_us == 0 || budget_us > 2000000u) return CB2_BAD_SHAPE;      // at most two seconds
  cb2::wait_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, 1000ull * budget_us, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}
