// Diagnostic entry point: exercises the bounded device-side wait that every tensor-core kernel
// of the library uses (mbar_wait), on a barrier that nothing ever signals, so that the give-up
// path — status word, clean exit, context still usable — can be tested without any fault.
#include "common.cuh"
#include "tcgen05.cuh"

namespace kcg {
int* device_status_word();  // runtime.cu
namespace {

__global__ void bounded_wait_kernel(uint64_t budget_ns, int* status, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    abort_flag = 0;
    sm100::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = sm100::global_ns();
    const bool ok = sm100::mbar_wait(&bar, 0, &abort_flag, budget_ns);   // nobody arrives: must give up
    *waited_ns = sm100::global_ns() - t0;
    if (!ok) {
      abort_flag = 1;
      *status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  }
  __syncthreads();
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_selftest_bounded_wait(uint64_t budget_ns, unsigned long long* waited_ns_device, void* stream) {
  using namespace kcg;
  clear_error();
  if (budget_ns == 0 || budget_ns > 100000000ull)
    return fail(KCG_ERR_INVALID_ARG, "selftest: the wait budget must be between 1 ns and 100 ms");
  if (!waited_ns_device) return fail(KCG_ERR_INVALID_ARG, "selftest: null pointer");
  int* status = device_status_word();
  if (!status) return fail(KCG_ERR_CUDA, "selftest: could not allocate the host-mapped status word");
  bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(budget_ns, status, waited_ns_device);
  return check_launch("bounded_wait_kernel");
}
