// Self-test of the bounded device-side wait: a kernel that waits on an mbarrier nobody arrives on.
//
// Every kernel of this library that waits on the device does so through ascdev::mbar_wait, which gives up after a
// time limit, records an error code in the device's status word and lets the kernel return normally; the host
// then reports status 5 (ASC_ERR_DEVICE_TIMEOUT) from asc_cuda_check_device_status.  In a healthy run that path
// never executes.  This entry point runs it on purpose, with a limit of half a millisecond instead of the
// kernels' 400 ms: the wait runs out, the kernel exits like any other (no trap, no fault, nothing left
// running), and the caller can check that the status arrives and that the next launch works.
#include "../../include/asc_cuda.h"
#include "../../include/asc_cuda_tuning.h"
#include "host_common.h"

namespace {

using namespace ascdev;

constexpr uint64_t kSelfTestLimitNs = 500ull * 1000ull;

__global__ void __launch_bounds__(32) wait_runs_out_kernel(uint32_t* status, uint32_t* gave_up) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncwarp();
  // phase 0 of a barrier that expects one arrival and never gets one
  const bool ok = mbar_wait<0, kSelfTestLimitNs>(smem_u32(&bar), 0, &abort_flag, status, ASC_DEV_TIMEOUT_OTHER);
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = ok ? 0u : 1u;
}

}  // namespace

extern "C" int32_t asc_cuda_selftest_wait_runs_out(uint32_t* gave_up, void* stream) {
  uint32_t* status = nullptr;
  int32_t rc = aschost::device_status_word(&status);
  if (rc != ASC_OK) return rc;
  wait_runs_out_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, gave_up);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}
