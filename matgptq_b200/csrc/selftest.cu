// Self-test of the bounded waits: a wait that nothing will ever satisfy has to give up, record its status
// code and let the kernel finish, so that the context stays usable.  The kernels of this library wait on
// mbarriers that asynchronous copies complete (async.cuh); here one warp arms such a barrier for bytes that
// no copy delivers and waits on it with a short poll limit.  Nothing is faulted, trapped or left spinning.
// The reference has no counterpart (its only error path is exit(1), csrc/include/common.cuh:44-51).
#include <cuda_runtime.h>

#include "../../include/matgptq_b200.h"
#include "async.cuh"
#include "kernels.h"

namespace mg {

__global__ void __launch_bounds__(32, 1) wait_timeout_probe_kernel(int code, unsigned polls, int *gave_up) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_arrive_expect_tx(bar, 64);  // 64 bytes are expected; no copy is issued
  __syncwarp();
  const bool ok = mbar_wait_bounded(bar, 0, polls);
  if (!ok) {
    report_status(code);
    if (threadIdx.x == 0 && gave_up) *gave_up = 1;
  }
}

int selftest_wait_timeout_launch(int code, unsigned polls, int *gave_up, cudaStream_t stream) {
  wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(code, polls, gave_up);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

MG_DEFINE_STATUS_ACCESSOR(selftest_device_status)

}  // namespace mg

extern "C" int matgptq_b200_selftest_wait_timeout(int status_code, int *gave_up_flag, void *stream) {
  if (status_code != mg::kStatusWeightCopyTimeout && status_code != mg::kStatusActivationCopyTimeout &&
      status_code != mg::kStatusMmaTimeout)
    return MG_ERR_BAD_ARG;
  // 4096 polls of about 40 ns each and the hardware's own try_wait time-out: well under a second
  return mg::selftest_wait_timeout_launch(status_code, 4096u, gave_up_flag, static_cast<cudaStream_t>(stream));
}
