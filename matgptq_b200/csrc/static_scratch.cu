// Packed matmul for callers that must not allocate device memory.
//
// The tensor-core path splits K over several CTAs for shapes with few 128-row tiles (gemm_tc.cu).
// Their fp32 sums normally meet inside a thread-block cluster; they go through scratch memory and a
// second kernel when the caller asks for that form (MATGPTQ_B200_FLAG_SCRATCH_REDUCE) or when the
// device cannot place the cluster.  matgptq_b200_matmul_ws takes that scratch from the caller.  Some
// callers have none to give and cannot get any: a serving process whose memory pool was sized up
// front and already owns the whole device, a plugin called from inside such a host without access
// to its allocator, or a latency-critical loop in which cudaMalloc (which synchronises the device)
// is forbidden.  For them the scratch lives in the library image itself: a fixed array in device
// global memory.  The CUDA runtime loads device code lazily and this file has no kernel of its
// own, so the array comes into a GPU's memory when its address is first asked for on that GPU (the
// first call below for a shape that splits K), and stays until the process exits.  That first call
// is the only one that can change the amount of free device memory; it has to come before the
// host hands the rest of the device to its pool.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/matgptq_b200.h"
#include "kernels.h"

namespace {

// 8 MiB of split-K partial sums.  In host code this name is only a handle for the runtime
// (it is not a device address); the address the kernels use comes from cudaGetSymbolAddress.
constexpr long long kStaticScratchBytes = MATGPTQ_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;  // devices beyond this index are refused (bad argument)
std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices] = {};
bool g_scratch_ready[kMaxDevices] = {};

// Device address of the array on the current device, resolved once per device.
int static_scratch_address(void **out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return MG_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ready[dev]) {
    void *ptr = nullptr;
    // loads this module on the device if it is not there yet: the driver takes the array's bytes now
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();  // the failure is reported through the status code, not left pending
      return MATGPTQ_B200_ERR_SCRATCH_UNAVAILABLE;
    }
    g_scratch_address[dev] = ptr;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_address[dev];
  return MG_OK;
}

}  // namespace

extern "C" int matgptq_b200_matmul_static_scratch(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in,
                                                   int64_t batch, const void *w, const void *s, const void *x, void *y,
                                                   void *stream, uint32_t flags) {
  int64_t need = matgptq_b200_matmul_workspace_bytes(n_out, n_in, batch);
  if (need > kStaticScratchBytes) {
    // the sums cannot go through the array; without the flag they do not have to (they meet inside the cluster)
    if (flags & MATGPTQ_B200_FLAG_SCRATCH_REDUCE) return MATGPTQ_B200_ERR_SCRATCH_TOO_SMALL;
    need = 0;
  }
  void *scratch = nullptr;
  if (need > 0) {
    const int st = static_scratch_address(&scratch);
    if (st != MG_OK) return st;
  }
  // Nothing has to be cleared: every partial sum the reduction reads is written by this call first.
  return matgptq_b200_matmul_ws(bitwidth, group_size, n_out, n_in, batch, w, s, x, y, stream, flags, scratch, need, 0, 0);
}
