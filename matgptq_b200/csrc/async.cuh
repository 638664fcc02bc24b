// mbarrier + bulk asynchronous copy (TMA, untiled) helpers with bounded waits.
//
// Every wait in this library gives up after a fixed number of polls, records a
// status word that the host can read (matgptq_b200_device_status) and lets the
// kernel run to its end, so a copy that never completes cannot hang the GPU.
#pragma once
#include <cstdint>

namespace mg {

// First failure seen by a kernel of the including translation unit since the last
// reset; 0 = none.  One copy per .cu file (the library is built without relocatable
// device code); each file exports a host accessor built with MG_DEFINE_STATUS_ACCESSOR.
static __device__ int g_device_status;

#define MG_DEFINE_STATUS_ACCESSOR(name)                                                             \
  int name(int *status_out, int reset) {                                                            \
    int v = 0;                                                                                      \
    if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return MG_ERR_CUDA;  \
    if (status_out) *status_out = v;                                                                \
    if (reset && v != 0) {                                                                          \
      const int zero = 0;                                                                           \
      if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess) return MG_ERR_CUDA; \
    }                                                                                               \
    return MG_OK;                                                                                   \
  }

constexpr int kStatusWeightCopyTimeout = 101;
constexpr int kStatusActivationCopyTimeout = 102;
constexpr int kStatusMmaTimeout = 103;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// global -> this CTA's shared memory; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

constexpr uint32_t kWaitPolls = 1u << 22;

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Polls at most `polls` times; false when the phase did not complete.
static __device__ __noinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t polls) {
  for (uint32_t it = 0; it < polls; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 4) __nanosleep(40);  // waiting warps should not take issue slots from working ones
  }
  return false;
}

// The rare path of mbar_wait, kept out of line so that the loops that wait stay small.
static __device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  return mbar_wait_bounded(bar, parity, kWaitPolls);
}

// Returns false when the phase did not complete within kWaitPolls polls.  try_wait itself blocks for a
// hardware-defined time, so the first poll succeeds whenever the data is not far away.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}

__device__ __forceinline__ void report_status(int code) { atomicCAS(&g_device_status, 0, code); }

}  // namespace mg
