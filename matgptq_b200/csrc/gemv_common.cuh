// Pieces shared by the GEMV kernels: the register-fragment MMA, accumulator chains per bit
// offset, scale and output conversions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "layout.cuh"

namespace mg {

// D = A*B + C on the tensor pipe, fp16 operands, fp32 accumulate.  ZERO_C starts a new
// accumulation without first clearing registers.
template <bool ZERO_C>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (ZERO_C) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Accumulator chains of a block.  A k-step whose fields decode at bit offset p carries
// the factor 2^p, so k-steps are spread over chains by offset; bitwidths with a single
// offset still use two chains so that consecutive mma do not depend on each other.
template <int B> struct Chains {
  static constexpr int N = (B == 2 || B == 3) ? 3 : 2;
  __host__ __device__ static constexpr int of(int i) { return (B == 2) ? i % 3 : (B == 3) ? (i < 3 ? 0 : (i < 6 ? 1 : 2)) : (i & 1); }
  __host__ __device__ static constexpr bool first(int i) { return (B == 3) ? (i == 0 || i == 3 || i == 6) : (i < N); }
  // 2^-offset of chain c
  __host__ __device__ static constexpr float inv_factor(int c) {
    return (B == 2) ? (c == 0 ? 1.f : (c == 1 ? 0.25f : 0.0625f))
                    : (B == 3) ? (c == 0 ? 1.f : (c == 1 ? 0.125f : 0.015625f)) : (B == 4) ? (c == 0 ? 1.f : 0.0625f) : 1.f;
  }
};

template <bool BF16> __device__ __forceinline__ float scale_to_float(uint16_t v) {
  if constexpr (BF16) {
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
  } else {
    return __half2float(__ushort_as_half(v));
  }
}

template <bool BF16> __device__ __forceinline__ uint16_t float_to_out(float v) {
  if constexpr (BF16) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  } else {
    return __half_as_ushort(__float2half_rn(v));
  }
}

__device__ __forceinline__ uint16_t ldg_u16(const uint16_t *p) {
  uint16_t r;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
  return r;
}

}  // namespace mg
