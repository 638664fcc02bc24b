// In-register decode of a lane's packed words into mma A fragments.
//
// Replaces the reference's plane merge + magic-number converters
// (csrc/matgptq_gemm.cu:90-295).  A pair of b-bit codes stored at bit offset p
// of both halves of a word is isolated by ONE LOP3 (field_pair).  Left as it is,
// the result is the half2 of fp16 subnormals (c_lo, c_hi) * 2^(p-24), which the
// tensor core multiplies exactly: the GEMV feeds these straight into mma and
// settles the factor 2^(24-p) and the zero point once per group in fp32.  With
// 0x6400 OR-ed in by the same LOP3 it is (1024 + c*2^p), and one HFMA2 with
// constants (2^-p, -(1024*2^-p + Z)) gives the exact integers (c - Z), Z = 2^(b-1)
// (decode_pair), for the paths that need dense weights.  Fields whose top bit
// would leave the 10-bit fp16 mantissa are reached through one shared right shift
// of the word.  On B200 LOP3, SHF, PRMT and HFMA2 all issue at half rate
// (16 lanes per clock and scheduler), which is why the GEMV avoids the HFMA2.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "layout.cuh"

namespace mg {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return r;
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

constexpr uint32_t kMagic = 0x64006400u;  // half2(1024, 1024)

// Bit pattern of an fp16 value that is exactly representable and normal, duplicated into both halves.
constexpr uint32_t half2_const(float v) {
  uint32_t sign = 0;
  if (v < 0.0f) {
    sign = 0x8000u;
    v = -v;
  }
  int e = 0;
  while (v >= 2.0f) {
    v *= 0.5f;
    ++e;
  }
  while (v < 1.0f) {
    v *= 2.0f;
    --e;
  }
  const uint32_t mant = static_cast<uint32_t>((v - 1.0f) * 1024.0f);
  const uint32_t h = sign | (static_cast<uint32_t>(e + 15) << 10) | mant;
  return h | (h << 16);
}

// (1024 + c*2^P) -> (c - Z) for both halves.
template <int Z, int P> __device__ __forceinline__ uint32_t normalize_at(uint32_t x) {
  constexpr float inv = 1.0f / static_cast<float>(1 << P);
  constexpr uint32_t mul = half2_const(inv);
  constexpr uint32_t add = half2_const(-(1024.0f * inv + static_cast<float>(Z)));
  return h2_bits(__hfma2(bits_h2(x), bits_h2(mul), bits_h2(add)));
}

// p is a compile-time constant at every call site once the caller's loops are unrolled.
template <int Z> __device__ __forceinline__ uint32_t normalize(uint32_t x, int p) {
  switch (p) {
    case 0: return normalize_at<Z, 0>(x);
    case 2: return normalize_at<Z, 2>(x);
    case 3: return normalize_at<Z, 3>(x);
    case 4: return normalize_at<Z, 4>(x);
    case 6: return normalize_at<Z, 6>(x);
    default: return normalize_at<Z, 8>(x);
  }
}

// Raw field pair P of a lane: both codes isolated at bit offset kstep_offset<B>(P >> 2)
// of their 16-bit halves, every other bit zero.  Read as half2 these are the subnormals
// code * 2^(offset - 24).  `orv` is OR-ed in by the same instruction (0, or the magic 0x64006400).
template <int B> __device__ __forceinline__ uint32_t field_pair(const uint32_t (&w)[2 * B], int P, uint32_t orv) {
  const int i = P >> 2, r = P & 3;
  if constexpr (B == 2) {
    const uint32_t W = w[r] >> (6 * (i / 3));
    return lop3_and_or(W, 0x00030003u << (2 * (i % 3)), orv);
  } else if constexpr (B == 4) {
    const int q = i & 3;
    const uint32_t W = w[4 * (i >> 2) + r] >> (8 * (q >> 1));
    return lop3_and_or(W, 0x000F000Fu << (4 * (q & 1)), orv);
  } else if constexpr (B == 8) {
    const uint32_t W = w[4 * (i >> 1) + r];
    if ((i & 1) == 0) return lop3_and_or(W, 0x00FF00FFu, orv);
    uint32_t x;
    asm("prmt.b32 %0, %1, %2, 0x7351;" : "=r"(x) : "r"(W), "r"(orv));  // bytes (W.b1, orv.b1, W.b3, orv.b3)
    return x;
  } else if constexpr (B == 3) {
    if (i < 6) {
      const int e = 4 * (i % 3) + r;
      const int u = e / 6, f = e % 6;
      const uint32_t W = w[3 * u + (f >> 1)] >> ((f & 1) ? 9 : 0);
      return lop3_and_or(W, 0x00070007u << (i < 3 ? 0 : 3), orv);
    }
    const int u = i - 6;
    if (r < 3) return lop3_and_or(w[3 * u + r], 0x01C001C0u, orv);
    uint32_t x = lop3_and_or(w[3 * u] >> 9, 0x00400040u, orv);
    x = lop3_and_or(w[3 * u + 1] >> 8, 0x00800080u, x);
    x = lop3_and_or(w[3 * u + 2] >> 7, 0x01000100u, x);
    return x;
  } else {
    static_assert(B == 6, "bitwidth must be one of 2, 3, 4, 6, 8");
    const int u = i >> 1, e = 4 * (i & 1) + r;
    if (e < 6) {
      const uint32_t W = w[3 * u + (e >> 1)] >> (6 * (e & 1));
      return lop3_and_or(W, 0x003F003Fu, orv);
    }
    uint32_t x;
    if (e == 6) {
      x = lop3_and_or(w[3 * u] >> 12, 0x000F000Fu, orv);
      x = lop3_and_or(w[3 * u + 1] >> 8, 0x00300030u, x);
    } else {
      x = lop3_and_or(w[3 * u + 1] >> 14, 0x00030003u, orv);
      x = lop3_and_or(w[3 * u + 2] >> 10, 0x003C003Cu, x);
    }
    return x;
  }
}

// Decoded pair P of a lane as half2 of exact integers (code - Z).
template <int B> __device__ __forceinline__ uint32_t decode_pair(const uint32_t (&w)[2 * B], int P) {
  constexpr int Z = BlockTraits<B>::ZERO;
  return normalize<Z>(field_pair<B>(w, P, kMagic), kstep_offset<B>(P >> 2));
}

// half2 of small exact integers -> bfloat162 of the same integers.
__device__ __forceinline__ uint32_t h2_to_bf2(uint32_t v) {
  const float2 f = __half22float2(bits_h2(v));
  const __nv_bfloat162 r = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t *>(&r);
}

__device__ __forceinline__ uint32_t splat16(uint16_t v) {
  return static_cast<uint32_t>(v) | (static_cast<uint32_t>(v) << 16);
}

// v: pair of exact integers (code - Z) as half2.  Returns the dequantised pair in the output dtype.
template <int B, bool BF16>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t v, uint16_t scale, bool has_zero, uint16_t zero) {
  constexpr float kShift = static_cast<float>(1 << (8 - B));
  if constexpr (BF16) {
    const uint32_t vb = h2_to_bf2(v);
    const __nv_bfloat162 vi = *reinterpret_cast<const __nv_bfloat162 *>(&vb);
    const __nv_bfloat162 sh = __float2bfloat162_rn(kShift);
    __nv_bfloat162 off = __float2bfloat162_rn(0.f);
    if (has_zero) {
      const uint32_t zb = splat16(zero);
      off = __hsub2(__float2bfloat162_rn(128.f), *reinterpret_cast<const __nv_bfloat162 *>(&zb));
    }
    const __nv_bfloat162 q = __hfma2(vi, sh, off);  // exact integer
    const uint32_t sb = splat16(scale);
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&sb), q);
    return *reinterpret_cast<const uint32_t *>(&r);
  } else {
    const __half2 vi = bits_h2(v);
    const __half2 sh = __float2half2_rn(kShift);
    __half2 off = __float2half2_rn(0.f);
    if (has_zero) off = __hsub2(__float2half2_rn(128.f), bits_h2(splat16(zero)));
    const __half2 q = __hfma2(vi, sh, off);  // exact integer
    return h2_bits(__hmul2(bits_h2(splat16(scale)), q));
  }
}

// Dense-weight tiles of the tensor-core path: pair P of a lane as s * (code - Z) * 2^(8-b), bit-exact with
// dequant_pair(decode_pair(..)), in three instructions for fp16 (LOP3, HFMA2, HMUL2).  The
// HFMA2 turns 1024 + code*2^p straight into the exact integer (code - Z) * kDensePre; the rest of 2^(8-b)
// (a factor 2, for b = 2 only, where (1024 + Z) * 64 would leave the fp16 range) is folded into the scale by
// dense_scale().  The product is rounded once, as in dequantize() (src/quant_utils_matgpqt.py:19-22).
template <int B> struct DensePre {
  static constexpr int value = (B == 2) ? 32 : (1 << (8 - B));
};

// A finite scale whose multiple leaves the finite range is clamped to the largest finite value instead of
// becoming infinite: times a code off the zero point the product overflows to the same infinity that
// dequantize() gives, and times the code on the zero point it stays zero (infinity would make it NaN).
template <int B, bool BF16> __device__ __forceinline__ uint32_t dense_scale(uint16_t scale) {
  constexpr float rest = static_cast<float>((1 << (8 - B)) / DensePre<B>::value);
  if constexpr (rest == 1.f) return splat16(scale);
  constexpr uint16_t kInf = BF16 ? 0x7F80u : 0x7C00u;
  uint16_t r;
  if constexpr (BF16) {
    r = __bfloat16_as_ushort(__hmul(__ushort_as_bfloat16(scale), __float2bfloat16_rn(rest)));
  } else {
    r = __half_as_ushort(__hmul(__ushort_as_half(scale), __float2half_rn(rest)));
  }
  if ((r & 0x7FFFu) == kInf && (scale & 0x7FFFu) != kInf) r -= 1;  // largest finite value of the same sign
  return splat16(r);
}

template <int B, int P_OFF> __device__ __forceinline__ uint32_t dense_int_at(uint32_t x) {
  constexpr int Z = BlockTraits<B>::ZERO;
  constexpr float pre = static_cast<float>(DensePre<B>::value);
  constexpr float inv = pre / static_cast<float>(1 << P_OFF);
  constexpr uint32_t mul = half2_const(inv);
  constexpr uint32_t add = half2_const(-(1024.0f * inv + static_cast<float>(Z) * pre));
  return h2_bits(__hfma2(bits_h2(x), bits_h2(mul), bits_h2(add)));
}

// Bit pattern of a bfloat16 value that is exactly representable and normal, duplicated into both halves.
constexpr uint32_t bf162_const(float v) {
  uint32_t sign = 0;
  if (v < 0.0f) {
    sign = 0x8000u;
    v = -v;
  }
  int e = 0;
  while (v >= 2.0f) {
    v *= 0.5f;
    ++e;
  }
  while (v < 1.0f) {
    v *= 2.0f;
    --e;
  }
  const uint32_t mant = static_cast<uint32_t>((v - 1.0f) * 128.0f);
  const uint32_t h = sign | (static_cast<uint32_t>(e + 127) << 7) | mant;
  return h | (h << 16);
}

// (128 + c*2^P) -> (c - Z) * DensePre<B> for both bfloat16 halves, one fused multiply-add with exact operands
template <int B, int P_OFF> __device__ __forceinline__ uint32_t dense_int_bf16_at(uint32_t x) {
  constexpr float pre = static_cast<float>(DensePre<B>::value);
  constexpr float inv = pre / static_cast<float>(1 << P_OFF);
  constexpr uint32_t mul = bf162_const(inv);
  constexpr uint32_t add = bf162_const(-(128.0f * inv + static_cast<float>(BlockTraits<B>::ZERO) * pre));
  const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162 *>(&x), *reinterpret_cast<const __nv_bfloat162 *>(&mul),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&add));
  return *reinterpret_cast<const uint32_t *>(&r);
}

// Pair P of a lane as bfloat16 integers (code - Z) * DensePre<B>, WITHOUT the detour over fp16 (magic, fma, two
// conversions): the field is isolated inside the 7 mantissa bits of bfloat16 with the exponent of 128 OR-ed in by
// the same LOP3 (value 128 + code * 2^p), and one bfloat16 fma makes the integer.  Needs code * 2^p < 128, i.e.
// the field shifted down to bit 0 first where it sits higher (every 4-bit field but the lowest, the third offset of
// 3-bit codes); 8-bit codes go in as two fields.
template <int B> __device__ __forceinline__ uint32_t dense_int_bf16(const uint32_t (&w)[2 * B], int P) {
  constexpr uint32_t kMagicBf = 0x43004300u;  // bfloat162(128, 128)
  const int i = P >> 2, r = P & 3;
  if constexpr (B == 8) {
    // Eight bits do not fit the 7 mantissa bits, so the code goes in as two fields: the low seven bits under the
    // magic (t = 128 + low) and the top bit on the exponent's lowest bit (q = 128 or 256).  Then
    // code - 128 = t + (q - 384), two bfloat16 additions whose results are exact (-256 or -128, then -128..127).
    const uint32_t W = w[4 * (i >> 1) + r] >> (8 * (i & 1));
    const uint32_t t = lop3_and_or(W, 0x007F007Fu, kMagicBf);
    const uint32_t q = lop3_and_or(W, 0x00800080u, kMagicBf);
    constexpr uint32_t k384 = bf162_const(-384.0f);
    const __nv_bfloat162 u = __hadd2(*reinterpret_cast<const __nv_bfloat162 *>(&q), *reinterpret_cast<const __nv_bfloat162 *>(&k384));
    const __nv_bfloat162 v = __hadd2(*reinterpret_cast<const __nv_bfloat162 *>(&t), u);
    static_assert(DensePre<8>::value == 1, "8-bit codes are used as they are");
    return *reinterpret_cast<const uint32_t *>(&v);
  } else if constexpr (B == 4) {
    const uint32_t W = w[4 * (i >> 2) + r] >> (4 * (i & 3));
    return dense_int_bf16_at<4, 0>(lop3_and_or(W, 0x000F000Fu, kMagicBf));
  } else if constexpr (B == 3) {
    if (i < 3) return dense_int_bf16_at<3, 0>(field_pair<3>(w, P, kMagicBf));
    if (i < 6) return dense_int_bf16_at<3, 3>(field_pair<3>(w, P, kMagicBf));
    return dense_int_bf16_at<3, 0>((field_pair<3>(w, P, 0u) >> 6) | kMagicBf);
  } else if constexpr (B == 2) {
    const uint32_t x = field_pair<2>(w, P, kMagicBf);
    switch (kstep_offset<2>(i)) {
      case 0: return dense_int_bf16_at<2, 0>(x);
      case 2: return dense_int_bf16_at<2, 2>(x);
      default: return dense_int_bf16_at<2, 4>(x);
    }
  } else {
    return dense_int_bf16_at<6, 0>(field_pair<6>(w, P, kMagicBf));
  }
}

// scale2: dense_scale() of the row's scale
template <int B, bool BF16>
__device__ __forceinline__ uint32_t dense_pair(const uint32_t (&w)[2 * B], int P, uint32_t scale2) {
  if constexpr (BF16) {
    const uint32_t vb = dense_int_bf16<B>(w, P);
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&scale2), *reinterpret_cast<const __nv_bfloat162 *>(&vb));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  const uint32_t x = field_pair<B>(w, P, kMagic);
  uint32_t v;
  switch (kstep_offset<B>(P >> 2)) {  // a compile-time constant once the caller's loops are unrolled
    case 0: v = dense_int_at<B, 0>(x); break;
    case 2: v = dense_int_at<B, 2>(x); break;
    case 3: v = dense_int_at<B, 3>(x); break;
    case 4: v = dense_int_at<B, 4>(x); break;
    case 6: v = dense_int_at<B, 6>(x); break;
    default: v = dense_int_at<B, 8>(x); break;
  }
  return h2_bits(__hmul2(bits_h2(scale2), bits_h2(v)));
}

// Coalesced load of a lane's words of one block (all lanes of a warp call it).
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void *p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}

template <int B> __device__ __forceinline__ void load_block(const uint32_t *blk, int lane, uint32_t (&w)[2 * B]) {
  constexpr int NV = BlockTraits<B>::NV;
  constexpr int TAIL = BlockTraits<B>::TAIL;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const uint4 q = ldg_stream_v4(blk + v * 128 + lane * 4);
    w[4 * v + 0] = q.x;
    w[4 * v + 1] = q.y;
    w[4 * v + 2] = q.z;
    w[4 * v + 3] = q.w;
  }
  if constexpr (TAIL == 2) {
    const uint2 q = ldg_stream_v2(blk + NV * 128 + lane * 2);
    w[4 * NV + 0] = q.x;
    w[4 * NV + 1] = q.y;
  }
}

}  // namespace mg
