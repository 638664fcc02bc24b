// Packed weight layout of the B200 bit-sliced linear layer, shared by the host
// packer, the GPU packer and every kernel that decodes it.
//
// The reference packs b-bit codes into mma.m16n8k16 A-fragment order as up to
// eight nibble-aligned bit-plane arrays (csrc/utils.cpp:22-217, kernel side
// csrc/matgptq_gemm.cu:196-279).  The packed tensor is opaque to every caller of
// the three ops (only dtype u32, 1-D and numel == b*N*K/32 are checked,
// csrc/bindings.cpp:157-160), so this implementation uses its own layout:
//
//   * The weight matrix [N, K] is cut into BLOCKS of 16 out-features x 128
//     in-features (one scale group when group_size == 128).  Blocks are stored
//     row-tile major: block (tile, kb) starts at u32 index (tile*K/128 + kb)*64*b.
//   * A block is decoded by one warp.  Each lane owns 64 codes = 32 code PAIRS =
//     the A fragments of 8 mma k-steps, held in 2*b 32-bit words.
//   * Words are stored so that a warp reads them with fully coalesced 16-byte
//     loads: word j of lane l sits at (j/4)*128 + l*4 + j%4; the two words of a
//     3-bit block that do not fill a 16-byte vector follow as 8 bytes per lane.
//   * In a word the two codes of a pair sit at the same bit offset of the low
//     and the high 16-bit half, so that ONE logic instruction (after at most one
//     shared shift of the word) isolates them as a half2 whose halves are the fp16
//     subnormals code * 2^(offset-24); the tensor core multiplies subnormals
//     exactly.  OR-ing 0x6400 into the same bits gives (1024 + code * 2^offset),
//     the classic magic-number form, where exact integers are wanted instead.
//   * The four A registers of one mma k-step always come from fields at the same
//     bit offset, so a whole k-step carries one power-of-two factor; k-steps with
//     different factors accumulate into different accumulators.
//   * 3-bit and 6-bit codes do not tile 16 bits: five (two) fields per half are
//     stored directly and the spare bits of three consecutive words carry one
//     (two) more pair(s).
//
// Pair P (0..31) of lane (g = lane/4, t = lane%4) covers, for h in {0,1}:
//     row = g + 8*(P&1)
//     col = 32*(P>>3) + 8*t + 4*((P>>2)&1) + 2*((P>>1)&1) + h        (inside the block)
// i.e. pairs 4i..4i+3 are registers a0..a3 of k-step i, and the four k-slots a
// lane holds in one k-step map to four consecutive in-features, so that a lane's
// B fragments for two k-steps are 16 contiguous bytes of an activation row.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MG_HD __host__ __device__ __forceinline__
#else
#define MG_HD inline
#endif

namespace mg {

constexpr int kTileRows = 16;
constexpr int kBlockK = 128;
constexpr int kPairs = 32;

template <int B> struct BlockTraits {
  static constexpr int WPL = 2 * B;          // words per lane per block
  static constexpr int NV = WPL / 4;         // full 16-byte vectors per lane
  static constexpr int TAIL = WPL - 4 * NV;  // remaining words per lane (0 or 2)
  static constexpr int WORDS = 64 * B;       // u32 per block
  static constexpr int ZERO = 1 << (B - 1);  // implicit zero point in sliced units
};

// u32 index, inside a block, of word j of a lane.
template <int B> MG_HD int word_slot(int lane, int j) {
  constexpr int NV = BlockTraits<B>::NV;
  constexpr int TAIL = BlockTraits<B>::TAIL;
  if (j < 4 * NV) return (j >> 2) * 128 + lane * 4 + (j & 3);
  return NV * 128 + lane * TAIL + (j - 4 * NV);
}

// Matrix coordinates (inside the block) of half h of pair P of a lane.
MG_HD void pair_coord(int lane, int P, int h, int &row, int &col) {
  const int g = lane >> 2, t = lane & 3;
  row = g + 8 * (P & 1);
  col = 32 * (P >> 3) + 8 * t + 4 * ((P >> 2) & 1) + 2 * ((P >> 1) & 1) + h;
}

// Where the bits of one code live: `nbits` bits of the code starting at bit
// `cshift` are stored in word `word` at bit `off`.
struct Piece {
  int word, off, nbits, cshift;
};

template <int B> MG_HD int code_pieces(int P, int h, Piece (&out)[3]) {
  const int hb = 16 * h;
  const int i = P >> 2, r = P & 3;  // mma k-step and A register
  if (B == 2) {
    // one 16-byte vector per lane: register r of k-step i is field i of word r
    out[0] = {r, hb + 2 * i, 2, 0};
    return 1;
  } else if (B == 4) {
    out[0] = {4 * (i >> 2) + r, hb + 4 * (i & 3), 4, 0};
    return 1;
  } else if (B == 8) {
    out[0] = {4 * (i >> 1) + r, hb + 8 * (i & 1), 8, 0};
    return 1;
  } else if (B == 3) {
    // two units of three words; fields at bits 0,3,6,9,12 of each half, bit 15 spare.
    // k-steps 0-2 take the fields that decode at offset 0 (bits 0 and 9), k-steps 3-5
    // those at offset 3 (bits 3 and 12), k-steps 6-7 those at offset 6 plus the pair
    // assembled from the spare bits.
    if (i < 6) {
      const int e = 4 * (i % 3) + r;  // 0..11 inside the class
      const int u = e / 6, f = e % 6;
      const int q = (i < 3) ? ((f & 1) ? 3 : 0) : ((f & 1) ? 4 : 1);
      out[0] = {3 * u + (f >> 1), hb + 3 * q, 3, 0};
      return 1;
    }
    const int u = i - 6;
    if (r < 3) {
      out[0] = {3 * u + r, hb + 6, 3, 0};
      return 1;
    }
    out[0] = {3 * u + 0, hb + 15, 1, 0};
    out[1] = {3 * u + 1, hb + 15, 1, 1};
    out[2] = {3 * u + 2, hb + 15, 1, 2};
    return 3;
  } else {  // B == 6
    // four units of three words; fields at bits 0 and 6 of each half, bits 12-15 spare
    const int u = i >> 1, e = 4 * (i & 1) + r;
    if (e < 6) {
      out[0] = {3 * u + (e >> 1), hb + 6 * (e & 1), 6, 0};
      return 1;
    }
    if (e == 6) {
      out[0] = {3 * u + 0, hb + 12, 4, 0};
      out[1] = {3 * u + 1, hb + 12, 2, 4};
      return 2;
    }
    out[0] = {3 * u + 1, hb + 14, 2, 0};
    out[1] = {3 * u + 2, hb + 12, 4, 2};
    return 2;
  }
}

// Bit offset (inside the 10-bit fp16 mantissa) at which the fields of k-step i decode.
template <int B> MG_HD constexpr int kstep_offset(int i) {
  return (B == 2) ? 2 * (i % 3) : (B == 4) ? 4 * (i & 1) : (B == 3) ? (i < 3 ? 0 : (i < 6 ? 3 : 6)) : 0;
}

// Store code c (b bits) as half h of pair P into a lane's words.
template <int B> MG_HD void place_code(uint32_t (&w)[2 * B], int P, int h, uint32_t c) {
  Piece pc[3];
  const int n = code_pieces<B>(P, h, pc);
  for (int i = 0; i < n; ++i) {
    const uint32_t bits = (c >> pc[i].cshift) & ((1u << pc[i].nbits) - 1u);
    w[pc[i].word] |= bits << pc[i].off;
  }
}

// Plain integer extraction, the inverse of place_code (no floating-point tricks).
template <int B> MG_HD uint32_t extract_code(const uint32_t (&w)[2 * B], int P, int h) {
  Piece pc[3];
  const int n = code_pieces<B>(P, h, pc);
  uint32_t c = 0;
  for (int i = 0; i < n; ++i) {
    const uint32_t bits = (w[pc[i].word] >> pc[i].off) & ((1u << pc[i].nbits) - 1u);
    c |= bits << pc[i].cshift;
  }
  return c;
}

// Round-to-nearest MSB slice with saturation (src/quant_utils_matgpqt.py:9-17):
// the drop is 8 - b whatever the master bitwidth; no rounding bit when b == master.
MG_HD uint32_t matryoshka_slice(uint32_t x, int master_bitwidth, int b) {
  const int drop = 8 - b;
  uint32_t v = x >> drop;
  if (master_bitwidth != b && drop > 0) v += (x >> (drop - 1)) & 1u;
  const uint32_t maxq = (1u << b) - 1u;
  return v > maxq ? maxq : v;
}

}  // namespace mg
