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
//     and the high 16-bit half, so that one LOP3 turns them into a half2 of
//     (1024 + code * 2^offset) (the fp16 "magic number" conversion).
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
  if (B == 2) {
    out[0] = {P >> 3, hb + 2 * (P & 7), 2, 0};
    return 1;
  } else if (B == 4) {
    out[0] = {P >> 2, hb + 4 * (P & 3), 4, 0};
    return 1;
  } else if (B == 8) {
    out[0] = {P >> 1, hb + 8 * (P & 1), 8, 0};
    return 1;
  } else if (B == 3) {
    const int u = P >> 4, p = P & 15;
    if (p < 15) {
      out[0] = {3 * u + p / 5, hb + 3 * (p % 5), 3, 0};
      return 1;
    }
    out[0] = {3 * u + 0, hb + 15, 1, 0};
    out[1] = {3 * u + 1, hb + 15, 1, 1};
    out[2] = {3 * u + 2, hb + 15, 1, 2};
    return 3;
  } else {  // B == 6
    const int u = P >> 3, p = P & 7;
    if (p < 6) {
      out[0] = {3 * u + (p >> 1), hb + 6 * (p & 1), 6, 0};
      return 1;
    }
    if (p == 6) {
      out[0] = {3 * u + 0, hb + 12, 4, 0};
      out[1] = {3 * u + 1, hb + 12, 2, 4};
      return 2;
    }
    out[0] = {3 * u + 1, hb + 14, 2, 0};
    out[1] = {3 * u + 2, hb + 12, 4, 2};
    return 2;
  }
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
