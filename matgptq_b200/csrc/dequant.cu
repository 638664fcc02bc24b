// Packed weights -> dense fp16/bf16 matrix W[N, K], bit-exact with the reference's
// dequantize() (src/quant_utils_matgpqt.py:19-22):
//     W = round_to_dtype(scale * ((code << (8 - b)) - zero)),  zero = 128 unless given.
// (code << (8-b)) - zero is an exact integer in fp16 and bf16; the product rounds once.
//
// The kernel decodes with the same in-register routine as the GEMV (decode.cuh),
// so that a bit-exact dense matrix also certifies the decode the GEMV runs on.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "decode.cuh"
#include "kernels.h"

namespace mg {

template <int B, int GS, bool BF16>
__global__ void __launch_bounds__(256) dequant_kernel(const uint32_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                                      const uint16_t *__restrict__ zeros, uint16_t *__restrict__ w_out, int tiles,
                                                      int kblocks, int K) {
  const int lane = threadIdx.x & 31;
  const long long blk = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (blk >= static_cast<long long>(tiles) * kblocks) return;
  const int tile = static_cast<int>(blk / kblocks), kb = static_cast<int>(blk % kblocks);
  const int g = lane >> 2, t = lane & 3;
  const int groups = (GS == -1) ? 1 : K / GS;

  uint32_t w[2 * B];
  load_block<B>(packed + blk * BlockTraits<B>::WORDS, lane, w);

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int grp;
    if constexpr (GS == 128) grp = kb;
    else if constexpr (GS == 32) grp = 4 * kb + (i >> 1);
    else grp = 0;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const size_t sidx = (static_cast<size_t>(tile) * groups + grp) * 16 + g + 8 * rr;
      const uint16_t sc = scales[sidx];
      const uint16_t zp = zeros ? zeros[sidx] : 0;
      uint2 o;
      o.x = dequant_pair<B, BF16>(decode_pair<B>(w, 4 * i + rr), sc, zeros != nullptr, zp);
      o.y = dequant_pair<B, BF16>(decode_pair<B>(w, 4 * i + 2 + rr), sc, zeros != nullptr, zp);
      const int row = tile * 16 + g + 8 * rr;
      const int col = kb * 128 + 32 * (i >> 1) + 8 * t + 4 * (i & 1);
      *reinterpret_cast<uint2 *>(w_out + static_cast<size_t>(row) * K + col) = o;
    }
  }
}

template <int B, int GS>
static int dequant_launch_t(const uint32_t *packed, const uint16_t *scales, const uint16_t *zeros, uint16_t *w_out, int N,
                            int K, bool bf16, cudaStream_t stream) {
  const int tiles = N / 16, kblocks = K / 128;
  const long long warps = static_cast<long long>(tiles) * kblocks;
  if (warps == 0) return MG_OK;
  const long long blocks = (warps + 7) / 8;
  if (bf16)
    dequant_kernel<B, GS, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(packed, scales, zeros, w_out, tiles, kblocks, K);
  else
    dequant_kernel<B, GS, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(packed, scales, zeros, w_out, tiles, kblocks, K);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <int B>
static int dequant_launch_b(const uint32_t *packed, const uint16_t *scales, const uint16_t *zeros, uint16_t *w_out, int N,
                            int K, int group_size, bool bf16, cudaStream_t stream) {
  switch (group_size) {
    case -1: return dequant_launch_t<B, -1>(packed, scales, zeros, w_out, N, K, bf16, stream);
    case 32: return dequant_launch_t<B, 32>(packed, scales, zeros, w_out, N, K, bf16, stream);
    case 128: return dequant_launch_t<B, 128>(packed, scales, zeros, w_out, N, K, bf16, stream);
    default: return MG_ERR_BAD_ARG;
  }
}

int dequant_launch(const uint32_t *packed, const uint16_t *scales, const uint16_t *zeros, uint16_t *w_out, int N, int K,
                   int bitwidth, int group_size, bool bf16, cudaStream_t stream) {
  switch (bitwidth) {
    case 2: return dequant_launch_b<2>(packed, scales, zeros, w_out, N, K, group_size, bf16, stream);
    case 3: return dequant_launch_b<3>(packed, scales, zeros, w_out, N, K, group_size, bf16, stream);
    case 4: return dequant_launch_b<4>(packed, scales, zeros, w_out, N, K, group_size, bf16, stream);
    case 6: return dequant_launch_b<6>(packed, scales, zeros, w_out, N, K, group_size, bf16, stream);
    case 8: return dequant_launch_b<8>(packed, scales, zeros, w_out, N, K, group_size, bf16, stream);
    default: return MG_ERR_BAD_ARG;
  }
}

}  // namespace mg
