// Load-time kernels: MSB slicing, weight packing and scale reordering, each with
// a host (CPU) twin that uses the same layout functions.
//
// Replaces matryoshka_slice (src/quant_utils_matgpqt.py:9-17), the single-threaded
// CPU packers swizzle_weights / split_up_n_bits / swizzle_matgptq
// (csrc/utils.cpp:22-217) behind pack_matgptq_qweights (csrc/bindings.cpp:43-84)
// and reorder_matgptq_scales (csrc/bindings.cpp:86-142).  The reference copies the
// codes to the host, packs on one thread and copies back; here slicing and
// packing are one pass over the codes on the GPU.
#include <cuda_runtime.h>

#include <cstring>

#include "kernels.h"
#include "layout.cuh"

namespace mg {

// ---------------------------------------------------------------------------
// slicing
// ---------------------------------------------------------------------------
__global__ void slice_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, long long numel,
                             int master_bitwidth, int bitwidth) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nvec = numel / 16;
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (aligned) {
    for (long long v = tid; v < nvec; v += stride) {
      uint4 q = reinterpret_cast<const uint4 *>(in)[v];
      uint32_t *words = reinterpret_cast<uint32_t *>(&q);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t o = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) o |= matryoshka_slice((words[i] >> (8 * e)) & 0xFFu, master_bitwidth, bitwidth) << (8 * e);
        words[i] = o;
      }
      reinterpret_cast<uint4 *>(out)[v] = q;
    }
    for (long long i = nvec * 16 + tid; i < numel; i += stride) out[i] = static_cast<uint8_t>(matryoshka_slice(in[i], master_bitwidth, bitwidth));
  } else {
    for (long long i = tid; i < numel; i += stride) out[i] = static_cast<uint8_t>(matryoshka_slice(in[i], master_bitwidth, bitwidth));
  }
}

int slice_launch(const uint8_t *in, uint8_t *out, long long numel, int master_bitwidth, int bitwidth,
                 cudaStream_t stream) {
  if (numel == 0) return MG_OK;
  const int threads = 256;
  long long blocks = (numel / 16 + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  slice_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(in, out, numel, master_bitwidth, bitwidth);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// packing: one thread builds the 2*b words that one lane will later decode
// ---------------------------------------------------------------------------
template <int B>
MG_HD void pack_lane(const uint8_t *codes, int K, int tile, int kb, int lane, int slice_from_master,
                     uint32_t (&w)[2 * B]) {
  for (int j = 0; j < 2 * B; ++j) w[j] = 0u;
  const int g = lane >> 2, t = lane & 3;
  for (int i = 0; i < 8; ++i) {
    for (int rr = 0; rr < 2; ++rr) {
      const int row = tile * 16 + g + 8 * rr;
      const int col = kb * 128 + 32 * (i >> 1) + 8 * t + 4 * (i & 1);
      const uint8_t *src = codes + static_cast<size_t>(row) * K + col;
      for (int e = 0; e < 4; ++e) {
        uint32_t c = src[e];
        if (slice_from_master > 0) c = matryoshka_slice(c, slice_from_master, B);
        c &= (1u << B) - 1u;
        place_code<B>(w, 4 * i + 2 * (e >> 1) + rr, e & 1, c);
      }
    }
  }
}

template <int B>
__global__ void pack_kernel(const uint8_t *__restrict__ codes, uint32_t *__restrict__ packed, int tiles, int kblocks,
                            int K, int slice_from_master) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nblocks = static_cast<long long>(tiles) * kblocks;
  const long long blk = gid >> 5;
  const int lane = static_cast<int>(gid & 31);
  if (blk >= nblocks) return;
  const int tile = static_cast<int>(blk / kblocks), kb = static_cast<int>(blk % kblocks);
  uint32_t w[2 * B];
  pack_lane<B>(codes, K, tile, kb, lane, slice_from_master, w);
  uint32_t *dst = packed + blk * BlockTraits<B>::WORDS;
#pragma unroll
  for (int j = 0; j < 2 * B; ++j) dst[word_slot<B>(lane, j)] = w[j];
}

template <int B>
static int pack_launch_b(const uint8_t *codes, uint32_t *packed, int N, int K, int slice_from_master,
                         cudaStream_t stream) {
  const int tiles = N / 16, kblocks = K / 128;
  const long long threads_total = static_cast<long long>(tiles) * kblocks * 32;
  if (threads_total == 0) return MG_OK;
  const int threads = 128;
  const long long blocks = (threads_total + threads - 1) / threads;
  pack_kernel<B><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(codes, packed, tiles, kblocks, K, slice_from_master);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

int pack_launch(const uint8_t *codes, uint32_t *packed, int N, int K, int bitwidth, int slice_from_master,
                cudaStream_t stream) {
  switch (bitwidth) {
    case 2: return pack_launch_b<2>(codes, packed, N, K, slice_from_master, stream);
    case 3: return pack_launch_b<3>(codes, packed, N, K, slice_from_master, stream);
    case 4: return pack_launch_b<4>(codes, packed, N, K, slice_from_master, stream);
    case 6: return pack_launch_b<6>(codes, packed, N, K, slice_from_master, stream);
    case 8: return pack_launch_b<8>(codes, packed, N, K, slice_from_master, stream);
    default: return MG_ERR_BAD_ARG;
  }
}

template <int B> static void pack_host_b(const uint8_t *codes, uint32_t *packed, int N, int K, int slice_from_master) {
  const int tiles = N / 16, kblocks = K / 128;
  for (int tile = 0; tile < tiles; ++tile)
    for (int kb = 0; kb < kblocks; ++kb) {
      uint32_t *dst = packed + (static_cast<size_t>(tile) * kblocks + kb) * BlockTraits<B>::WORDS;
      for (int lane = 0; lane < 32; ++lane) {
        uint32_t w[2 * B];
        pack_lane<B>(codes, K, tile, kb, lane, slice_from_master, w);
        for (int j = 0; j < 2 * B; ++j) dst[word_slot<B>(lane, j)] = w[j];
      }
    }
}

int pack_host(const uint8_t *codes, uint32_t *packed, int N, int K, int bitwidth, int slice_from_master) {
  switch (bitwidth) {
    case 2: pack_host_b<2>(codes, packed, N, K, slice_from_master); return MG_OK;
    case 3: pack_host_b<3>(codes, packed, N, K, slice_from_master); return MG_OK;
    case 4: pack_host_b<4>(codes, packed, N, K, slice_from_master); return MG_OK;
    case 6: pack_host_b<6>(codes, packed, N, K, slice_from_master); return MG_OK;
    case 8: pack_host_b<8>(codes, packed, N, K, slice_from_master); return MG_OK;
    default: return MG_ERR_BAD_ARG;
  }
}

template <int B> static void unpack_host_b(const uint32_t *packed, uint8_t *codes, int N, int K) {
  const int tiles = N / 16, kblocks = K / 128;
  for (int tile = 0; tile < tiles; ++tile)
    for (int kb = 0; kb < kblocks; ++kb) {
      const uint32_t *src = packed + (static_cast<size_t>(tile) * kblocks + kb) * BlockTraits<B>::WORDS;
      for (int lane = 0; lane < 32; ++lane) {
        uint32_t w[2 * B];
        for (int j = 0; j < 2 * B; ++j) w[j] = src[word_slot<B>(lane, j)];
        for (int P = 0; P < kPairs; ++P)
          for (int h = 0; h < 2; ++h) {
            int row, col;
            pair_coord(lane, P, h, row, col);
            codes[static_cast<size_t>(tile * 16 + row) * K + kb * 128 + col] = static_cast<uint8_t>(extract_code<B>(w, P, h));
          }
      }
    }
}

int unpack_host(const uint32_t *packed, uint8_t *codes, int N, int K, int bitwidth) {
  switch (bitwidth) {
    case 2: unpack_host_b<2>(packed, codes, N, K); return MG_OK;
    case 3: unpack_host_b<3>(packed, codes, N, K); return MG_OK;
    case 4: unpack_host_b<4>(packed, codes, N, K); return MG_OK;
    case 6: unpack_host_b<6>(packed, codes, N, K); return MG_OK;
    case 8: unpack_host_b<8>(packed, codes, N, K); return MG_OK;
    default: return MG_ERR_BAD_ARG;
  }
}

// ---------------------------------------------------------------------------
// scales: [N, G] -> [N/16, G, 16] so that the 16 scales a warp needs for one
// block are one 32-byte sector (same order as csrc/bindings.cpp:113-119)
// ---------------------------------------------------------------------------
__global__ void reorder_scales_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, int N, int G) {
  const long long total = static_cast<long long>(N) * G;
  for (long long o = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
       o += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(o & 15);
    const long long tg = o >> 4;
    const int grp = static_cast<int>(tg % G);
    const long long tile = tg / G;
    out[o] = in[(tile * 16 + r) * G + grp];
  }
}

int reorder_scales_launch(const uint16_t *in, uint16_t *out, int N, int K, int group_size, cudaStream_t stream) {
  const int G = group_size == -1 ? 1 : K / group_size;
  const long long total = static_cast<long long>(N) * G;
  if (total == 0) return MG_OK;
  if (G == 1) {
    return cudaMemcpyAsync(out, in, total * 2, cudaMemcpyDeviceToDevice, stream) == cudaSuccess ? MG_OK : MG_ERR_CUDA;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  reorder_scales_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(in, out, N, G);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

int reorder_scales_host(const uint16_t *in, uint16_t *out, int N, int K, int group_size) {
  const int G = group_size == -1 ? 1 : K / group_size;
  for (long long tile = 0; tile < N / 16; ++tile)
    for (int grp = 0; grp < G; ++grp)
      for (int r = 0; r < 16; ++r) out[(tile * G + grp) * 16 + r] = in[(tile * 16 + r) * G + grp];
  return MG_OK;
}

}  // namespace mg
