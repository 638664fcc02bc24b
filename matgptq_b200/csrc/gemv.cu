// Bit-sliced GEMV family for small batches (1..16 activation rows per pass).
//
// Replaces gptq_matryoshka_simt / gptq_matryoshka and their dispatch
// (csrc/matgptq_gemm.cu:337-953, 955-1065).  y[M,N] = x[M,K] . Wdq^T with
// Wdq[n,k] = (q[n,k] - 2^(b-1)) * s[n, k/g] * 2^(8-b), fp32 accumulation.
//
// Shape of the computation
//   * one warp streams 16 out-features x a K slice: per block (16 x 128 codes) it
//     issues 16-byte coalesced loads, decodes its 64 codes in registers straight
//     into mma.m16n8k16 A fragments (exact integers), multiplies them with the
//     activation fragments on the tensor pipe into a per-group fp32 accumulator
//     and folds the group's scale in fp32 (one FMA per accumulator and group);
//   * the R warps of a CTA cover R consecutive row tiles over the same K slice and
//     share the activation slice staged once in shared memory;
//   * K is split over the S CTAs of a thread-block cluster (split-K for skinny
//     shapes); partial sums meet in distributed shared memory and are added in a
//     fixed order, so results do not depend on scheduling and no global scratch
//     or atomics are used;
//   * weight loads of the first blocks are issued before griddepcontrol.wait, so
//     with programmatic dependent launch they overlap the previous kernel's tail.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "decode.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace mg {

struct GemvParams {
  const uint32_t *w;
  const uint16_t *s;
  const uint16_t *x;
  uint16_t *y;
  int N, K, M;
  int tiles;    // N / 16
  int kblocks;  // K / 128
  int split;    // CTAs per cluster along K
};

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

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

// Scales a lane needs for one block: rows g and g+8 of each group in the block.
template <int GS> struct ScaleRegs {
  static constexpr int NG = (GS == 32) ? 4 : 1;
  uint16_t lo[NG], hi[NG];
};

template <int GS>
__device__ __forceinline__ void load_scales(const uint16_t *s, int tile, int kb, int groups, int lane, ScaleRegs<GS> &r) {
  if constexpr (GS == -1) {
    (void)s; (void)tile; (void)kb; (void)groups; (void)lane; (void)r;
  } else {
    constexpr int NG = ScaleRegs<GS>::NG;
    const uint16_t *base = s + (static_cast<size_t>(tile) * groups + static_cast<size_t>(kb) * NG) * 16 + (lane >> 2);
#pragma unroll
    for (int j = 0; j < NG; ++j) {
      r.lo[j] = ldg_u16(base + j * 16);
      r.hi[j] = ldg_u16(base + j * 16 + 8);
    }
  }
}

// B: bitwidth, GS: group size (-1, 32, 128), BF16: activation/scale/output type,
// NT: batch tiles of 8 rows handled per pass, D: blocks a warp keeps in flight.
template <int B, int GS, bool BF16, int NT, int D>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int R = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int S = p.split;
  const int crank = (S > 1) ? static_cast<int>(cg::this_cluster().block_rank()) : 0;
  const int rg = blockIdx.x / S;
  const int tile = rg * R + warp;
  const bool active = tile < p.tiles;
  const int kb_lo = static_cast<int>(static_cast<long long>(crank) * p.kblocks / S);
  const int kb_hi = static_cast<int>(static_cast<long long>(crank + 1) * p.kblocks / S);
  const int nblk = kb_hi - kb_lo;
  const int max_nblk = (p.kblocks + S - 1) / S;
  const int m0 = blockIdx.y * (NT * 8);
  const int mvalid = min(p.M - m0, NT * 8);
  const int groups = (GS == -1) ? 1 : p.K / GS;

  // shared memory: activation stage [NT*8][stage + 32 halves], then partial sums [NT*8][R*16 + 4] floats
  constexpr int XB = D * ((16 + D - 1) / D);  // blocks per activation stage, a multiple of D
  const int stage_blocks = min(max_nblk, XB);
  const int xstride = stage_blocks * 128 + 32;  // halves; +64 bytes keeps 16-byte fragment reads conflict free
  uint16_t *xs = reinterpret_cast<uint16_t *>(smem_raw);
  const int rstride = R * 16 + 4;
  float *red = reinterpret_cast<float *>(smem_raw + static_cast<size_t>(NT * 8) * xstride * 2);

  constexpr int BW = BlockTraits<B>::WORDS;
  const uint32_t *wbase = p.w + (static_cast<size_t>(active ? tile : 0) * p.kblocks + kb_lo) * BW;

  uint32_t wbuf[D][2 * B];
  ScaleRegs<GS> sbuf[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    if (active && d < nblk) {
      load_block<B>(wbase + static_cast<size_t>(d) * BW, lane, wbuf[d]);
      load_scales<GS>(p.s, tile, kb_lo + d, groups, lane, sbuf[d]);
    }
  }

  // Everything above reads only weights and scales, which no kernel writes.  The
  // activations may come from the kernel launched just before this one.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float yacc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) yacc[nt][e] = 0.f;

  for (int st = 0; st < nblk; st += XB) {
    // stage the activations of blocks [st, st + XB) of this CTA's K slice
    const int st_blocks = min(XB, nblk - st);
    if (st > 0) __syncthreads();
    {
      const int chunks = st_blocks * 16;  // 16-byte chunks per activation row in this stage
      const uint16_t *xsrc = p.x + static_cast<size_t>(m0) * p.K + static_cast<size_t>(kb_lo + st) * 128;
      for (int idx = threadIdx.x; idx < mvalid * chunks; idx += blockDim.x) {
        const int m = idx / chunks, c = idx - m * chunks;
        const uint4 v = *reinterpret_cast<const uint4 *>(xsrc + static_cast<size_t>(m) * p.K + c * 8);
        *reinterpret_cast<uint4 *>(xs + m * xstride + c * 8) = v;
      }
    }
    __syncthreads();
    if (!active) continue;

    for (int i0 = st; i0 < st + st_blocks; i0 += D) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const int i = i0 + d;
        if (i < nblk) {
          float acc[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint32_t a_lo[4], a_hi[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              a_lo[q] = decode_pair<B>(wbuf[d], 8 * jj + q);
              a_hi[q] = decode_pair<B>(wbuf[d], 8 * jj + 4 + q);
              if constexpr (BF16) {
                a_lo[q] = h2_to_bf2(a_lo[q]);
                a_hi[q] = h2_to_bf2(a_hi[q]);
              }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint4 xb = make_uint4(0u, 0u, 0u, 0u);
              if (nt * 8 + g < mvalid)
                xb = *reinterpret_cast<const uint4 *>(xs + (nt * 8 + g) * xstride + (i - st) * 128 + 32 * jj + 8 * t);
              if constexpr (GS == -1) {
                mma16816<BF16>(yacc[nt], a_lo, xb.x, xb.y);
                mma16816<BF16>(yacc[nt], a_hi, xb.z, xb.w);
              } else {
                mma16816<BF16>(acc[nt], a_lo, xb.x, xb.y);
                mma16816<BF16>(acc[nt], a_hi, xb.z, xb.w);
              }
            }
            if constexpr (GS == 32) {
              const float slo = scale_to_float<BF16>(sbuf[d].lo[jj]);
              const float shi = scale_to_float<BF16>(sbuf[d].hi[jj]);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                yacc[nt][0] = fmaf(slo, acc[nt][0], yacc[nt][0]);
                yacc[nt][1] = fmaf(slo, acc[nt][1], yacc[nt][1]);
                yacc[nt][2] = fmaf(shi, acc[nt][2], yacc[nt][2]);
                yacc[nt][3] = fmaf(shi, acc[nt][3], yacc[nt][3]);
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
              }
            }
          }
          if constexpr (GS == 128) {
            const float slo = scale_to_float<BF16>(sbuf[d].lo[0]);
            const float shi = scale_to_float<BF16>(sbuf[d].hi[0]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              yacc[nt][0] = fmaf(slo, acc[nt][0], yacc[nt][0]);
              yacc[nt][1] = fmaf(slo, acc[nt][1], yacc[nt][1]);
              yacc[nt][2] = fmaf(shi, acc[nt][2], yacc[nt][2]);
              yacc[nt][3] = fmaf(shi, acc[nt][3], yacc[nt][3]);
            }
          }
          if (i + D < nblk) {
            load_block<B>(wbase + static_cast<size_t>(i + D) * BW, lane, wbuf[d]);
            load_scales<GS>(p.s, tile, kb_lo + i + D, groups, lane, sbuf[d]);
          }
        }
      }
    }
  }

  if (active) {
    // 2^(8-b) (exact) and, for one scale per row, the row scale, both in fp32
    // (csrc/matgptq_gemm.cu:615-633, 943-949).
    float mlo = static_cast<float>(1 << (8 - B)), mhi = mlo;
    if constexpr (GS == -1) {
      mlo *= scale_to_float<BF16>(ldg_u16(p.s + static_cast<size_t>(tile) * 16 + g));
      mhi *= scale_to_float<BF16>(ldg_u16(p.s + static_cast<size_t>(tile) * 16 + g + 8));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[(nt * 8 + 2 * t + 0) * rstride + warp * 16 + g] = yacc[nt][0] * mlo;
      red[(nt * 8 + 2 * t + 1) * rstride + warp * 16 + g] = yacc[nt][1] * mlo;
      red[(nt * 8 + 2 * t + 0) * rstride + warp * 16 + g + 8] = yacc[nt][2] * mhi;
      red[(nt * 8 + 2 * t + 1) * rstride + warp * 16 + g + 8] = yacc[nt][3] * mhi;
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[(nt * 8 + 2 * t + 0) * rstride + warp * 16 + g] = 0.f;
      red[(nt * 8 + 2 * t + 1) * rstride + warp * 16 + g] = 0.f;
      red[(nt * 8 + 2 * t + 0) * rstride + warp * 16 + g + 8] = 0.f;
      red[(nt * 8 + 2 * t + 1) * rstride + warp * 16 + g + 8] = 0.f;
    }
  }

  const int cols = R * 16;
  const int n0 = rg * cols;
  const int outputs = mvalid * cols;
  if (S == 1) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < outputs; idx += blockDim.x) {
      const int m = idx / cols, n = idx - m * cols;
      if (n0 + n < p.N) p.y[static_cast<size_t>(m0 + m) * p.N + n0 + n] = float_to_out<BF16>(red[m * rstride + n]);
    }
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int lo = static_cast<int>(static_cast<long long>(crank) * outputs / S);
    const int hi = static_cast<int>(static_cast<long long>(crank + 1) * outputs / S);
    for (int idx = lo + threadIdx.x; idx < hi; idx += blockDim.x) {
      const int m = idx / cols, n = idx - m * cols;
      float sum = 0.f;
      for (int r = 0; r < S; ++r) sum += *cluster.map_shared_rank(red + m * rstride + n, r);
      if (n0 + n < p.N) p.y[static_cast<size_t>(m0 + m) * p.N + n0 + n] = float_to_out<BF16>(sum);
    }
    cluster.sync();  // peers may still be reading this CTA's partial sums
  }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
template <int B> struct Depth {
  static constexpr int value = (B == 2) ? 8 : (B == 3) ? 5 : (B == 4) ? 4 : (B == 6) ? 3 : 2;
};

static int g_sm_count = 0;

template <int B, int GS, bool BF16, int NT>
static int launch_gemv(const GemvParams &p, int R, cudaStream_t stream, bool pdl) {
  constexpr int D = Depth<B>::value;
  auto kernel = gemv_kernel<B, GS, BF16, NT, D>;
  const int S = p.split;
  const int max_nblk = (p.kblocks + S - 1) / S;
  constexpr int XB = D * ((16 + D - 1) / D);
  const int stage_blocks = max_nblk < XB ? max_nblk : XB;
  const size_t smem = static_cast<size_t>(NT * 8) * (stage_blocks * 128 + 32) * 2 + static_cast<size_t>(NT * 8) * (R * 16 + 4) * 4;
  if (smem > 48 * 1024) {
    // at most NT*8 = 16 rows x (20 blocks x 256 B + 64 B) + partial sums < 96 KiB: opt in once per device
    static bool opted_in[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
    if (dev < 0 || dev >= 64) return MG_ERR_BAD_ARG;
    if (!opted_in[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      if (e != cudaSuccess) return MG_ERR_CUDA;
      opted_in[dev] = true;
    }
  }
  const int row_groups = (p.tiles + R - 1) / R;
  const int passes = (p.M + NT * 8 - 1) / (NT * 8);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(row_groups * S, passes, 1);
  cfg.blockDim = dim3(R * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (S > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = S;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  return e == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <int B, int GS, bool BF16>
static int launch_gemv_nt(const GemvParams &p, int R, cudaStream_t stream, bool pdl) {
  if (p.M <= 8) return launch_gemv<B, GS, BF16, 1>(p, R, stream, pdl);
  return launch_gemv<B, GS, BF16, 2>(p, R, stream, pdl);
}

template <int B, int GS>
static int launch_gemv_type(const GemvParams &p, int R, bool bf16, cudaStream_t stream, bool pdl) {
  if (bf16) return launch_gemv_nt<B, GS, true>(p, R, stream, pdl);
  return launch_gemv_nt<B, GS, false>(p, R, stream, pdl);
}

template <int B>
static int launch_gemv_group(const GemvParams &p, int R, int group_size, bool bf16, cudaStream_t stream, bool pdl) {
  switch (group_size) {
    case -1: return launch_gemv_type<B, -1>(p, R, bf16, stream, pdl);
    case 32: return launch_gemv_type<B, 32>(p, R, bf16, stream, pdl);
    case 128: return launch_gemv_type<B, 128>(p, R, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

// Pick warps per CTA (R) and CTAs per cluster along K (S): enough CTAs to cover
// every SM a few times over, a K slice of at least two blocks per warp where the
// shape allows, and R as large as that permits so that the staged activations
// are reused by many row tiles.
void gemv_pick_config(int tiles, int kblocks, int sm_count, int *R_out, int *S_out) {
  const int want = 2 * sm_count;
  int bestR = 8, bestS = 1;
  long long best_score = -1;
  for (int R = 8; R >= 2; R >>= 1) {
    for (int S = 1; S <= 8; S <<= 1) {
      if (S > kblocks) break;
      const int per_warp = kblocks / S;
      if (S > 1 && per_warp < 2) break;
      const long long ctas = static_cast<long long>((tiles + R - 1) / R) * S;
      const long long filled = ctas >= want ? want : ctas;
      // prefer filling the machine, then larger R, then smaller S
      const long long score = filled * 1000 + R * 10 - S;
      if (score > best_score) {
        best_score = score;
        bestR = R;
        bestS = S;
      }
    }
  }
  *R_out = bestR;
  *S_out = bestS;
}

int gemv_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                void *y, bool bf16, bool pdl, int R_override, int S_override, cudaStream_t stream) {
  if (g_sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
    if (cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MG_ERR_CUDA;
  }
  GemvParams p;
  p.w = static_cast<const uint32_t *>(w);
  p.s = static_cast<const uint16_t *>(s);
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.N = N;
  p.K = K;
  p.M = M;
  p.tiles = N / 16;
  p.kblocks = K / 128;
  int R, S;
  gemv_pick_config(p.tiles, p.kblocks, g_sm_count, &R, &S);
  if (R_override > 0) R = R_override;
  if (S_override > 0) S = S_override;
  if (R < 1 || R > 8 || S < 1 || S > 8 || (S & (S - 1)) != 0 || S > p.kblocks) return MG_ERR_BAD_ARG;
  p.split = S;
  switch (bitwidth) {
    case 2: return launch_gemv_group<2>(p, R, group_size, bf16, stream, pdl);
    case 3: return launch_gemv_group<3>(p, R, group_size, bf16, stream, pdl);
    case 4: return launch_gemv_group<4>(p, R, group_size, bf16, stream, pdl);
    case 6: return launch_gemv_group<6>(p, R, group_size, bf16, stream, pdl);
    case 8: return launch_gemv_group<8>(p, R, group_size, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

}  // namespace mg
