// Persistent "stream-K" GEMV for the smallest batches (1..4 activation rows).
//
// Same arithmetic as gemv.cu (and the same reference code it replaces,
// csrc/matgptq_gemm.cu:636-953), different work distribution.  The cluster kernel gives
// every CTA a fixed (row tiles x K slice) rectangle, so the number of CTAs rarely divides
// the SMs evenly and each CTA pays its own set-up, activation copy and reduction.  Here
//   * one CTA per SM stays resident with 24-32 warps; the blocks of the whole matrix
//     (row-tile major, so a warp's share is ONE contiguous byte range of packed weights
//     and of scales) are dealt out evenly over all warps of the grid, whatever the shape;
//   * each warp streams its range through its ring of bulk-copy stages without ever
//     draining it at a tile boundary; a tile's partial sum is parked in shared memory
//     when the range crosses into the next tile;
//   * the whole activation matrix (M <= 4 rows) and its per-group row sums are staged
//     once per CTA;
//   * partial sums of a tile are added in warp order inside the CTA; a tile that spans
//     CTAs is finished by the CTA that owns its end: the earlier CTAs publish their part
//     in global scratch behind a flag (a per-launch epoch value, cleared again by its one
//     consumer), the finisher adds the parts in CTA order.  Waits go from higher to lower
//     CTA indices only and are bounded.
// Results do not depend on scheduling: every sum has a fixed order.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "async.cuh"
#include "decode.cuh"
#include "gemv_common.cuh"
#include "kernels.h"

namespace mg {

constexpr int kStreamMaxRows = 4;   // activation rows the kernel takes
constexpr int kStreamMaxSegs = 3;   // tiles a warp's range may touch
constexpr int kStatusFixupTimeout = 104;

struct StreamParams {
  const unsigned char *w;
  const unsigned char *s;
  const uint16_t *x;
  uint16_t *y;
  float *fix;                  // [ctas][16 * kStreamMaxRows]: each CTA's part of the tile that continues in the next CTA
  unsigned long long *flags;   // [ctas]: == epoch once that part is published
  unsigned long long epoch;
  int N, K, M, tiles, kblocks;
  long long total;             // tiles * kblocks
};

template <int B> struct StreamCfg {
  static constexpr int CB = (B == 2) ? 4 : (B <= 4) ? 2 : 1;  // blocks per ring stage (1.5 to 2 KB)
  static constexpr int NS = 3;                               // ring stages per warp
  static constexpr int WARPS = 24;                           // warps per CTA
};

struct StreamPlan {
  int xstride_h, stage_bytes, scale_bytes_per_block, sums_per_block;
  int off_bars, off_meta, off_x, off_sums, off_slots, off_ring, total;
};

template <int B, int GS> __host__ __device__ inline StreamPlan stream_plan(int W, int M, int K) {
  StreamPlan p;
  const int kblocks = K / 128;
  p.xstride_h = K + 32;  // halves; +64 bytes keeps 16-byte fragment reads conflict free
  p.scale_bytes_per_block = (GS == -1) ? 0 : (GS == 32 ? 128 : 32);
  p.stage_bytes = StreamCfg<B>::CB * (BlockTraits<B>::WORDS * 4 + p.scale_bytes_per_block);
  p.sums_per_block = ((GS == 32) ? 4 : 1) * 8;
  p.off_bars = 0;
  p.off_meta = 128 * ((8 * (W * StreamCfg<B>::NS + 1) + 127) / 128);  // first tile and segment count per warp
  p.off_x = p.off_meta + 128 * ((W * 8 + 127) / 128);
  p.off_sums = p.off_x + 128 * ((M * p.xstride_h * 2 + 127) / 128);
  p.off_slots = p.off_sums + 128 * ((kblocks * p.sums_per_block * 4 + 127) / 128);
  p.off_ring = p.off_slots + 128 * ((W * kStreamMaxSegs * 16 * M * 4 + 127) / 128);
  p.total = p.off_ring + W * StreamCfg<B>::NS * p.stage_bytes;
  return p;
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <int B, int GS, bool BF16>
__global__ void __launch_bounds__(768, 1) gemv_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int CB = StreamCfg<B>::CB, NS = StreamCfg<B>::NS;
  constexpr int WBYTES = BlockTraits<B>::WORDS * 4;
  constexpr int NCH = Chains<B>::N;
  constexpr float kNegZero = -static_cast<float>(BlockTraits<B>::ZERO) * 5.9604644775390625e-08f;  // -Z * 2^-24

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int M = p.M, kblocks = p.kblocks;
  const StreamPlan plan = stream_plan<B, GS>(W, M, p.K);
  const int SCB = plan.scale_bytes_per_block;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bar_ring = smem_base + plan.off_bars + warp * NS * 8;
  const uint32_t bar_x = smem_base + plan.off_bars + W * NS * 8;
  int *meta = reinterpret_cast<int *>(smem_raw + plan.off_meta);  // [W][2]
  uint16_t *xs = reinterpret_cast<uint16_t *>(smem_raw + plan.off_x);
  float *sums = reinterpret_cast<float *>(smem_raw + plan.off_sums);
  float *slots = reinterpret_cast<float *>(smem_raw + plan.off_slots);
  const unsigned char *ring = smem_raw + plan.off_ring + warp * NS * plan.stage_bytes;
  const uint32_t ring_u32 = smem_base + plan.off_ring + warp * NS * plan.stage_bytes;
  const int xstride = plan.xstride_h;

  // this warp's share of the blocks, and this CTA's
  const long long G = static_cast<long long>(gridDim.x) * W;
  const long long gw = static_cast<long long>(blockIdx.x) * W + warp;
  const long long lo = gw * p.total / G, hi = (gw + 1) * p.total / G;
  const int cnt = static_cast<int>(hi - lo);
  const long long clo = static_cast<long long>(blockIdx.x) * W * p.total / G;
  const long long chi = (static_cast<long long>(blockIdx.x) + 1) * W * p.total / G;

  if (lane == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(bar_ring + i * 8, 1);
    if (warp == 0) mbar_init(bar_x, 1);
    mbar_init_fence();
  }
  __syncthreads();

  const int nchunks = (cnt + CB - 1) / CB;
  auto issue_chunk = [&](int c) {
    const int nb = min(CB, cnt - c * CB);
    const int st = c % NS;
    const uint32_t bar = bar_ring + st * 8;
    const uint32_t dst = ring_u32 + st * plan.stage_bytes;
    mbar_arrive_expect_tx(bar, nb * (WBYTES + SCB));
    bulk_copy_g2s(dst, p.w + (lo + static_cast<long long>(c) * CB) * WBYTES, nb * WBYTES, bar);
    if (GS != -1) bulk_copy_g2s(dst + CB * WBYTES, p.s + (lo + static_cast<long long>(c) * CB) * SCB, nb * SCB, bar);
  };
  if (lane == 0) {
    for (int c = 0; c < NS && c < nchunks; ++c) issue_chunk(c);
  }

  // Everything above reads only weights and scales, which no kernel writes.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_x, M * p.K * 2);
    for (int m = 0; m < M; ++m)
      bulk_copy_g2s(smem_base + plan.off_x + m * xstride * 2, p.x + static_cast<size_t>(m) * p.K, p.K * 2, bar_x);
  }
  bool failed = false;
  if (!mbar_wait(bar_x, 0)) {
    failed = true;
    report_status(kStatusActivationCopyTimeout);
  }
  if constexpr (BF16) {
    // bf16 activations become fp16 in place (saturating at +-65504)
    const int chunks_per_row = p.K / 8;
    for (int ci = threadIdx.x; ci < M * chunks_per_row; ci += blockDim.x) {
      const int m = ci / chunks_per_row, cc = ci - m * chunks_per_row;
      uint4 *ptr = reinterpret_cast<uint4 *>(xs + m * xstride + cc * 8);
      uint4 v = *ptr;
      uint32_t *vw = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = __uint_as_float(vw[e] << 16), b = __uint_as_float(vw[e] & 0xFFFF0000u);
        a = fminf(fmaxf(a, -65504.f), 65504.f);
        b = fminf(fmaxf(b, -65504.f), 65504.f);
        vw[e] = h2_bits(__floats2half2_rn(a, b));
      }
      *ptr = v;
    }
    __syncthreads();
  }
  // row sums of the activations per group, times -Z*2^-24 (the zero-point term), via an all-ones A fragment
  for (int blk = warp; blk < kblocks; blk += W) {
    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
    const int xrow = min(g, M - 1);
    float sacc[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint4 xv = *reinterpret_cast<const uint4 *>(xs + xrow * xstride + blk * 128 + 32 * jj + 8 * t);
      if (GS == 32 || jj == 0)
        mma16816<true>(sacc, ones, xv.x, xv.y);
      else
        mma16816<false>(sacc, ones, xv.x, xv.y);
      mma16816<false>(sacc, ones, xv.z, xv.w);
      if (GS == 32 && g == 0)
        *reinterpret_cast<float2 *>(sums + blk * plan.sums_per_block + jj * 8 + 2 * t) = make_float2(kNegZero * sacc[0], kNegZero * sacc[1]);
    }
    if (GS != 32 && g == 0)
      *reinterpret_cast<float2 *>(sums + blk * plan.sums_per_block + 2 * t) = make_float2(kNegZero * sacc[0], kNegZero * sacc[1]);
  }
  __syncthreads();

  // ---------------------------------------------------------------- stream this warp's range
  int tile = static_cast<int>(lo / kblocks);
  int kb = static_cast<int>(lo - static_cast<long long>(tile) * kblocks);
  const int first_tile = tile;
  int seg = 0;
  float yacc[4] = {0.f, 0.f, 0.f, 0.f};
  const int xrow = min(g, M - 1);
  const float out_scale = static_cast<float>(1 << (8 - B)) * 16777216.f;  // 2^(8-b) and the subnormal scale 2^24

  auto park_segment = [&]() {
    float mlo = out_scale, mhi = out_scale;
    if constexpr (GS == -1) {
      const uint16_t *sp = reinterpret_cast<const uint16_t *>(p.s) + static_cast<size_t>(tile) * 16;
      mlo *= scale_to_float<BF16>(__ldg(sp + g));
      mhi *= scale_to_float<BF16>(__ldg(sp + g + 8));
    }
    float *slot = slots + (warp * kStreamMaxSegs + seg) * 16 * M;
    if (2 * t < M) {
      slot[g * M + 2 * t] = yacc[0] * mlo;
      slot[(g + 8) * M + 2 * t] = yacc[2] * mhi;
    }
    if (2 * t + 1 < M) {
      slot[g * M + 2 * t + 1] = yacc[1] * mlo;
      slot[(g + 8) * M + 2 * t + 1] = yacc[3] * mhi;
    }
    yacc[0] = yacc[1] = yacc[2] = yacc[3] = 0.f;
    ++seg;
  };

  int done = 0;
  for (int c = 0; c < nchunks && !failed; ++c) {
    const int st = c % NS;
    if (!mbar_wait(bar_ring + st * 8, (c / NS) & 1)) {
      failed = true;
      report_status(kStatusWeightCopyTimeout);
      break;
    }
    const unsigned char *stage = ring + st * plan.stage_bytes;
    const int nb = min(CB, cnt - c * CB);
#pragma unroll
    for (int cb = 0; cb < CB; ++cb) {
      if (cb >= nb) break;
      uint32_t w[2 * B];
      {
        const uint32_t *blk = reinterpret_cast<const uint32_t *>(stage + cb * WBYTES);
#pragma unroll
        for (int v = 0; v < BlockTraits<B>::NV; ++v) {
          const uint4 q = *reinterpret_cast<const uint4 *>(blk + v * 128 + lane * 4);
          w[4 * v + 0] = q.x;
          w[4 * v + 1] = q.y;
          w[4 * v + 2] = q.z;
          w[4 * v + 3] = q.w;
        }
        if constexpr (BlockTraits<B>::TAIL == 2) {
          const uint2 q = *reinterpret_cast<const uint2 *>(blk + BlockTraits<B>::NV * 128 + lane * 2);
          w[4 * BlockTraits<B>::NV + 0] = q.x;
          w[4 * BlockTraits<B>::NV + 1] = q.y;
        }
      }
      const uint16_t *sblk = reinterpret_cast<const uint16_t *>(stage + CB * WBYTES + cb * SCB);
      const float *bsum = sums + kb * plan.sums_per_block;
      uint4 xb[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        xb[jj] = *reinterpret_cast<const uint4 *>(xs + xrow * xstride + kb * 128 + 32 * jj + 8 * t);

      if constexpr (GS == 32) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          float d0[4], d1[4];
          uint32_t a0[4], a1[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            a0[q] = field_pair<B>(w, 8 * jj + q, 0u);
            a1[q] = field_pair<B>(w, 8 * jj + 4 + q, 0u);
          }
          const float f0 = 1.f / static_cast<float>(1 << kstep_offset<B>(2 * jj));
          const float f1 = 1.f / static_cast<float>(1 << kstep_offset<B>(2 * jj + 1));
          const float slo = scale_to_float<BF16>(sblk[jj * 16 + g]);
          const float shi = scale_to_float<BF16>(sblk[jj * 16 + g + 8]);
          mma16816<true>(d0, a0, xb[jj].x, xb[jj].y);
          mma16816<true>(d1, a1, xb[jj].z, xb[jj].w);
          const float2 zs = *reinterpret_cast<const float2 *>(bsum + jj * 8 + 2 * t);
          yacc[0] = fmaf(slo, fmaf(d1[0], f1, fmaf(d0[0], f0, zs.x)), yacc[0]);
          yacc[1] = fmaf(slo, fmaf(d1[1], f1, fmaf(d0[1], f0, zs.y)), yacc[1]);
          yacc[2] = fmaf(shi, fmaf(d1[2], f1, fmaf(d0[2], f0, zs.x)), yacc[2]);
          yacc[3] = fmaf(shi, fmaf(d1[3], f1, fmaf(d0[3], f0, zs.y)), yacc[3]);
        }
      } else {
        float acc[NCH][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t a[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) a[q] = field_pair<B>(w, 4 * i + q, 0u);
          const uint32_t b0 = (i & 1) ? xb[i >> 1].z : xb[i >> 1].x;
          const uint32_t b1 = (i & 1) ? xb[i >> 1].w : xb[i >> 1].y;
          if (Chains<B>::first(i))
            mma16816<true>(acc[Chains<B>::of(i)], a, b0, b1);
          else
            mma16816<false>(acc[Chains<B>::of(i)], a, b0, b1);
        }
        float slo = 1.f, shi = 1.f;
        if constexpr (GS == 128) {
          slo = scale_to_float<BF16>(sblk[g]);
          shi = scale_to_float<BF16>(sblk[g + 8]);
        }
        const float2 zs = *reinterpret_cast<const float2 *>(bsum + 2 * t);
        float tsum[4] = {zs.x, zs.y, zs.x, zs.y};
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
          for (int e = 0; e < 4; ++e) tsum[e] = fmaf(acc[ch][e], Chains<B>::inv_factor(ch), tsum[e]);
        yacc[0] = fmaf(slo, tsum[0], yacc[0]);
        yacc[1] = fmaf(slo, tsum[1], yacc[1]);
        yacc[2] = fmaf(shi, tsum[2], yacc[2]);
        yacc[3] = fmaf(shi, tsum[3], yacc[3]);
      }
      ++done;
      if (kb == kblocks - 1 || done == cnt) park_segment();  // end of a tile, or of this warp's range
      if (++kb == kblocks) {
        kb = 0;
        ++tile;
      }
    }
    __syncwarp();  // the stage has been read into registers by every lane: refill it
    if (lane == 0 && c + NS < nchunks) issue_chunk(c + NS);
  }
  if (lane == 0) {
    meta[2 * warp] = first_tile;
    meta[2 * warp + 1] = failed ? 0 : seg;
  }
  __syncthreads();

  // ---------------------------------------------------------------- add the parts of every tile of this CTA
  const int t_first = static_cast<int>(clo / kblocks), t_last = static_cast<int>((chi - 1) / kblocks);
  const bool head_shared = (clo % kblocks) != 0;                    // the first tile began in an earlier CTA
  const bool tail_shared = (chi % kblocks) != 0;                    // the last tile continues in a later CTA
  const int per_tile = 16 * M;
  const int outputs = (t_last - t_first + 1) * per_tile;
  for (int o = threadIdx.x; o < outputs; o += blockDim.x) {
    const int T = t_first + o / per_tile, rem = o % per_tile, row = rem / M, col = rem % M;
    float sum = 0.f;
    for (int w2 = 0; w2 < W; ++w2) {
      const int d = T - meta[2 * w2];
      if (d >= 0 && d < meta[2 * w2 + 1]) sum += slots[(w2 * kStreamMaxSegs + d) * per_tile + rem];
    }
    const bool is_tail = (T == t_last) && tail_shared;
    const bool is_head = (T == t_first) && head_shared;
    if (is_tail) {
      p.fix[static_cast<size_t>(blockIdx.x) * 16 * kStreamMaxRows + rem] = sum;  // finished by a later CTA
    } else if (is_head) {
      slots[rem] = sum;  // finished below, once the earlier CTAs' parts are in (slot 0 of warp 0 is no longer needed)
    } else {
      const int n = T * 16 + row;
      p.y[static_cast<size_t>(col) * p.N + n] = float_to_out<BF16>(sum);
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0 && tail_shared) st_release_u64(p.flags + blockIdx.x, p.epoch);

  if (head_shared && !((t_first == t_last) && tail_shared)) {
    // this CTA owns the end of its first tile: add the parts of the CTAs before it, in CTA order.
    // c_first: the CTA whose range contains the tile's first block.
    const long long tile_start = static_cast<long long>(t_first) * kblocks;
    int c_first = blockIdx.x - 1;
    while (c_first > 0 && static_cast<long long>(c_first) * W * p.total / G > tile_start) --c_first;
    for (int o = threadIdx.x; o < per_tile; o += blockDim.x) {
      float sum = 0.f;
      bool ok = true;
      for (int cc = c_first; cc < static_cast<int>(blockIdx.x) && ok; ++cc) {
        uint32_t polls = 0;
        while (ld_acquire_u64(p.flags + cc) != p.epoch) {
          if (++polls > (1u << 22)) {
            ok = false;
            report_status(kStatusFixupTimeout);
            break;
          }
          __nanosleep(32);
        }
        if (ok) sum += __ldcg(p.fix + static_cast<size_t>(cc) * 16 * kStreamMaxRows + o);
      }
      sum += slots[o];
      const int row = o / M, col = o % M;
      p.y[static_cast<size_t>(col) * p.N + t_first * 16 + row] = float_to_out<BF16>(sum);
    }
    // Every flag has exactly one consumer (this CTA): clear them, so that a replay of this very launch
    // from a CUDA graph (same epoch) starts clean.  The next launch publishes only after this grid is done.
    __syncthreads();
    for (int cc = c_first + threadIdx.x; cc < static_cast<int>(blockIdx.x); cc += blockDim.x) p.flags[cc] = 0ull;
  }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static std::atomic<unsigned long long> g_stream_epoch{1};

long long gemv_stream_workspace_bytes(int sm_count) {
  // per CTA: 16 * kStreamMaxRows floats of partial sums, one 64-bit flag; flags first, 256-byte aligned parts
  const long long flags = 256 * ((static_cast<long long>(sm_count) * 8 + 255) / 256);
  return flags + static_cast<long long>(sm_count) * 16 * kStreamMaxRows * 4;
}

template <int B, int GS, bool BF16>
static int launch_stream(StreamParams p, int sm_count, void *workspace, cudaStream_t stream, bool pdl) {
  constexpr int W = StreamCfg<B>::WARPS;
  auto kernel = gemv_stream_kernel<B, GS, BF16>;
  const StreamPlan plan = stream_plan<B, GS>(W, p.M, p.K);
  if (plan.total > 224 * 1024) return MG_ERR_UNSUPPORTED;  // activations of this shape do not fit beside the rings
  int ctas = static_cast<int>(p.total / W);
  if (ctas > sm_count) ctas = sm_count;
  if (ctas < 1) ctas = 1;
  const long long G = static_cast<long long>(ctas) * W;
  if ((p.total + G - 1) / G > 2LL * p.kblocks) return MG_ERR_UNSUPPORTED;  // a warp's range may touch three tiles at most
  static bool opted_in[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
  if (dev < 0 || dev >= 64) return MG_ERR_BAD_ARG;
  if (!opted_in[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) != cudaSuccess) return MG_ERR_CUDA;
    opted_in[dev] = true;
  }
  const long long flag_bytes = 256 * ((static_cast<long long>(sm_count) * 8 + 255) / 256);
  p.flags = static_cast<unsigned long long *>(workspace);
  p.fix = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + flag_bytes);
  p.epoch = 0xA5C3000000000000ull | (g_stream_epoch.fetch_add(1) & 0xFFFFFFFFFFFFull);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, 1, 1);
  cfg.blockDim = dim3(W * 32, 1, 1);
  cfg.dynamicSmemBytes = plan.total;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kernel, p) == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <int B, int GS>
static int launch_stream_type(const StreamParams &p, int sm_count, void *ws, bool bf16, cudaStream_t stream, bool pdl) {
  if (bf16) return launch_stream<B, GS, true>(p, sm_count, ws, stream, pdl);
  return launch_stream<B, GS, false>(p, sm_count, ws, stream, pdl);
}

template <int B>
static int launch_stream_group(const StreamParams &p, int sm_count, void *ws, int group_size, bool bf16, cudaStream_t stream, bool pdl) {
  switch (group_size) {
    case -1: return launch_stream_type<B, -1>(p, sm_count, ws, bf16, stream, pdl);
    case 32: return launch_stream_type<B, 32>(p, sm_count, ws, bf16, stream, pdl);
    case 128: return launch_stream_type<B, 128>(p, sm_count, ws, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

// Returns MG_ERR_UNSUPPORTED (and launches nothing) for shapes this kernel does not take; the caller
// then uses the cluster kernel.  workspace: gemv_stream_workspace_bytes() bytes, contents arbitrary.
int gemv_stream_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                       void *y, void *workspace, long long workspace_bytes, bool bf16, bool pdl, cudaStream_t stream) {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MG_ERR_CUDA;
  }
  if (M < 1 || M > kStreamMaxRows) return MG_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < gemv_stream_workspace_bytes(sm_count)) return MG_ERR_UNSUPPORTED;
  StreamParams p;
  p.w = static_cast<const unsigned char *>(w);
  p.s = static_cast<const unsigned char *>(s);
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.fix = nullptr;
  p.flags = nullptr;
  p.epoch = 0;
  p.N = N;
  p.K = K;
  p.M = M;
  p.tiles = N / 16;
  p.kblocks = K / 128;
  p.total = static_cast<long long>(p.tiles) * p.kblocks;
  switch (bitwidth) {
    case 2: return launch_stream_group<2>(p, sm_count, workspace, group_size, bf16, stream, pdl);
    case 3: return launch_stream_group<3>(p, sm_count, workspace, group_size, bf16, stream, pdl);
    case 4: return launch_stream_group<4>(p, sm_count, workspace, group_size, bf16, stream, pdl);
    case 6: return launch_stream_group<6>(p, sm_count, workspace, group_size, bf16, stream, pdl);
    case 8: return launch_stream_group<8>(p, sm_count, workspace, group_size, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

MG_DEFINE_STATUS_ACCESSOR(gemv_stream_device_status)

}  // namespace mg
