// Bit-sliced GEMV family for small batches (1..16 activation rows per pass).
//
// Replaces gptq_matryoshka_simt / gptq_matryoshka and their dispatch
// (csrc/matgptq_gemm.cu:337-953, 955-1065).  y[M,N] = x[M,K] . Wdq^T with
// Wdq[n,k] = (q[n,k] - 2^(b-1)) * s[n, k/g] * 2^(8-b), fp32 accumulation.
//
// Shape of the computation
//   * one warp streams 16 out-features x a K slice.  Lane 0 moves the slice with
//     bulk asynchronous copies (cp.async.bulk, the untiled TMA path) into a ring of
//     shared-memory stages guarded by mbarriers, a few KB ahead of the math, so the
//     bytes in flight do not depend on registers or occupancy;
//   * per block (16 x 128 codes) a lane reads its words with 16-byte shared loads,
//     decodes its 64 codes in registers straight into mma.m16n8k16 A fragments
//     (exact integers), multiplies them with the activation fragments on the
//     tensor pipe into a per-group fp32 accumulator and folds the group's scale in
//     fp32 (one FMA per accumulator and group);
//   * the R warps of a CTA are Rt consecutive row tiles x RK slices of the CTA's K range
//     and share the activations staged in shared memory: the CTA's whole K slice in one
//     piece when it fits (no barrier inside the loop), else double-buffered stages;
//   * K is split over the S CTAs of a thread-block cluster (split-K for skinny
//     shapes); every CTA stores its partial sums into the shared memory of the CTA
//     that owns the columns (distributed shared memory), which adds them in a fixed
//     order after one cluster barrier, so results do not depend on scheduling and no
//     global scratch or atomics are used;
//   * the weight copies of the first stages are issued before griddepcontrol.wait,
//     so with programmatic dependent launch they overlap the previous kernel's tail;
//   * every mbarrier wait is bounded (async.cuh): on a timeout the kernel records a
//     status word and finishes.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "async.cuh"
#include "decode.cuh"
#include "gemv_common.cuh"
#include "host_util.h"
#include "kernels.h"

namespace cg = cooperative_groups;

// This file is compiled twice: as it is (implicit zero point 2^(b-1), what the reference's operator computes)
// and from gemv_zp.cu with MG_GEMV_ZP = 1 (per-group zero points, an extension).  Everything that differs
// between the two carries kZP in its template arguments or its name, so the two objects link together.
#ifndef MG_GEMV_ZP
#define MG_GEMV_ZP 0
#endif

namespace mg {

constexpr bool kZP = MG_GEMV_ZP != 0;

struct GemvParams {
  const uint32_t *w;
  const uint16_t *s;
  const uint16_t *z;  // zero points in master units, laid out like the scales (only read when kZP)
  const uint16_t *x;
  uint16_t *y;
  int N, K, M;
  int ldy;      // elements between two rows of y (N unless the call writes a column block of a wider output)
  int tiles;    // N / 16
  int kblocks;  // K / 128
  int split;    // CTAs per cluster along K
  int stages;   // ring stages per warp
  int xblocks;  // blocks (128 in-features) per activation stage: a multiple of ChunkBlocks, or the whole K slice
  int kslices;  // warps of a CTA that share one row tile and split the CTA's K range (needs the whole slice staged)
};

// Blocks per ring stage (1.1 to 4.2 KB of packed weights and scales; the blocks of a stage are decoded
// without a wait or a refill between them).  The number of stages per warp is chosen by the host from
// the shared memory it wants the CTA to take.
template <int B, int NT> struct ChunkBlocks {
  // (two-block stages for two batch tiles were tried: the whole-slice staging then fits for down at b <= 4,
  // batch 16 (-14 %), but every other batch-16 cell loses 2-5 % to the extra waits; net zero)
  static constexpr int value = (B <= 4) ? 4 : 2;
};
// Shared-memory plan of one CTA, computed identically on host and device.
struct SmemPlan {
  int xrows, xstride_h, rstride, stage_bytes, scale_bytes_per_block, sums_per_block;
  int off_bars, off_x, off_sums, off_red, off_ring, total;
};

template <int B, int GS, int NT, bool ZP>
__host__ __device__ inline SmemPlan make_plan(int R, int M, int max_nblk, int stages, int xblocks) {
  SmemPlan p;
  p.xrows = M < NT * 8 ? M : NT * 8;
  const int xb = max_nblk < xblocks ? max_nblk : xblocks;
  const int xbufs = xblocks >= max_nblk ? 1 : 2;  // the whole K slice at once needs no second buffer
  p.xstride_h = xb * 128 + 32;  // halves; +64 bytes keeps 16-byte fragment reads conflict free
  p.rstride = R * 16 + 4;
  p.scale_bytes_per_block = (GS == -1) ? 0 : (GS == 32 ? 128 : 32);
  p.stage_bytes = ChunkBlocks<B, NT>::value * (BlockTraits<B>::WORDS * 4 + p.scale_bytes_per_block * (ZP ? 2 : 1));
  p.off_bars = 0;
  p.off_x = 128 * ((8 * (R * stages + 2) + 127) / 128);
  // per activation stage: for every block and group the sum of each activation row (fp32)
  p.sums_per_block = ((GS == 32) ? 4 : 1) * NT * 8;
  p.off_sums = p.off_x + xbufs * p.xrows * p.xstride_h * 2;
  p.off_red = p.off_sums + xbufs * xb * p.sums_per_block * 4;
  p.off_ring = 128 * ((p.off_red + NT * 8 * p.rstride * 4 + 127) / 128);
  p.total = p.off_ring + R * stages * p.stage_bytes;
  return p;
}

// B: bitwidth, GS: group size (-1, 32, 128), BF16: activation/scale/output type,
// NT: batch tiles of 8 rows handled per pass.
// The whole computation of one CTA; `block_x` is the CTA's index among the CTAs of this product (blockIdx.x for a
// plain launch, the index inside its segment for a grouped one).
// 8-byte accesses that are single transactions: a value and its flag travel and become visible together
__device__ __forceinline__ void st_volatile_v2(uint2 *ptr, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(ptr), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const uint2 *ptr) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
  return v;
}

template <int B, int GS, bool BF16, int NT, bool ZP, bool AR = false>
__device__ __forceinline__ void gemv_body(const GemvParams &p, const int block_x, const ArParams *ar = nullptr) {
  extern __shared__ __align__(128) unsigned char smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // the shuffle tells the compiler it is warp-uniform
  const int R = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int S = p.split;
  const int crank = (S > 1) ? static_cast<int>(cg::this_cluster().block_rank()) : 0;
  const int log2s = 31 - __clz(S);  // S is a power of two (checked by the host)
  const int rg = block_x >> log2s;
  // The CTA's warps form Rt row tiles x RK slices of the CTA's K range.
  const int RK = p.kslices;
  const int Rt = R / RK;
  const int kq = warp / Rt, tw = warp - kq * Rt;
  const int tile = rg * Rt + tw;
  const bool active = tile < p.tiles;
  const int kb_lo = (crank * p.kblocks) >> log2s;  // the CTA's K range, in blocks
  const int kb_hi = ((crank + 1) * p.kblocks) >> log2s;
  const int nblk_cta = kb_hi - kb_lo;
  const int w_lo = kq * nblk_cta / RK;  // this warp's part of it, relative to kb_lo
  const int nblk = (kq + 1) * nblk_cta / RK - w_lo;
  const int max_nblk = (p.kblocks + S - 1) >> log2s;
  const int m0 = blockIdx.y * (NT * 8);
  const int mvalid = min(p.M - m0, NT * 8);
  const int groups = (GS == -1) ? 1 : p.K / GS;

  constexpr int CB = ChunkBlocks<B, NT>::value;
  const int kStages = p.stages;
  const int kXBlocks = p.xblocks;
  constexpr int BW = BlockTraits<B>::WORDS;
  constexpr int WBYTES = BW * 4;  // packed bytes per block
  const SmemPlan plan = make_plan<B, GS, NT, kZP>(R, p.M, max_nblk, kStages, kXBlocks);
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bar_full0 = smem_base + plan.off_bars + warp * kStages * 8;  // this warp's ring barriers
  const uint32_t bar_x0 = smem_base + plan.off_bars + R * kStages * 8;        // two activation barriers
  float *red = reinterpret_cast<float *>(smem_raw + plan.off_red);
  const unsigned char *ring = smem_raw + plan.off_ring + warp * kStages * plan.stage_bytes;  // this warp's stages
  const uint32_t ring_u32 = smem_base + plan.off_ring + warp * kStages * plan.stage_bytes;
  const int xstride = plan.xstride_h;
  constexpr int SCB = (GS == -1) ? 0 : (GS == 32 ? 128 : 32);  // scale bytes per block
  constexpr int kStageBytes = CB * (WBYTES + SCB * (ZP ? 2 : 1));

  if (lane == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(bar_full0 + i * 8, 1);
    if (warp == 0) {
      mbar_init(bar_x0, 1);
      mbar_init(bar_x0 + 8, 1);
    }
    mbar_init_fence();
  }
  __syncthreads();
  // Tell the cluster that this CTA is running; the matching wait stands before the first store into a
  // peer's shared memory, long after every peer has arrived.
  if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  const int nchunks = (nblk + CB - 1) / CB;
  const unsigned char *wsrc = reinterpret_cast<const unsigned char *>(p.w) +
                              (static_cast<size_t>(active ? tile : 0) * p.kblocks + kb_lo + w_lo) * WBYTES;
  const unsigned char *ssrc = reinterpret_cast<const unsigned char *>(p.s) +
                              (static_cast<size_t>(active ? tile : 0) * groups) * 32 + static_cast<size_t>(kb_lo + w_lo) * SCB;

  const unsigned char *zsrc = reinterpret_cast<const unsigned char *>(p.z) +
                              (static_cast<size_t>(active ? tile : 0) * groups) * 32 + static_cast<size_t>(kb_lo + w_lo) * SCB;

  // Producer state (used by lane 0): the next chunk to request, as running pointers, so that a refill costs no
  // multiplications.  issue_next() fills the ring stage at byte offset `off` / barrier `bar` with that chunk.
  int issue_left = nblk;  // blocks not requested yet
  auto issue_next = [&](uint32_t off, uint32_t bar) {  // called by every lane; lane 0 issues the copies
    const int nb = min(CB, issue_left);
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, nb * (WBYTES + SCB * (ZP ? 2 : 1)));
      bulk_copy_g2s(ring_u32 + off, wsrc, nb * WBYTES, bar);
      if (GS != -1) bulk_copy_g2s(ring_u32 + off + CB * WBYTES, ssrc, nb * SCB, bar);
      if (GS != -1 && ZP) bulk_copy_g2s(ring_u32 + off + CB * (WBYTES + SCB), zsrc, nb * SCB, bar);
    }
    wsrc += CB * WBYTES;
    ssrc += CB * SCB;
    zsrc += CB * SCB;
    issue_left -= CB;
  };

  if (active) {
    for (int c = 0; c < kStages && c < nchunks; ++c) issue_next(c * kStageBytes, bar_full0 + c * 8);
  }

  // Everything above reads only weights and scales, which no kernel writes.  The
  // activations may come from the kernel launched just before this one.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int nxst = (nblk_cta + kXBlocks - 1) / kXBlocks;  // 1 whenever RK > 1
  // thread 0: copy the activations of x stage xi (rows m0.., blocks [xi*kXBlocks, ...)) into buffer xi & 1
  auto issue_x = [&](int xi) {
    const int nb = min(kXBlocks, nblk_cta - xi * kXBlocks);
    const uint32_t bar = bar_x0 + (xi & 1) * 8;
    const uint32_t dst = smem_base + plan.off_x + (xi & 1) * plan.xrows * xstride * 2;
    mbar_arrive_expect_tx(bar, mvalid * nb * 256);
    const uint16_t *src = p.x + static_cast<size_t>(m0) * p.K + static_cast<size_t>(kb_lo + xi * kXBlocks) * 128;
    for (int m = 0; m < mvalid; ++m) bulk_copy_g2s(dst + m * xstride * 2, src + static_cast<size_t>(m) * p.K, nb * 256, bar);
  };
  if (threadIdx.x == 0) {
    issue_x(0);
    if (nxst > 1) issue_x(1);
  }

  // y accumulates sum_g s_g * (sum_k code*x - Z*sum_k x) in units of 2^-24 (the subnormal scale)
  float yacc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) yacc[nt][e] = 0.f;

  constexpr int NCH = Chains<B>::N;
  // factor of the activation row sums: -Z * 2^-24 with the implicit zero point Z = 2^(b-1); with zero points
  // -2^-24, and the zero point of the row and group (in code units: master units / 2^(8-b)) multiplies later
  constexpr float kNegZero = -(ZP ? 1.f : static_cast<float>(BlockTraits<B>::ZERO)) * 5.9604644775390625e-08f;
  constexpr float kZeroToCode = 1.f / static_cast<float>(1 << (8 - B));
  float zrow_lo = 1.f, zrow_hi = 1.f;  // one zero point per row (GS == -1)
  if constexpr (ZP && GS == -1) {
    if (active) {
      zrow_lo = kZeroToCode * scale_to_float<BF16>(ldg_u16(p.z + static_cast<size_t>(tile) * 16 + g));
      zrow_hi = kZeroToCode * scale_to_float<BF16>(ldg_u16(p.z + static_cast<size_t>(tile) * 16 + g + 8));
    }
  }
  float *sums = reinterpret_cast<float *>(smem_raw + plan.off_sums);

  // Loop-invariant per-lane addresses: everything inside the block loop is base + running offset + constant.
  const unsigned char *w_lane = ring + lane * 16;                        // 16-byte vectors of the packed words
  const unsigned char *w_tail = ring + BlockTraits<B>::NV * 512 + lane * 8;  // the 8-byte tail (3-bit blocks)
  const unsigned char *s_lane = ring + CB * WBYTES + g * 2;              // scales of rows g and g+8
  const unsigned char *zp_lane = s_lane + CB * SCB;                      // their zero points (kZP)
  const uint16_t *x_lane[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    x_lane[nt] = reinterpret_cast<const uint16_t *>(smem_raw + plan.off_x) + min(nt * 8 + g, mvalid - 1) * xstride + 8 * t;
  const float *z_lane = sums + 2 * t;
  const int xbuf_halves = plan.xrows * xstride;
  constexpr int kSumsPerBlock = ((GS == 32) ? 4 : 1) * NT * 8;

  // Consumer state of the ring: stage byte offset, barrier and parity of the next chunk.
  uint32_t st_off = 0, st_bar = bar_full0, st_parity = 0;
  int left = nblk;  // blocks not consumed yet

  bool failed = false;
  for (int xi = 0; xi < nxst; ++xi) {
    if (!failed && !mbar_wait(bar_x0 + (xi & 1) * 8, (xi >> 1) & 1)) {
      failed = true;
      report_status(kStatusActivationCopyTimeout);
    }
    uint16_t *xbuf = reinterpret_cast<uint16_t *>(smem_raw + plan.off_x) + (xi & 1) * xbuf_halves;
    float *xsum = sums + (xi & 1) * kXBlocks * kSumsPerBlock;
    const int st_blocks = min(kXBlocks, nblk_cta - xi * kXBlocks);

    // bf16 activations become fp16 in place (saturating at +-65504): the type the tensor
    // pipe multiplies with the fp16 codes.
    if constexpr (BF16) {
      const int chunks_per_row = st_blocks * 16;  // 16-byte chunks
      for (int ci = threadIdx.x; ci < mvalid * chunks_per_row; ci += blockDim.x) {
        const int m = ci / chunks_per_row, cc = ci - m * chunks_per_row;
        uint4 *ptr = reinterpret_cast<uint4 *>(xbuf + m * xstride + cc * 8);
        uint4 v = *ptr;
        uint32_t *vw = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo = __uint_as_float(vw[e] << 16), hi = __uint_as_float(vw[e] & 0xFFFF0000u);
          lo = fminf(fmaxf(lo, -65504.f), 65504.f);
          hi = fminf(fmaxf(hi, -65504.f), 65504.f);
          vw[e] = h2_bits(__floats2half2_rn(lo, hi));
        }
        *ptr = v;
      }
      __syncthreads();
    }

    // Row sums of the activations per group, times -Z*2^-24: the zero-point term of every
    // output this CTA produces from this stage.  One warp per block multiplies the same B
    // fragments the main loop uses with an A fragment of ones, so the sums come out in the
    // accumulator layout (batch columns 2t, 2t+1) and need no shuffles.
    for (int blk = warp; blk < st_blocks; blk += R) {
      const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint16_t *xp = x_lane[nt] + (xi & 1) * xbuf_halves + blk * 128;
        if constexpr (GS == 32) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 xv = *reinterpret_cast<const uint4 *>(xp + 32 * jj);
            float sacc[4];
            mma16816<true>(sacc, ones, xv.x, xv.y);
            mma16816<false>(sacc, ones, xv.z, xv.w);
            if (g == 0)
              *reinterpret_cast<float2 *>(xsum + blk * kSumsPerBlock + jj * (NT * 8) + nt * 8 + 2 * t) =
                  make_float2(kNegZero * sacc[0], kNegZero * sacc[1]);
          }
        } else {
          // four independent accumulators, added at the end: the chain of dependent MMAs is two deep, not eight
          float sacc[4][4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 xv = *reinterpret_cast<const uint4 *>(xp + 32 * jj);
            mma16816<true>(sacc[jj], ones, xv.x, xv.y);
            mma16816<false>(sacc[jj], ones, xv.z, xv.w);
          }
          if (g == 0)
            *reinterpret_cast<float2 *>(xsum + blk * kSumsPerBlock + nt * 8 + 2 * t) =
                make_float2(kNegZero * ((sacc[0][0] + sacc[1][0]) + (sacc[2][0] + sacc[3][0])),
                            kNegZero * ((sacc[0][1] + sacc[1][1]) + (sacc[2][1] + sacc[3][1])));
        }
      }
    }
    __syncthreads();

    if (active && !failed) {
      // running offsets inside this activation stage: halves into the x rows, floats into the sums
      int x_off = (xi & 1) * xbuf_halves + w_lo * 128;  // w_lo is 0 unless the whole slice is staged
      int z_off = (xi & 1) * kXBlocks * kSumsPerBlock + w_lo * kSumsPerBlock;
      const int stage_blocks = min(kXBlocks, left);
      const int full_chunks = stage_blocks / CB, rem_blocks = stage_blocks - full_chunks * CB;
      auto do_block = [&](int cb) {
          uint32_t w[2 * B];
          {
            const unsigned char *blk = w_lane + st_off + cb * WBYTES;
#pragma unroll
            for (int v = 0; v < BlockTraits<B>::NV; ++v) {
              const uint4 q = *reinterpret_cast<const uint4 *>(blk + v * 512);
              w[4 * v + 0] = q.x;
              w[4 * v + 1] = q.y;
              w[4 * v + 2] = q.z;
              w[4 * v + 3] = q.w;
            }
            if constexpr (BlockTraits<B>::TAIL == 2) {
              const uint2 q = *reinterpret_cast<const uint2 *>(w_tail + st_off + cb * WBYTES);
              w[4 * BlockTraits<B>::NV + 0] = q.x;
              w[4 * BlockTraits<B>::NV + 1] = q.y;
            }
          }
          const uint16_t *sblk = reinterpret_cast<const uint16_t *>(s_lane + st_off + cb * SCB);  // [0]: row g, [8]: row g+8
          const float *bsum = z_lane + z_off + cb * kSumsPerBlock;
          const uint16_t *zblk = reinterpret_cast<const uint16_t *>(zp_lane + st_off + cb * SCB);

          // lanes whose batch column does not exist read the last valid row: their
          // accumulator columns are never written out
          uint4 xb[4][NT];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint16_t *xp = x_lane[nt] + x_off + cb * 128;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) xb[jj][nt] = *reinterpret_cast<const uint4 *>(xp + 32 * jj);
          }

          if constexpr (GS == 32) {
            // one group per pair of k-steps: each k-step gets its own accumulator
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              float d0[NT][4], d1[NT][4];
              uint32_t a0[4], a1[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                a0[q] = field_pair<B>(w, 8 * jj + q, 0u);
                a1[q] = field_pair<B>(w, 8 * jj + 4 + q, 0u);
              }
              const float f0 = 1.f / static_cast<float>(1 << kstep_offset<B>(2 * jj));
              const float f1 = 1.f / static_cast<float>(1 << kstep_offset<B>(2 * jj + 1));
              const float slo = scale_to_float<BF16>(sblk[jj * 16]);
              const float shi = scale_to_float<BF16>(sblk[jj * 16 + 8]);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma16816<true>(d0[nt], a0, xb[jj][nt].x, xb[jj][nt].y);
                mma16816<true>(d1[nt], a1, xb[jj][nt].z, xb[jj][nt].w);
                const float2 zs = *reinterpret_cast<const float2 *>(bsum + jj * (NT * 8) + nt * 8);
                float z4[4] = {zs.x, zs.y, zs.x, zs.y};
                if constexpr (ZP) {
                  const float zl = kZeroToCode * scale_to_float<BF16>(zblk[jj * 16]);
                  const float zh = kZeroToCode * scale_to_float<BF16>(zblk[jj * 16 + 8]);
                  z4[0] *= zl;
                  z4[1] *= zl;
                  z4[2] *= zh;
                  z4[3] *= zh;
                }
                yacc[nt][0] = fmaf(slo, fmaf(d1[nt][0], f1, fmaf(d0[nt][0], f0, z4[0])), yacc[nt][0]);
                yacc[nt][1] = fmaf(slo, fmaf(d1[nt][1], f1, fmaf(d0[nt][1], f0, z4[1])), yacc[nt][1]);
                yacc[nt][2] = fmaf(shi, fmaf(d1[nt][2], f1, fmaf(d0[nt][2], f0, z4[2])), yacc[nt][2]);
                yacc[nt][3] = fmaf(shi, fmaf(d1[nt][3], f1, fmaf(d0[nt][3], f0, z4[3])), yacc[nt][3]);
              }
            }
          } else {
            float acc[NCH][NT][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              uint32_t a[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) a[q] = field_pair<B>(w, 4 * i + q, 0u);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b0 = (i & 1) ? xb[i >> 1][nt].z : xb[i >> 1][nt].x;
                const uint32_t b1 = (i & 1) ? xb[i >> 1][nt].w : xb[i >> 1][nt].y;
                if (Chains<B>::first(i))
                  mma16816<true>(acc[Chains<B>::of(i)][nt], a, b0, b1);
                else
                  mma16816<false>(acc[Chains<B>::of(i)][nt], a, b0, b1);
              }
            }
            float slo = 1.f, shi = 1.f;
            if constexpr (GS == 128) {
              slo = scale_to_float<BF16>(sblk[0]);
              shi = scale_to_float<BF16>(sblk[8]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const float2 zs = *reinterpret_cast<const float2 *>(bsum + nt * 8);
              float tsum[4] = {zs.x, zs.y, zs.x, zs.y};
              if constexpr (ZP) {
                float zl = zrow_lo, zh = zrow_hi;
                if constexpr (GS == 128) {
                  zl = kZeroToCode * scale_to_float<BF16>(zblk[0]);
                  zh = kZeroToCode * scale_to_float<BF16>(zblk[8]);
                }
                tsum[0] *= zl;
                tsum[1] *= zl;
                tsum[2] *= zh;
                tsum[3] *= zh;
              }
#pragma unroll
              for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                for (int e = 0; e < 4; ++e) tsum[e] = fmaf(acc[ch][nt][e], Chains<B>::inv_factor(ch), tsum[e]);
              yacc[nt][0] = fmaf(slo, tsum[0], yacc[nt][0]);
              yacc[nt][1] = fmaf(slo, tsum[1], yacc[nt][1]);
              yacc[nt][2] = fmaf(shi, tsum[2], yacc[nt][2]);
              yacc[nt][3] = fmaf(shi, tsum[3], yacc[nt][3]);
            }
          }
      };
      // after a chunk: the stage has been read into registers by every lane, so it is refilled, and the
      // consumer moves to the next stage
      auto advance = [&]() {
        left -= CB;
        x_off += CB * 128;
        z_off += CB * kSumsPerBlock;
        __syncwarp();
        if (issue_left > 0) issue_next(st_off, st_bar);
        st_off += kStageBytes;
        st_bar += 8;
        if (st_off == kStages * kStageBytes) {
          st_off = 0;
          st_bar = bar_full0;
          st_parity ^= 1;
        }
      };
      for (int cc = 0; cc < full_chunks; ++cc) {
        if (!mbar_wait(st_bar, st_parity)) {
          failed = true;
          break;
        }
        // no per-block branches, so the blocks' instruction streams can interleave
#pragma unroll
        for (int cb = 0; cb < CB; ++cb) do_block(cb);
        advance();
      }
      if (CB > 1 && rem_blocks > 0 && !failed) {
        if (mbar_wait(st_bar, st_parity)) {
          for (int cb = 0; cb < rem_blocks; ++cb) do_block(cb);
          advance();
        } else {
          failed = true;
        }
      }
      if (failed) report_status(kStatusWeightCopyTimeout);
    }
    if (xi + 2 < nxst) {
      __syncthreads();  // every warp is done with this activation buffer
      if (threadIdx.x == 0) {
        // the buffer was read (and, for bf16, rewritten) through the generic proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue_x(xi + 2);
      }
    }
  }

  // 2^(8-b) (exact) and, for one scale per row, the row scale, both in fp32
  // (csrc/matgptq_gemm.cu:615-633, 943-949), together with 2^24 that undoes the
  // subnormal encoding of the codes.
  float mlo = static_cast<float>(1 << (8 - B)) * 16777216.f, mhi = mlo;
  if constexpr (GS == -1) {
    if (active) {
      mlo *= scale_to_float<BF16>(ldg_u16(p.s + static_cast<size_t>(tile) * 16 + g));
      mhi *= scale_to_float<BF16>(ldg_u16(p.s + static_cast<size_t>(tile) * 16 + g + 8));
    }
  }
  const int cols = Rt * 16;
  const int n0 = rg * cols;
  const int nslots = S * RK;  // partial sums per output
  if (nslots == 1 && !AR) {
    // nothing to add up: lane (g, t) holds rows g, g+8 of its tile for the batch columns 2t, 2t+1 of every batch tile
    if (active) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int m = nt * 8 + 2 * t + e;
          if (m < mvalid) {
            uint16_t *dst = p.y + static_cast<size_t>(m0 + m) * p.ldy + n0 + tw * 16 + g;
            dst[0] = float_to_out<BF16>(yacc[nt][e] * mlo);
            dst[8] = float_to_out<BF16>(yacc[nt][2 + e] * mhi);
          }
        }
    }
  } else {
    // Partial sums: slot (CTA rank, K slice) of the CTA that owns the column.  CTA r of the cluster owns the
    // columns [r*cw, (r+1)*cw) of this row group.  Every lane stores its partial sums straight into the owner's
    // shared memory (distributed shared memory when that is a peer), one barrier makes them visible, and the
    // owner adds the slots in a fixed order.  Nobody reads remote memory, so a CTA may leave as soon as it has
    // passed the barrier.
    const int cw = cols >> log2s;
    const float inv_cw = 1.f / static_cast<float>(cw);
    const uint32_t red_u32 = smem_base + plan.off_red;
    const int slot = crank * RK + kq;
    if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every peer has started
    if (active) {
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int col = tw * 16 + g + 8 * hrow;
        const int owner = static_cast<int>((static_cast<float>(col) + 0.5f) * inv_cw);
        const int j = col - owner * cw;
        uint32_t dst = red_u32 + (slot * plan.xrows * cw + j) * 4;
        if (S > 1) asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(dst), "r"(owner));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int m = nt * 8 + 2 * t + e;
            if (m < mvalid)
              asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + m * cw * 4),
                           "f"(yacc[nt][2 * hrow + e] * (hrow ? mhi : mlo))
                           : "memory");
          }
      }
    }
    if (S > 1) {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
      __syncthreads();
    }
    const int nbase = n0 + crank * cw;
    if constexpr (!AR) {
      for (int idx = threadIdx.x; idx < mvalid * cw; idx += blockDim.x) {
        const int m = static_cast<int>((static_cast<float>(idx) + 0.5f) * inv_cw), j = idx - m * cw;
        float sum = 0.f;
        for (int r = 0; r < nslots; ++r) sum += red[(r * plan.xrows + m) * cw + j];
        if (nbase + j < p.N) p.y[static_cast<size_t>(m0 + m) * p.ldy + nbase + j] = float_to_out<BF16>(sum);
      }
    } else {
      // ---- all-reduce over peer memory, fused: this CTA's column block of this rank's partial product ----
      const unsigned epoch = *reinterpret_cast<volatile unsigned *>(ar->ctrl) + 1u;  // the previous reduction has finished (stream order)
      const int set = static_cast<int>(epoch & 1u);
      const int nr = ar->nranks, me = ar->rank;
      const long long set_base = static_cast<long long>(set) * nr * ar->slot_elems;
      const uint2 *mine = ar->data[me] + set_base;  // what the other ranks store for this rank
      bool late = false;
      for (int idx = threadIdx.x; idx < mvalid * cw; idx += blockDim.x) {
        const int m = static_cast<int>((static_cast<float>(idx) + 0.5f) * inv_cw), j = idx - m * cw;
        float sum = 0.f;
        for (int r = 0; r < nslots; ++r) sum += red[(r * plan.xrows + m) * cw + j];
        if (nbase + j >= p.N) continue;
        const long long off = static_cast<long long>(m0 + m) * p.N + nbase + j;
        // 1. value and epoch in one 8-byte store into this rank's slot on every other rank
        const uint2 packet = make_uint2(__float_as_uint(sum), epoch);
        for (int q = 0; q < nr; ++q)
          if (q != me || ar->push_only) st_volatile_v2(ar->data[q] + set_base + me * ar->slot_elems + off, packet);
        if (ar->push_only) continue;
        // 2. the other ranks' values of the same output, in rank order (every rank adds the same numbers in the
        //    same order); a word that does not show the epoch within about a second is reported, not waited for
        float total = 0.f;
        for (int r = 0; r < nr; ++r) {
          if (r == me) {
            total += sum;
            continue;
          }
          const uint2 *src = mine + r * ar->slot_elems + off;
          uint2 v = ld_volatile_v2(src);
          for (unsigned it = 0; v.y != epoch && it < (1u << 22); ++it) {
            if (it > 16) __nanosleep(it < 4096 ? 32 : 256);
            v = ld_volatile_v2(src);
          }
          if (v.y != epoch) late = true;
          total += __uint_as_float(v.x);
        }
        p.y[static_cast<size_t>(m0 + m) * p.ldy + nbase + j] = float_to_out<BF16>(total);
      }
      if (late) report_status(kStatusPeerTimeout);
      // 5. the last CTA of the launch closes the epoch (with push_only the finishing kernel does)
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y;
        __threadfence();
        const unsigned ticket = atomicAdd(ar->ctrl + 1, 1u);
        if (ticket == total - 1) {
          ar->ctrl[1] = 0;
          __threadfence();
          if (!ar->push_only) *reinterpret_cast<volatile unsigned *>(ar->ctrl) = epoch;
        }
      }
    }
  }
}

template <int B, int GS, bool BF16, int NT, bool ZP>
__global__ void __launch_bounds__(512, 1) gemv_kernel(const GemvParams p) {
  gemv_body<B, GS, BF16, NT, ZP>(p, static_cast<int>(blockIdx.x));
}

#if !MG_GEMV_ZP
// Row-parallel product fused with the all-reduce of its output (group size 128; see ArParams in kernels.h).
template <int B, bool BF16, int NT>
__global__ void __launch_bounds__(512, 1) gemv_allreduce_kernel(const GemvParams p, const ArParams ar) {
  gemv_body<B, 128, BF16, NT, false, true>(p, static_cast<int>(blockIdx.x), &ar);
}

// Second half of the protocol as a kernel of its own, for launches made with push_only (one GPU standing in for all
// ranks: the ranks' products run one after the other, so nothing may wait inside them): adds the slots in rank
// order, reports any value that does not carry the current epoch, closes the epoch.
template <bool BF16>
__global__ void allreduce_finish_kernel(const ArParams ar, uint16_t *y, int N, int M) {
  const unsigned epoch = *reinterpret_cast<volatile unsigned *>(ar.ctrl) + 1u;
  const int set = static_cast<int>(epoch & 1u);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const uint2 *mine = ar.data[ar.rank] + static_cast<long long>(set) * ar.nranks * ar.slot_elems;
  bool missing = false;
  for (long long i = tid; i < static_cast<long long>(M) * N; i += nthreads) {
    float sum = 0.f;
    for (int r = 0; r < ar.nranks; ++r) {
      const uint2 v = ld_volatile_v2(mine + r * ar.slot_elems + i);
      if (v.y != epoch) missing = true;
      sum += __uint_as_float(v.x);
    }
    y[i] = float_to_out<BF16>(sum);
  }
  if (missing) report_status(kStatusPeerTimeout);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ar.ctrl + 1, 1u) == gridDim.x - 1) {
      ar.ctrl[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned *>(ar.ctrl) = epoch;
    }
  }
}

// ----------------------------------------------------------------------------
// Grouped launch: several products over the SAME activations in one kernel, each with its own packed
// weights, scales, out-features and bitwidth, written side by side into one output [M, sum N_i].  This is
// what a fused qkv or gate_up layer with per-layer bitwidths needs (vLLM fuses those layers,
// inference_lib/vllm_matgptq.py:113-121; a bitwidth file gives each checkpoint layer its own b,
// evo_quant_search.py:659-671): one launch and one fixed cost instead of one per bitwidth segment.
// Every CTA finds its segment from the table and runs that segment's body; all segments share the launch
// shape (warps, K slices, cluster size) and the shared-memory request.
// ----------------------------------------------------------------------------
constexpr int kMaxSegments = 8;

struct GroupedParams {
  const uint32_t *w[kMaxSegments];
  const uint16_t *s[kMaxSegments];
  int n_out[kMaxSegments];
  int col0[kMaxSegments];    // first output column of the segment
  int cta0[kMaxSegments + 1];  // first CTA (blockIdx.x) of the segment; cta0[nseg] = gridDim.x
  signed char bits[kMaxSegments];
  signed char stages[kMaxSegments];
  int nseg;
  const uint16_t *x;
  uint16_t *y;
  int ldy, K, M, kblocks, split, xblocks, kslices;
};

template <int GS, bool BF16, int NT>
__global__ void __launch_bounds__(512, 1) gemv_grouped_kernel(const GroupedParams gp) {
  int seg = 0;
  const int bx = static_cast<int>(blockIdx.x);
#pragma unroll
  for (int i = 1; i < kMaxSegments; ++i)
    if (i < gp.nseg && bx >= gp.cta0[i]) seg = i;
  GemvParams p;
  p.w = gp.w[seg];
  p.s = gp.s[seg];
  p.z = nullptr;
  p.x = gp.x;
  p.y = gp.y + gp.col0[seg];
  p.N = gp.n_out[seg];
  p.K = gp.K;
  p.M = gp.M;
  p.ldy = gp.ldy;
  p.tiles = p.N / 16;
  p.kblocks = gp.kblocks;
  p.split = gp.split;
  p.stages = gp.stages[seg];
  p.xblocks = gp.xblocks;
  p.kslices = gp.kslices;
  const int local = bx - gp.cta0[seg];
  switch (gp.bits[seg]) {  // uniform over the CTA (and over its cluster: segments start at cluster boundaries)
    case 2: gemv_body<2, GS, BF16, NT, false>(p, local); break;
    case 3: gemv_body<3, GS, BF16, NT, false>(p, local); break;
    case 4: gemv_body<4, GS, BF16, NT, false>(p, local); break;
    case 6: gemv_body<6, GS, BF16, NT, false>(p, local); break;
    default: gemv_body<8, GS, BF16, NT, false>(p, local); break;
  }
}
#endif

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
// Shared memory per CTA that leaves room for exactly `ctas` CTAs on an SM (227 KB usable, 1 KB reserved per CTA).
static inline int smem_for_ctas_per_sm(int ctas) { return (227 * 1024) / ctas - 1024; }

template <int B, int GS, bool BF16, int NT>
static int launch_gemv(GemvParams p, int R, cudaStream_t stream, bool pdl) {
  auto kernel = gemv_kernel<B, GS, BF16, NT, kZP>;
  const int S = p.split;
  const int max_nblk = (p.kblocks + S - 1) / S;
  // About 16 warps per SM: CTAs of R warps come 16/R to an SM.  The ring takes what is left of that share of
  // the shared memory after the activations (2 to 8 stages), and the request is padded so that one CTA more
  // does not fit: the block scheduler otherwise stacks CTAs on the SMs that free up first.
  const int ctas_per_sm = R >= 16 ? 1 : 16 / R;
  const int budget = smem_for_ctas_per_sm(ctas_per_sm);
  const int nchunks = (max_nblk + ChunkBlocks<B, NT>::value - 1) / ChunkBlocks<B, NT>::value;
  // Activations: the whole K slice of the CTA in one piece when that leaves room for two ring stages (no
  // buffer turnover, so the warps never meet at a barrier inside the loop), else double-buffered stages.
  int xblocks = max_nblk;
  if (make_plan<B, GS, NT, kZP>(R, p.M, max_nblk, 2, xblocks).total > budget) {
    if (p.kslices > 1) return MG_ERR_UNSUPPORTED;  // K slices inside a CTA need the whole slice of the activations staged
    xblocks = (NT == 1) ? 8 : 4;
  }
  if (xblocks > max_nblk) xblocks = max_nblk;
  int stages = 2;
  while (stages < 8 && stages < nchunks && make_plan<B, GS, NT, kZP>(R, p.M, max_nblk, stages + 1, xblocks).total <= budget) ++stages;
  p.stages = stages;
  p.xblocks = xblocks;
  const SmemPlan plan = make_plan<B, GS, NT, kZP>(R, p.M, max_nblk, stages, xblocks);
  if (plan.total > 227 * 1024 - 1024) return MG_ERR_UNSUPPORTED;
  const int floor_bytes = smem_for_ctas_per_sm(ctas_per_sm + 1) + 1;
  const size_t smem = static_cast<size_t>(plan.total > floor_bytes ? plan.total : floor_bytes);
  if (smem > 48 * 1024) {
    static SharedMemoryOptIn opt_in;  // one per instantiation of this launcher
    const int st = opt_in.ensure(kernel, 226 * 1024);
    if (st != MG_OK) return st;
  }
  const int Rt = R / p.kslices;
  const int row_groups = (p.tiles + Rt - 1) / Rt;
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

// Launch shape: R warps per CTA as Rt row tiles x RK slices of the CTA's K range, S CTAs per cluster along K.
// Measured on B200 (Llama-3-8B shapes, b in {2,4,8}, batch 1/8/16):
//   * the kernel wants 12-14 warps per SM in total, so K is split T = S * RK ways with tiles * T close to
//     14 * SMs, and no further (every split pays set-up, an activation copy and the reduction);
//   * CTAs of 8 warps, two to an SM, beat fatter CTAs for batches up to 8; with more than 8 rows the
//     activations dominate shared memory and one 16-warp CTA per SM that stages its whole K slice wins;
//   * for T >= 4 half of the split is better done inside the CTA (RK = 2: partial sums meet in local shared
//     memory, smaller clusters), provided the CTA's whole K slice of the activations fits (`second` is the
//     shape to use when it does not).
struct GemvShape {
  int R, RK, S;
};

static void gemv_pick_config(int tiles, int kblocks, int batch, int sm_count, GemvShape *first, GemvShape *second) {
  const int want_warps = 14 * sm_count;
  int T = 1;
  while (T < 16 && tiles * T * 2 <= want_warps && T * 2 <= kblocks) T <<= 1;
  int S = T > 8 ? 8 : T;
  int R = 8;
  while (R > 1 && static_cast<long long>((tiles + R - 1) / R) * S < sm_count) R >>= 1;
  *second = GemvShape{R, 1, S};
  *first = *second;
  if (T >= 4 && tiles >= 4) {
    *first = GemvShape{8, 2, T / 2};
  } else if (batch > 8 && T == 2 && tiles >= 16 * sm_count / 4) {
    *first = GemvShape{16, 1, 2};
  }
}

static int launch_shape(GemvParams p, const GemvShape &c, int bitwidth, int group_size, bool bf16, bool pdl,
                        cudaStream_t stream) {
  const int R = c.R, S = c.S, RK = c.RK;
  if (R < 1 || R > 16 || S < 1 || S > 8 || (S & (S - 1)) != 0 || S > p.kblocks) return MG_ERR_BAD_ARG;
  if (RK < 1 || R % RK != 0 || RK > p.kblocks / S) return MG_ERR_BAD_ARG;
  if ((R / RK) * 16 % S != 0) return MG_ERR_BAD_ARG;  // the columns of a row group are shared out evenly over the cluster
  p.split = S;
  p.kslices = RK;
  switch (bitwidth) {
    case 2: return launch_gemv_group<2>(p, R, group_size, bf16, stream, pdl);
    case 3: return launch_gemv_group<3>(p, R, group_size, bf16, stream, pdl);
    case 4: return launch_gemv_group<4>(p, R, group_size, bf16, stream, pdl);
    case 6: return launch_gemv_group<6>(p, R, group_size, bf16, stream, pdl);
    case 8: return launch_gemv_group<8>(p, R, group_size, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

#if MG_GEMV_ZP
#define MG_GEMV_LAUNCH gemv_zp_launch
#define MG_GEMV_STATUS gemv_zp_device_status
#else
#define MG_GEMV_LAUNCH gemv_launch
#define MG_GEMV_STATUS gemv_device_status
#endif

// z: zero points (reordered like the scales) for the build with zero points, null for the other one
int MG_GEMV_LAUNCH(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *z,
                   const void *x, void *y, bool bf16, bool pdl, int R_override, int S_override, cudaStream_t stream,
                   int ldy) {
  if (kZP != (z != nullptr)) return MG_ERR_BAD_ARG;
  int sm_count = 0;
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  GemvParams p;
  p.w = static_cast<const uint32_t *>(w);
  p.s = static_cast<const uint16_t *>(s);
  p.z = static_cast<const uint16_t *>(z);
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.N = N;
  p.K = K;
  p.M = M;
  p.ldy = ldy > 0 ? ldy : N;
  p.tiles = N / 16;
  p.kblocks = K / 128;
  GemvShape first, second;
  gemv_pick_config(p.tiles, p.kblocks, M < 16 ? M : 16, sm_count, &first, &second);
  if (R_override > 0 || S_override > 0) {
    // forced shape.  warps: low byte = warps per CTA, next byte = K slices inside the CTA (0 means 1)
    GemvShape forced = second;
    if (R_override > 0) {
      forced.R = R_override & 0xFF;
      forced.RK = (R_override >> 8) & 0xFF;
      if (forced.RK == 0) forced.RK = 1;
    }
    if (S_override > 0) forced.S = S_override;
    return launch_shape(p, forced, bitwidth, group_size, bf16, pdl, stream);
  }
  int r = launch_shape(p, first, bitwidth, group_size, bf16, pdl, stream);
  // Nothing was launched when the shape does not fit in shared memory: use the plain cluster split.
  if (r == MG_ERR_UNSUPPORTED) r = launch_shape(p, second, bitwidth, group_size, bf16, pdl, stream);
  return r;
}

#if !MG_GEMV_ZP
// ---- product + all-reduce, host side -----------------------------------------------------------------------
template <int B, bool BF16, int NT>
static int launch_allreduce(GemvParams p, const ArParams &ar, const GemvShape &c, cudaStream_t stream, bool pdl) {
  auto kernel = gemv_allreduce_kernel<B, BF16, NT>;
  const int R = c.R, S = c.S, RK = c.RK;
  if (R < 1 || R > 16 || S < 1 || S > 8 || (S & (S - 1)) != 0 || S > p.kblocks) return MG_ERR_UNSUPPORTED;
  if (RK < 1 || R % RK != 0 || RK > p.kblocks / S || (R / RK) * 16 % S != 0) return MG_ERR_UNSUPPORTED;
  p.split = S;
  p.kslices = RK;
  const int max_nblk = (p.kblocks + S - 1) / S;
  const int ctas_per_sm = R >= 16 ? 1 : 16 / R;
  const int budget = smem_for_ctas_per_sm(ctas_per_sm);
  const int nchunks = (max_nblk + ChunkBlocks<B, NT>::value - 1) / ChunkBlocks<B, NT>::value;
  int xblocks = max_nblk;
  if (make_plan<B, 128, NT, false>(R, p.M, max_nblk, 2, xblocks).total > budget) {
    if (RK > 1) return MG_ERR_UNSUPPORTED;
    xblocks = (NT == 1) ? 8 : 4;
  }
  if (xblocks > max_nblk) xblocks = max_nblk;
  int stages = 2;
  while (stages < 8 && stages < nchunks && make_plan<B, 128, NT, false>(R, p.M, max_nblk, stages + 1, xblocks).total <= budget) ++stages;
  p.stages = stages;
  p.xblocks = xblocks;
  const SmemPlan plan = make_plan<B, 128, NT, false>(R, p.M, max_nblk, stages, xblocks);
  if (plan.total > 227 * 1024 - 1024) return MG_ERR_UNSUPPORTED;
  const int floor_bytes = smem_for_ctas_per_sm(ctas_per_sm + 1) + 1;
  const size_t smem = static_cast<size_t>(plan.total > floor_bytes ? plan.total : floor_bytes);
  if (smem > 48 * 1024) {
    static SharedMemoryOptIn opt_in;
    const int st = opt_in.ensure(kernel, 226 * 1024);
    if (st != MG_OK) return st;
  }
  const int Rt = R / RK;
  const int row_groups = (p.tiles + Rt - 1) / Rt;
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
  return cudaLaunchKernelEx(&cfg, kernel, p, ar) == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <int B>
static int launch_allreduce_b(const GemvParams &p, const ArParams &ar, const GemvShape &c, bool bf16, cudaStream_t stream, bool pdl) {
  if (p.M <= 8)
    return bf16 ? launch_allreduce<B, true, 1>(p, ar, c, stream, pdl) : launch_allreduce<B, false, 1>(p, ar, c, stream, pdl);
  return bf16 ? launch_allreduce<B, true, 2>(p, ar, c, stream, pdl) : launch_allreduce<B, false, 2>(p, ar, c, stream, pdl);
}

// MG_ERR_UNSUPPORTED (nothing launched, nothing published) for group sizes other than 128 and shapes that do not fit.
int gemv_allreduce_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                          void *y, bool bf16, bool pdl, const ArParams &ar, cudaStream_t stream) {
  if (group_size != 128 || ar.nranks < 1 || ar.nranks > kArMaxRanks || ar.rank < 0 || ar.rank >= ar.nranks) return MG_ERR_UNSUPPORTED;
  if (static_cast<long long>(M) * N > ar.slot_elems) return MG_ERR_UNSUPPORTED;
  int sm_count = 0;
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  GemvParams p;
  p.w = static_cast<const uint32_t *>(w);
  p.s = static_cast<const uint16_t *>(s);
  p.z = nullptr;
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.N = N;
  p.K = K;
  p.M = M;
  p.ldy = N;
  p.tiles = N / 16;
  p.kblocks = K / 128;
  GemvShape first, second;
  gemv_pick_config(p.tiles, p.kblocks, M < 16 ? M : 16, sm_count, &first, &second);
  auto launch = [&](const GemvShape &c) {
    switch (bitwidth) {
      case 2: return launch_allreduce_b<2>(p, ar, c, bf16, stream, pdl);
      case 3: return launch_allreduce_b<3>(p, ar, c, bf16, stream, pdl);
      case 4: return launch_allreduce_b<4>(p, ar, c, bf16, stream, pdl);
      case 6: return launch_allreduce_b<6>(p, ar, c, bf16, stream, pdl);
      case 8: return launch_allreduce_b<8>(p, ar, c, bf16, stream, pdl);
      default: return static_cast<int>(MG_ERR_BAD_ARG);
    }
  };
  int r = launch(first);
  if (r == MG_ERR_UNSUPPORTED) r = launch(second);
  return r;
}

int allreduce_finish_launch(const ArParams &ar, void *y, int N, int M, bool bf16, cudaStream_t stream) {
  long long blocks = (static_cast<long long>(M) * N + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  if (bf16)
    allreduce_finish_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ar, static_cast<uint16_t *>(y), N, M);
  else
    allreduce_finish_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ar, static_cast<uint16_t *>(y), N, M);
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

// ---- grouped launch, host side --------------------------------------------------------------------------
template <int GS, int NT> static SmemPlan plan_for_bits(int bits, int R, int M, int max_nblk, int stages, int xblocks) {
  switch (bits) {
    case 2: return make_plan<2, GS, NT, false>(R, M, max_nblk, stages, xblocks);
    case 3: return make_plan<3, GS, NT, false>(R, M, max_nblk, stages, xblocks);
    case 4: return make_plan<4, GS, NT, false>(R, M, max_nblk, stages, xblocks);
    case 6: return make_plan<6, GS, NT, false>(R, M, max_nblk, stages, xblocks);
    default: return make_plan<8, GS, NT, false>(R, M, max_nblk, stages, xblocks);
  }
}

template <int GS, bool BF16, int NT>
static int launch_grouped(GroupedParams gp, const GroupedSegment *segments, const GemvShape &c, cudaStream_t stream, bool pdl) {
  auto kernel = gemv_grouped_kernel<GS, BF16, NT>;
  const int R = c.R, S = c.S, RK = c.RK;
  if (R < 1 || R > 16 || S < 1 || S > 8 || (S & (S - 1)) != 0 || S > gp.kblocks) return MG_ERR_UNSUPPORTED;
  if (RK < 1 || R % RK != 0 || RK > gp.kblocks / S) return MG_ERR_UNSUPPORTED;
  const int Rt = R / RK;
  if (Rt * 16 % S != 0) return MG_ERR_UNSUPPORTED;
  const int max_nblk = (gp.kblocks + S - 1) / S;
  const int ctas_per_sm = R >= 16 ? 1 : 16 / R;
  const int budget = smem_for_ctas_per_sm(ctas_per_sm);
  // activations: the CTA's whole K slice when that leaves every segment two ring stages, else stages of a few blocks
  int xblocks = max_nblk;
  for (int i = 0; i < gp.nseg; ++i)
    if (plan_for_bits<GS, NT>(gp.bits[i], R, gp.M, max_nblk, 2, xblocks).total > budget) xblocks = 0;
  if (xblocks == 0) {
    if (RK > 1) return MG_ERR_UNSUPPORTED;
    xblocks = (NT == 1) ? 8 : 4;
    if (xblocks > max_nblk) xblocks = max_nblk;
  }
  int smem = smem_for_ctas_per_sm(ctas_per_sm + 1) + 1;  // padded so that one CTA more does not fit on the SM
  int cta = 0;
  for (int i = 0; i < gp.nseg; ++i) {
    const int cb = gp.bits[i] <= 4 ? 4 : 2;  // ChunkBlocks
    const int nchunks = (max_nblk + cb - 1) / cb;
    int stages = 2;
    while (stages < 8 && stages < nchunks &&
           plan_for_bits<GS, NT>(gp.bits[i], R, gp.M, max_nblk, stages + 1, xblocks).total <= budget)
      ++stages;
    const int total = plan_for_bits<GS, NT>(gp.bits[i], R, gp.M, max_nblk, stages, xblocks).total;
    if (total > 227 * 1024 - 1024) return MG_ERR_UNSUPPORTED;
    if (total > smem) smem = total;
    gp.stages[i] = static_cast<signed char>(stages);
    gp.cta0[i] = cta;
    cta += ((segments[i].n_out / 16 + Rt - 1) / Rt) * S;
  }
  gp.cta0[gp.nseg] = cta;
  gp.split = S;
  gp.kslices = RK;
  gp.xblocks = xblocks;
  if (smem > 48 * 1024) {
    static SharedMemoryOptIn opt_in;
    const int st = opt_in.ensure(kernel, 226 * 1024);
    if (st != MG_OK) return st;
  }
  const int passes = (gp.M + NT * 8 - 1) / (NT * 8);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cta, passes, 1);
  cfg.blockDim = dim3(R * 32, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
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
  return cudaLaunchKernelEx(&cfg, kernel, gp) == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <int GS>
static int launch_grouped_gs(const GroupedParams &gp, const GroupedSegment *segments, const GemvShape &c, bool bf16,
                             cudaStream_t stream, bool pdl) {
  if (gp.M <= 8)
    return bf16 ? launch_grouped<GS, true, 1>(gp, segments, c, stream, pdl) : launch_grouped<GS, false, 1>(gp, segments, c, stream, pdl);
  return bf16 ? launch_grouped<GS, true, 2>(gp, segments, c, stream, pdl) : launch_grouped<GS, false, 2>(gp, segments, c, stream, pdl);
}

int gemv_grouped_launch(const GroupedSegment *segments, int nseg, int group_size, int K, int M, const void *x, void *y,
                        int ldy, bool bf16, bool pdl, cudaStream_t stream) {
  if (nseg < 1 || nseg > kMaxSegments) return MG_ERR_UNSUPPORTED;
  int sm_count = 0;
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  GroupedParams gp = {};
  int tiles = 0, col = 0;
  for (int i = 0; i < nseg; ++i) {
    gp.w[i] = static_cast<const uint32_t *>(segments[i].w);
    gp.s[i] = static_cast<const uint16_t *>(segments[i].s);
    gp.n_out[i] = segments[i].n_out;
    gp.col0[i] = col;
    gp.bits[i] = static_cast<signed char>(segments[i].bitwidth);
    col += segments[i].n_out;
    tiles += segments[i].n_out / 16;
  }
  gp.nseg = nseg;
  gp.x = static_cast<const uint16_t *>(x);
  gp.y = static_cast<uint16_t *>(y);
  gp.ldy = ldy;
  gp.K = K;
  gp.M = M;
  gp.kblocks = K / 128;
  GemvShape first, second;
  gemv_pick_config(tiles, gp.kblocks, M < 16 ? M : 16, sm_count, &first, &second);
  auto launch = [&](const GemvShape &c) {
    switch (group_size) {
      case -1: return launch_grouped_gs<-1>(gp, segments, c, bf16, stream, pdl);
      case 32: return launch_grouped_gs<32>(gp, segments, c, bf16, stream, pdl);
      case 128: return launch_grouped_gs<128>(gp, segments, c, bf16, stream, pdl);
      default: return static_cast<int>(MG_ERR_BAD_ARG);
    }
  };
  int r = launch(first);
  if (r == MG_ERR_UNSUPPORTED) r = launch(second);
  return r;
}
#endif

MG_DEFINE_STATUS_ACCESSOR(MG_GEMV_STATUS)

}  // namespace mg
