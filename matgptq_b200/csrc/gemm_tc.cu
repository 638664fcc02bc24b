// Tensor-core path for batches of more than 16 rows: tcgen05.mma with the accumulator
// in tensor memory.
//
// Replaces gptq_matryoshka for large batches (csrc/matgptq_gemm.cu:337-634), which
// re-reads the weights once per 8 batch columns and stays below a dense fp16 GEMM
// from M = 32 up.  Here one CTA owns 128 out-features and up to 256 batch rows:
//
//   * "dequant" warps (one per 16-row tile of the packed layout; two per tile, one 64-wide half each, when the
//     CTA has its SM to itself) decode their block to the exact dense weights of the reference's dequantize()
//     (round(scale * (code*2^(8-b) - 128)), fp16 or bf16) and store them K-major into a shared-memory stage
//     in the canonical no-swizzle UMMA layout (8 x 16-byte core matrices), with the packed words of the next
//     three to six blocks already in flight;
//   * one thread of the last warp fetches the activation tiles (batch rows x 64 in-features) with TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle, rows past the batch filled with zeros), as far ahead as
//     the pipeline has stages; an elected lane of the warp before it issues tcgen05.mma (M = 128 weight
//     rows, N = batch rows, K = 16) from shared-memory descriptors; D[128, N] lives in tensor memory;
//     completion of a stage's MMAs releases the stage through tcgen05.commit -> mbarrier;
//   * the epilogue reads D with tcgen05.ld (each warp its own 32 TMEM lanes), converts
//     and stores y[m, n] (the transpose of D); when K is split, the CTAs that share a tile form a
//     thread-block cluster, leave their fp32 sums in shared memory, and each adds and stores a share
//     of the batch rows through distributed shared memory, in the order of the K ranges.
//
// Every mbarrier wait is bounded (async.cuh); tensor memory is freed on every path.
#include <cuda.h>  // CUtensorMap and its enums; cuTensorMapEncodeTiled is resolved at run time
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "async.cuh"
#include "decode.cuh"
#include "host_util.h"
#include "kernels.h"

namespace mg {

// A pipeline stage covers 64 in-features (half a packed block).
constexpr int kTcChunkStride = 2080;   // bytes between 16-byte K chunks of the A stage: 128 rows * 16 B + 32 B
                                       // (the 32 bytes spread the four k-chunks a warp stores at once over all banks)
constexpr int kTcAStageBytes = 8 * kTcChunkStride;  // 8 chunks of 8 in-features

struct GemmParams {
  const uint32_t *w;
  const uint16_t *s;
  const uint16_t *x;
  uint16_t *y;
  int N, K, M;
  int ldy;      // elements between two rows of y (N unless the call writes a column block of a wider output)
  int kblocks;  // K / 128
  float *partial;  // null: the CTAs along K add their sums inside a cluster; else [split][M][N] fp32 scratch for them
  int split;    // CTAs along K
  int ncols;    // UMMA N: batch rows per pass rounded up to 16
  int stages;
};

// TMA load of one box of a 2-D tensor map into shared memory; x (the innermost coordinate) times the element
// size must be a multiple of 16 bytes: here x is a multiple of 64 two-byte elements.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
               : "memory");
}

// 64-bit shared-memory matrix descriptor (K-major).  layout_type: 0 = no swizzle, 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= static_cast<uint64_t>(layout_type & 7u) << 61;
  return d;
}

// 32-bit instruction descriptor: fp32 accumulate, A and B both K-major, both fp16 (0) or bf16 (1).
__host__ __device__ inline uint32_t umma_instr_desc(int fmt, int n) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  elect.sync _|p, 0xffffffff;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <bool BF16> __device__ __forceinline__ uint16_t to_out16(float f) {
  return BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f)) : __half_as_ushort(__float2half_rn(f));
}

// every thread of every CTA of the cluster; orders shared-memory writes before the other CTAs' reads
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// address of this CTA's shared-memory location `addr` in the CTA of rank `cta` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, int cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// shared-memory plan (host and device)
struct TcPlan {
  int b_stage_bytes, stage_bytes, off_stages, total;
};
__host__ __device__ inline TcPlan tc_plan(int ncols, int stages) {
  TcPlan p;
  p.b_stage_bytes = ncols * 128;                               // 64 in-features * 2 B per batch row
  p.stage_bytes = 1024 * ((kTcAStageBytes + p.b_stage_bytes + 1023) / 1024);  // B first, 1024-aligned for the swizzle
  p.off_stages = 1024;                                         // barriers and the TMEM address live below
  p.total = p.off_stages + stages * p.stage_bytes + 1024;      // slack to align the dynamic base to 1024
  return p;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint16_t ldg_u16_tc(const uint16_t *p) {
  uint16_t r;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
  return r;
}

// scale groups per 128-wide block
template <int GS> struct TcScales {
  static constexpr int NG = (GS == 32) ? 4 : 1;
};

// 16 bytes to shared memory at addr + OFF (OFF goes into the instruction)
template <int OFF> __device__ __forceinline__ void sts_v4(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.b32 [%0 + %5], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "n"(OFF)
               : "memory");
}

// Chunk JJ (0..3, 32 in-features) of a block: this lane's dense weights of rows g (lo) and g+8 (hi), eight each, as
// 16 bytes per row into the A tile whose lane address for chunk 0 is `addr`.
template <int B, bool BF16, int JJ>
__device__ __forceinline__ void tc_store_chunk(const uint32_t (&w)[2 * B], uint32_t s_lo, uint32_t s_hi, uint32_t addr) {
  uint4 lo, hi;
  lo.x = dense_pair<B, BF16>(w, 8 * JJ + 0, s_lo);
  lo.y = dense_pair<B, BF16>(w, 8 * JJ + 2, s_lo);
  lo.z = dense_pair<B, BF16>(w, 8 * JJ + 4, s_lo);
  lo.w = dense_pair<B, BF16>(w, 8 * JJ + 6, s_lo);
  hi.x = dense_pair<B, BF16>(w, 8 * JJ + 1, s_hi);
  hi.y = dense_pair<B, BF16>(w, 8 * JJ + 3, s_hi);
  hi.z = dense_pair<B, BF16>(w, 8 * JJ + 5, s_hi);
  hi.w = dense_pair<B, BF16>(w, 8 * JJ + 7, s_hi);
  sts_v4<(JJ & 1) * 4 * kTcChunkStride>(addr, lo);
  sts_v4<(JJ & 1) * 4 * kTcChunkStride + 128>(addr, hi);
}

// Half H (0, 1) of a block = chunks 2H and 2H+1 = one pipeline stage; slo/shi: raw scales of rows g and g+8
template <int B, int GS, bool BF16, int H>
__device__ __forceinline__ void tc_store_half(const uint32_t (&w)[2 * B], const uint16_t (&slo)[TcScales<GS>::NG],
                                              const uint16_t (&shi)[TcScales<GS>::NG], uint32_t addr) {
  constexpr int g0 = (GS == 32) ? 2 * H : 0, g1 = (GS == 32) ? 2 * H + 1 : 0;
  const uint32_t lo0 = dense_scale<B, BF16>(slo[g0]), hi0 = dense_scale<B, BF16>(shi[g0]);
  tc_store_chunk<B, BF16, 2 * H>(w, lo0, hi0, addr);
  const uint32_t lo1 = (GS == 32) ? dense_scale<B, BF16>(slo[g1]) : lo0, hi1 = (GS == 32) ? dense_scale<B, BF16>(shi[g1]) : hi0;
  tc_store_chunk<B, BF16, 2 * H + 1>(w, lo1, hi1, addr);
}

struct TcProducer {
  uint32_t off, idx8, parity;            // byte offset, barrier offset and empty-barrier parity of the current stage
  uint32_t stage_bytes, stages8;         // bytes per stage; 8 * number of stages
  uint32_t bar_full, bar_empty, a_lane;  // shared-memory addresses for stage 0
};

// One 64-wide half (H = 0, 1) of a block: wait for the stage, decode and store this lane's share, hand the stage
// over, move on to the next stage.  `mine` false: the half belongs to the other warp of the pair.
template <int B, int GS, bool BF16, int H>
__device__ __forceinline__ bool tc_producer_half(TcProducer &pr, bool mine, bool valid, int lane, const uint32_t (&w)[2 * B],
                                                 const uint16_t (&slo)[TcScales<GS>::NG],
                                                 const uint16_t (&shi)[TcScales<GS>::NG]) {
  if (mine) {
    if (!mbar_wait(pr.bar_empty + pr.idx8, pr.parity)) return false;  // the tensor pipe is done with what this stage held
    if (valid) tc_store_half<B, GS, BF16, H>(w, slo, shi, pr.a_lane + pr.off);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor pipe reads
    __syncwarp();
    if (lane == 0) mbar_arrive(pr.bar_full + pr.idx8);
  }
  pr.off += pr.stage_bytes;
  pr.idx8 += 8;
  if (pr.idx8 == pr.stages8) {
    pr.off = 0;
    pr.idx8 = 0;
    pr.parity ^= 1;
  }
  return true;
}

// PW producer warps: 8 (each decodes both 64-wide halves of its blocks; two CTAs share an SM) or 16 (warps w and
// w + 8 share a row tile and take one half each, so that a CTA that has the SM to itself overlaps the latency of
// one stage with the work of the next).
template <int B, int GS, bool BF16, int PW>
__device__ __forceinline__ void gemm_tc_body(const GemmParams &p, const CUtensorMap &xmap, const int tile128) {
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t raw_u32 = smem_u32(tc_smem_raw);
  const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u;
  unsigned char *base = tc_smem_raw + (base_u32 - raw_u32);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int stages = p.stages;
  const TcPlan plan = tc_plan(p.ncols, stages);
  const uint32_t bar_full = base_u32;               // stages barriers: 8 producer warps + the TMA issuer (and its bytes)
  const uint32_t bar_empty = base_u32 + 8 * 8;      // stages barriers, released by tcgen05.commit
  const uint32_t bar_done = base_u32 + 16 * 8;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base + 17 * 8);

  const int sk = blockIdx.y;
  const int m0 = blockIdx.z * 256;
  const int mrows = min(p.M - m0, 256);
  const int kb_lo = sk * p.kblocks / p.split;
  const int kb_hi = (sk + 1) * p.kblocks / p.split;
  const int nblk = kb_hi - kb_lo;
  const int nit = 2 * nblk;  // pipeline iterations of 64 in-features
  const int groups = (GS == -1) ? 1 : p.K / GS;
  int tmem_cols = 32;
  while (tmem_cols < p.ncols) tmem_cols <<= 1;

  if (warp == PW) {
    if (lane == 0) {
      for (int i = 0; i < stages; ++i) {
        mbar_init(bar_full + i * 8, 9);  // the eight producer warps of a stage and the thread that requests the activations
        mbar_init(bar_empty + i * 8, 1);
      }
      mbar_init(bar_done, 1);
      mbar_init_fence();
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base_u32 + 17 * 8), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Programmatic dependent launch: the producers only read weights and scales, which no kernel writes, so they
  // start at once; the thread that fetches the activations waits for the previous kernel before its first
  // request, and the producers wait before the epilogue writes anything.
  asm volatile("griddepcontrol.launch_dependents;");

  bool failed = false;
  if (warp < PW) {
    // ------------------------------------------------------------------ producers
    const int ptile = warp & 7, my_half = warp >> 3;
    const int tile16 = tile128 * 8 + ptile;
    const bool valid = tile16 < p.N / 16;
    constexpr int BW = BlockTraits<B>::WORDS;
    constexpr int NG = TcScales<GS>::NG;
    // Packed words and scales of three to six blocks in flight, in statically indexed registers: the block
    // loop is unrolled so that no register is copied while its load is still outstanding.  Everything
    // inside the loop is a per-lane base plus a running offset: no multiplications, divisions or
    // modulo by the (runtime) number of stages.
    constexpr int kAhead = (B >= 6) ? 3 : (PW == 16 ? 4 : 6);
    const uint32_t *wnext = p.w + (static_cast<size_t>(valid ? tile16 : 0) * p.kblocks + kb_lo) * BW;  // next block to load
    const uint16_t *snext = p.s + (static_cast<size_t>(valid ? tile16 : 0) * groups + ((GS == -1) ? 0 : kb_lo * NG)) * 16 + g;
    uint32_t wq[kAhead][2 * B];
    // raw scales of rows g and g+8, loaded with the block's words and only touched when the block is decoded
    // (dense_scale() applied on arrival would stall the warp on the load it has just issued)
    uint16_t sq_lo[kAhead][NG], sq_hi[kAhead][NG];
    auto load_next = [&](uint32_t (&wdst)[2 * B], uint16_t (&lo)[NG], uint16_t (&hi)[NG]) {
      load_block<B>(wnext, lane, wdst);
#pragma unroll
      for (int j = 0; j < NG; ++j) {
        lo[j] = ldg_u16_tc(snext + j * 16);
        hi[j] = ldg_u16_tc(snext + j * 16 + 8);
      }
      wnext += BW;
      if (GS != -1) snext += NG * 16;
    };
#pragma unroll
    for (int a = 0; a < kAhead; ++a)
      if (valid && a < nblk) load_next(wq[a], sq_lo[a], sq_hi[a]);

    // this lane's 16 bytes of rows g and g+8 in the A tile of stage 0, chunk t (shared-memory address)
    const uint32_t a_lane = base_u32 + plan.off_stages + plan.b_stage_bytes + t * kTcChunkStride + (2 * ptile) * 128 + g * 16;
    const uint32_t stages8 = static_cast<uint32_t>(stages) * 8;
    TcProducer pr;  // the stage the next half block goes to, and what does not change
    pr.off = 0;
    pr.idx8 = 0;
    pr.parity = 1;
    pr.stage_bytes = plan.stage_bytes;
    pr.stages8 = stages8;
    pr.bar_full = bar_full;
    pr.bar_empty = bar_empty;
    pr.a_lane = a_lane;
    for (int blk = 0; blk < nblk && !failed; blk += kAhead) {
#pragma unroll
      for (int a = 0; a < kAhead; ++a) {
        if (blk + a < nblk && !failed) {
          if (!tc_producer_half<B, GS, BF16, 0>(pr, PW == 8 || my_half == 0, valid, lane, wq[a], sq_lo[a], sq_hi[a]) ||
              !tc_producer_half<B, GS, BF16, 1>(pr, PW == 8 || my_half == 1, valid, lane, wq[a], sq_lo[a], sq_hi[a])) {
            failed = true;
          } else if (valid && blk + a + kAhead < nblk) {
            load_next(wq[a], sq_lo[a], sq_hi[a]);  // this block's registers are free: fetch the block kAhead ahead
          }
        }
      }
    }
    if (failed) report_status(kStatusMmaTimeout);
  } else if (warp == PW + 1 && lane == 0) {
    // ------------------------------------------------------------------ activation tiles
    // Iteration j needs rows m0.. and in-features (kb_lo*128 + 64 j ..+64) in the B part of its stage; each tile is
    // requested as soon as the tensor pipe has released the stage, so the requests run the whole ring ahead.
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may come from the kernel launched just before
    const uint32_t ring_bytes = static_cast<uint32_t>(stages) * plan.stage_bytes;
    uint32_t rq_off = 0, rq_idx8 = 0, rq_parity = 1;
    int rq_x = kb_lo * 128;
    for (int j = 0; j < nit; ++j) {
      if (!mbar_wait(bar_empty + rq_idx8, rq_parity)) {
        failed = true;
        report_status(kStatusMmaTimeout);
        break;
      }
      mbar_arrive_expect_tx(bar_full + rq_idx8, plan.b_stage_bytes);
      tma_load_2d(base_u32 + plan.off_stages + rq_off, &xmap, rq_x, m0, bar_full + rq_idx8);
      rq_x += 64;
      rq_off += plan.stage_bytes;
      rq_idx8 += 8;
      if (rq_off == ring_bytes) {
        rq_off = 0;
        rq_idx8 = 0;
        rq_parity ^= 1;
      }
    }
  } else if (warp == PW) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop, so that addresses and descriptors are warp-uniform values, and one elected
    // lane issues.  One thread issues every MMA, so this loop is the pipeline's clock: the descriptors of stage 0 are built once
    // and a stage or a K step only adds to their address field (bits 0..13, in units of 16 bytes).
    const uint32_t idesc = umma_instr_desc(BF16 ? 1 : 0, p.ncols);
    const uint32_t ring16 = static_cast<uint32_t>(stages) * plan.stage_bytes >> 4, stage16 = plan.stage_bytes >> 4;
    const uint32_t stage0_b = base_u32 + plan.off_stages;
    const uint64_t da0 = umma_smem_desc(stage0_b + plan.b_stage_bytes, kTcChunkStride, 128, 0);
    const uint64_t db0 = umma_smem_desc(stage0_b, 16, 1024, 2);
    uint32_t st16 = 0, st_idx8 = 0, parity = 0, accumulate = 0;
    for (int it = 0; it < nit; ++it) {
      if (!mbar_wait(bar_full + st_idx8, parity)) {
        failed = true;
        report_status(kStatusWeightCopyTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t da = da0 + st16, db = db0 + st16;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base, da + static_cast<uint64_t>(k * (2 * kTcChunkStride / 16)), db + static_cast<uint64_t>(k * 2), idesc,
                   (k > 0) ? 1u : accumulate);
        umma_commit(bar_empty + st_idx8);
      }
      accumulate = 1;
      __syncwarp();
      st16 += stage16;
      st_idx8 += 8;
      if (st16 == ring16) {
        st16 = 0;
        st_idx8 = 0;
        parity ^= 1;
      }
    }
    if (!failed && elect_one()) umma_commit(bar_done);
    __syncwarp();
  }

  // ---------------------------------------------------------------------- epilogue
  if (warp < PW) asm volatile("griddepcontrol.wait;" ::: "memory");  // nothing is written before the previous kernel is done
  if (warp < PW && !failed) {
    if (!mbar_wait(bar_done, 0)) {
      failed = true;
      report_status(kStatusMmaTimeout);
    }
  }
  // the pipeline's stages are free once every MMA is done; with K split they hold this CTA's fp32 partial sums
  float *staging = reinterpret_cast<float *>(base + plan.off_stages);
  if (warp < PW && !failed) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int q = warp & 3;
    const int n = tile128 * 128 + q * 32 + lane;
    const int nchunks = p.ncols / 16;
    for (int ci = (warp >> 2); ci < nchunks; ci += PW / 4) {
      uint32_t v[16];
      tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ci * 16, v);
      if (p.split > 1 && p.partial == nullptr) {
        // this CTA's share of the sum over K: staging[batch row][out-feature of the tile], fp32
#pragma unroll
        for (int j = 0; j < 16; ++j) staging[(ci * 16 + j) * 128 + q * 32 + lane] = __uint_as_float(v[j]);
      } else if (p.split > 1) {
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + ci * 16 + j;
            if (m < m0 + mrows) p.partial[(static_cast<size_t>(sk) * p.M + m) * p.N + n] = __uint_as_float(v[j]);
          }
        }
      } else if (n < p.N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + ci * 16 + j;
          if (m < m0 + mrows) p.y[static_cast<size_t>(m) * p.ldy + n] = to_out16<BF16>(__uint_as_float(v[j]));
        }
      }
    }
  }
  if (p.split > 1 && p.partial == nullptr) {
    // The CTAs that share a tile form one cluster along K.  Each adds, in the order of the K ranges, the batch
    // rows it owns from every CTA's staging area through distributed shared memory, and stores them.
    __syncwarp();
    cluster_sync_all();
    if (warp < PW) {
      const int per = (p.ncols + p.split - 1) / p.split;
      const int c_lo = sk * per, c_hi = min(c_lo + per, p.ncols);
      // Four out-features of one batch row per thread and step, two CTAs' values in flight at a time.  Measured on
      // B200: scalar loads one after the other cost gate/up at 128 rows (two CTAs along K, 64 batch rows each) 9 us
      // in this loop; with all of a thread's loads in flight at once that drops to 4 us, but clusters of eight then
      // lose ~1 us (q/o, k/v at 32 rows), so the loads go out in pairs.
      for (int idx = tid; idx < (c_hi - c_lo) * 32; idx += PW * 32) {
        const int c = c_lo + (idx >> 5), nn = (idx & 31) * 4;
        const int m = m0 + c, n = tile128 * 128 + nn;
        if (m < m0 + mrows && n < p.N) {
          const uint32_t local = smem_u32(staging + c * 128 + nn);
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s = 0; s < p.split; s += 2) {
            const float4 a = ld_cluster_f32x4(map_to_cta(local, s));
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s + 1 < p.split) b = ld_cluster_f32x4(map_to_cta(local, s + 1));
            sum.x = (sum.x + a.x) + b.x;
            sum.y = (sum.y + a.y) + b.y;
            sum.z = (sum.z + a.z) + b.z;
            sum.w = (sum.w + a.w) + b.w;
          }
          uint16_t *dst = p.y + static_cast<size_t>(m) * p.ldy + n;
          const uint16_t o0 = to_out16<BF16>(sum.x), o1 = to_out16<BF16>(sum.y), o2 = to_out16<BF16>(sum.z),
                         o3 = to_out16<BF16>(sum.w);
          if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
            *reinterpret_cast<uint2 *>(dst) = make_uint2(o0 | (static_cast<uint32_t>(o1) << 16), o2 | (static_cast<uint32_t>(o3) << 16));
          } else {
            dst[0] = o0;
            if (n + 1 < p.N) dst[1] = o1;
            if (n + 2 < p.N) dst[2] = o2;
            if (n + 3 < p.N) dst[3] = o3;
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();  // nobody leaves while its staging area is still being read
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == PW) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

template <int B, int GS, bool BF16, int PW>
__global__ void __launch_bounds__((PW + 2) * 32, PW == 8 ? 2 : 1) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
  gemm_tc_body<B, GS, BF16, PW>(p, xmap, static_cast<int>(blockIdx.x));
}

// partial[split][M][N] fp32 -> y[M][N] (rows ldy elements apart), added in the order of the K ranges: the second
// kernel of a K split that goes through scratch memory
template <bool BF16>
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, uint16_t *__restrict__ y, long long mn, int split,
                                     int n_cols, int ldy) {
  // launched with programmatic stream serialization right behind the kernel that writes `partial`
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < mn;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < split; ++s) sum += partial[static_cast<long long>(s) * mn + i];
    const long long m = i / n_cols;
    y[m * ldy + (i - m * n_cols)] = to_out16<BF16>(sum);
  }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static int round_up16(int v) { return (v + 15) / 16 * 16; }

// Up to 128 batch rows the kernel is bound by its producer warps (eight per CTA), so two CTAs share an SM
// whenever three pipeline stages of each fit in half of the SM's shared memory.  Measured on B200: two stages
// are too shallow (256 batch rows: 45 us with one CTA and four stages, 53 us with two CTAs and two stages); a
// CTA that has the SM to itself runs sixteen producer warps instead (gate/up at 256 rows: 37.9 -> 35.3 us).
constexpr int kTcHalfSmBytes = 112 * 1024;
static bool tc_two_ctas_per_sm(int ncols) { return tc_plan(ncols, 3).total <= kTcHalfSmBytes; }

// K split of the tensor-core path: one wave of CTAs over the SMs' slots; at least four blocks of K per CTA.
int gemm_tc_pick_split(int N, int K, int M, int sm_count) {
  const int ctas = ((N + 127) / 128) * ((M + 255) / 256);
  const int kblocks = K / 128;
  const int want = tc_two_ctas_per_sm(round_up16(M < 256 ? M : 256)) ? 2 * sm_count : sm_count;
  int split = 1;
  while (split < 8 && ctas * (split + 1) <= want && kblocks / (split + 1) >= 4) ++split;  // one wave
  return split;
}

// Scratch for a K split that goes through global memory (scratch_reduce, or a device that cannot place the cluster).
long long gemm_tc_workspace_bytes(int N, int K, int M, int sm_count) {
  const int split = gemm_tc_pick_split(N, K, M, sm_count);
  return split > 1 ? static_cast<long long>(split) * M * N * 4 : 0;
}

// Tensor map of the activations x[M, K] (two-byte elements, row-major) with boxes of 64 in-features x `box_rows`
// batch rows and the 128-byte swizzle the UMMA descriptor of the B operand expects; rows past M read as zeros.
static int make_x_tensor_map(CUtensorMap *map, const void *x, int M, int K, int box_rows) {
  typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  // looked up once; the initialisation of a function-local static is thread-safe
  static const EncodeTiled encode = []() -> EncodeTiled {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    return reinterpret_cast<EncodeTiled>(fn);
  }();
  if (!encode) return MG_ERR_CUDA;
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estride[2] = {1u, 1u};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(x), gdim, gstride, box, estride,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MG_OK : MG_ERR_CUDA;
}

// As many pipeline stages as fit: in half of the SM's shared memory with 8 producer warps (two CTAs per SM), in
// all of it with 16.
static int tc_pick_stages(int ncols, int producer_warps) {
  int stages = 8;
  if (producer_warps == 8) {
    while (stages > 3 && tc_plan(ncols, stages).total > kTcHalfSmBytes) --stages;
  } else {
    while (stages > 2 && tc_plan(ncols, stages).total > 2 * kTcHalfSmBytes) --stages;
  }
  return stages;
}

template <int B, int GS, bool BF16, int PW>
static int launch_gemm_tc_warps(GemmParams p, cudaStream_t stream, bool pdl, float *fallback_partial) {
  auto kernel = gemm_tc_kernel<B, GS, BF16, PW>;
  CUtensorMap xmap;
  if (make_x_tensor_map(&xmap, p.x, p.M, p.K, p.ncols) != MG_OK) return MG_ERR_CUDA;
  const int stages = tc_pick_stages(p.ncols, PW);
  p.stages = stages;
  const TcPlan plan = tc_plan(p.ncols, stages);
  static SharedMemoryOptIn opt_in;  // one per instantiation of this launcher
  {
    const int st = opt_in.ensure(kernel, 224 * 1024);
    if (st != MG_OK) return st;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + 127) / 128, p.split, (p.M + 255) / 256);
  cfg.blockDim = dim3((PW + 2) * 32, 1, 1);
  cfg.dynamicSmemBytes = plan.total;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.split > 1 && p.partial == nullptr) {  // the CTAs along K form a cluster and add their sums through distributed shared memory
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = static_cast<unsigned>(p.split);
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, kernel, p, xmap) != cudaSuccess) {
    if (p.split > 1 && p.partial == nullptr && fallback_partial != nullptr) {
      // the device could not place the cluster (a partitioned GPU, say): go through the caller's scratch instead
      (void)cudaGetLastError();
      p.partial = fallback_partial;
      cfg.numAttrs = pdl ? 1 : 0;
      if (cudaLaunchKernelEx(&cfg, kernel, p, xmap) != cudaSuccess) return MG_ERR_CUDA;
    } else {
      return MG_ERR_CUDA;
    }
  }
  if (p.split > 1 && p.partial != nullptr) {
    const long long mn = static_cast<long long>(p.M) * p.N;
    long long blocks = (mn + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaLaunchConfig_t rcfg = {};
    rcfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    rcfg.blockDim = dim3(256, 1, 1);
    rcfg.stream = stream;
    cudaLaunchAttribute rattr[1];
    rattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    rattr[0].val.programmaticStreamSerializationAllowed = 1;
    rcfg.attrs = rattr;
    rcfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&rcfg, splitk_reduce_kernel<BF16>, static_cast<const float *>(p.partial), p.y, mn, p.split, p.N, p.ldy) != cudaSuccess)
      return MG_ERR_CUDA;
  }
  return MG_OK;
}

// Sixteen producer warps when the CTA has its SM to itself: the stages are too large for two CTAs per SM, or there
// are no more CTAs than SMs.
template <int B, int GS, bool BF16>
static int launch_gemm_tc(GemmParams p, cudaStream_t stream, bool pdl, float *fallback_partial) {
  p.ncols = round_up16(p.M < 256 ? p.M : 256);
  int sm_count = 0;
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  const long long ctas = static_cast<long long>((p.N + 127) / 128) * p.split * ((p.M + 255) / 256);
  if (!tc_two_ctas_per_sm(p.ncols) || ctas <= sm_count) return launch_gemm_tc_warps<B, GS, BF16, 16>(p, stream, pdl, fallback_partial);
  return launch_gemm_tc_warps<B, GS, BF16, 8>(p, stream, pdl, fallback_partial);
}

template <int B, int GS>
static int launch_gemm_tc_type(const GemmParams &p, bool bf16, cudaStream_t stream, bool pdl, float *fb) {
  if (bf16) return launch_gemm_tc<B, GS, true>(p, stream, pdl, fb);
  return launch_gemm_tc<B, GS, false>(p, stream, pdl, fb);
}

template <int B>
static int launch_gemm_tc_group(const GemmParams &p, int group_size, bool bf16, cudaStream_t stream, bool pdl, float *fb) {
  switch (group_size) {
    case -1: return launch_gemm_tc_type<B, -1>(p, bf16, stream, pdl, fb);
    case 32: return launch_gemm_tc_type<B, 32>(p, bf16, stream, pdl, fb);
    case 128: return launch_gemm_tc_type<B, 128>(p, bf16, stream, pdl, fb);
    default: return MG_ERR_BAD_ARG;
  }
}

// workspace: fp32 scratch of at least gemm_tc_workspace_bytes() or null.  The sums of a split K meet inside a
// thread-block cluster; the scratch is used when scratch_reduce asks for it, or when the cluster cannot be launched.
int gemm_tc_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                   void *y, void *workspace, long long workspace_bytes, bool bf16, bool pdl, int split_override,
                   cudaStream_t stream, int ldy, bool scratch_reduce) {
  int sm_count = 0;  // of the current device
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  GemmParams p;
  p.w = static_cast<const uint32_t *>(w);
  p.s = static_cast<const uint16_t *>(s);
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.N = N;
  p.K = K;
  p.M = M;
  p.ldy = ldy > 0 ? ldy : N;
  p.kblocks = K / 128;
  int split = split_override > 0 ? split_override : gemm_tc_pick_split(N, K, M, sm_count);
  if (split > p.kblocks) split = p.kblocks;
  if (split > 8) return MG_ERR_BAD_ARG;  // the CTAs along K form one cluster
  const bool have_scratch = workspace != nullptr && workspace_bytes >= static_cast<long long>(split) * M * N * 4;
  if (scratch_reduce && split > 1 && !have_scratch) return MG_ERR_BAD_ARG;
  p.partial = (scratch_reduce && split > 1) ? static_cast<float *>(workspace) : nullptr;
  float *fb = (split > 1 && have_scratch) ? static_cast<float *>(workspace) : nullptr;
  p.split = split;
  p.ncols = 0;
  p.stages = 0;
  switch (bitwidth) {
    case 2: return launch_gemm_tc_group<2>(p, group_size, bf16, stream, pdl, fb);
    case 3: return launch_gemm_tc_group<3>(p, group_size, bf16, stream, pdl, fb);
    case 4: return launch_gemm_tc_group<4>(p, group_size, bf16, stream, pdl, fb);
    case 6: return launch_gemm_tc_group<6>(p, group_size, bf16, stream, pdl, fb);
    case 8: return launch_gemm_tc_group<8>(p, group_size, bf16, stream, pdl, fb);
    default: return MG_ERR_BAD_ARG;
  }
}

MG_DEFINE_STATUS_ACCESSOR(gemm_tc_device_status)

}  // namespace mg
