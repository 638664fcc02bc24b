// Tensor-core path for batches of 32 rows and more: tcgen05.mma with the accumulator
// in tensor memory.
//
// Replaces gptq_matryoshka for large batches (csrc/matgptq_gemm.cu:337-634), which
// re-reads the weights once per 8 batch columns and stays below a dense fp16 GEMM
// from M = 32 up.  Here one CTA owns 128 out-features and up to 256 batch rows:
//
//   * eight "dequant" warps (one per 16-row tile of the packed layout) decode their
//     block to the exact dense weights of the reference's dequantize()
//     (round(scale * (code*2^(8-b) - 128)), fp16 or bf16) and store them K-major into a
//     shared-memory stage in the canonical no-swizzle UMMA layout (8 x 16-byte core
//     matrices), with the packed words of the next two or three blocks already in flight;
//   * one thread of a ninth warp fetches the activation tiles (batch rows x 64 in-features) with TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle, rows past the batch filled with zeros), as far ahead as
//     the pipeline has stages, and issues tcgen05.mma (M = 128 weight rows, N = batch rows, K = 16)
//     from shared-memory descriptors; D[128, N] lives in tensor memory; completion of a stage's MMAs
//     releases the stage through tcgen05.commit -> mbarrier;
//   * the epilogue reads D with tcgen05.ld (each warp its own 32 TMEM lanes), converts
//     and stores y[m, n] (the transpose of D), or, when K is split over several CTAs,
//     stores fp32 partial sums into caller-provided scratch memory that a second small
//     kernel adds up in a fixed order.
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
constexpr int kTcThreads = 9 * 32;  // 8 producer warps and the MMA issuer

struct GemmParams {
  const uint32_t *w;
  const uint16_t *s;
  const uint16_t *x;
  uint16_t *y;
  float *partial;  // [split][M][N] fp32 when split > 1
  int N, K, M;
  int ldy;      // elements between two rows of y (N unless the call writes a column block of a wider output)
  int kblocks;  // K / 128
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

// scale groups per 128-wide block
template <int GS> struct TcScales {
  static constexpr int NG = (GS == 32) ? 4 : 1;
};

template <int B, int GS, bool BF16>
__global__ void __launch_bounds__(kTcThreads, 2) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
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

  const int tile128 = blockIdx.x, sk = blockIdx.y;
  const int m0 = blockIdx.z * 256;
  const int mrows = min(p.M - m0, 256);
  const int kb_lo = sk * p.kblocks / p.split;
  const int kb_hi = (sk + 1) * p.kblocks / p.split;
  const int nblk = kb_hi - kb_lo;
  const int nit = 2 * nblk;  // pipeline iterations of 64 in-features
  const int groups = (GS == -1) ? 1 : p.K / GS;
  int tmem_cols = 32;
  while (tmem_cols < p.ncols) tmem_cols <<= 1;

  if (warp == 8) {
    if (lane == 0) {
      for (int i = 0; i < stages; ++i) {
        mbar_init(bar_full + i * 8, 9);  // the eight producer warps and the thread that requests the activations
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

  // The activations may come from the kernel launched just before this one.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  bool failed = false;
  if (warp < 8) {
    // ------------------------------------------------------------------ producers
    const int tile16 = tile128 * 8 + warp;
    const bool valid = tile16 < p.N / 16;
    constexpr int BW = BlockTraits<B>::WORDS;
    constexpr int NG = TcScales<GS>::NG;
    // Packed words and scales of two or three blocks in flight, in statically indexed registers: the block
    // loop is unrolled so that no register is copied while its load is still outstanding.  Everything
    // inside the loop is a per-lane base plus a running offset: no multiplications, divisions or
    // modulo by the (runtime) number of stages.
    constexpr int kAhead = (B >= 6) ? 2 : 3;
    const uint32_t *wnext = p.w + (static_cast<size_t>(valid ? tile16 : 0) * p.kblocks + kb_lo) * BW;  // next block to load
    const uint16_t *snext = p.s + (static_cast<size_t>(valid ? tile16 : 0) * groups + ((GS == -1) ? 0 : kb_lo * NG)) * 16 + g;
    uint32_t wq[kAhead][2 * B];
    uint32_t sq_lo[kAhead][NG], sq_hi[kAhead][NG];  // dense_scale() of the scales of rows g and g+8
    auto load_next = [&](uint32_t (&wdst)[2 * B], uint32_t (&lo)[NG], uint32_t (&hi)[NG]) {
      load_block<B>(wnext, lane, wdst);
#pragma unroll
      for (int j = 0; j < NG; ++j) {
        lo[j] = dense_scale<B, BF16>(__ldg(snext + j * 16));
        hi[j] = dense_scale<B, BF16>(__ldg(snext + j * 16 + 8));
      }
      wnext += BW;
      if (GS != -1) snext += NG * 16;
    };
#pragma unroll
    for (int a = 0; a < kAhead; ++a)
      if (valid && a < nblk) load_next(wq[a], sq_lo[a], sq_hi[a]);

    const uint32_t ring_bytes = static_cast<uint32_t>(stages) * plan.stage_bytes;
    // this lane's 16 bytes of rows g and g+8 in the A tile of stage 0, chunk t
    unsigned char *a_lane = base + plan.off_stages + plan.b_stage_bytes + t * kTcChunkStride + (2 * warp) * 128 + g * 16;
    uint32_t cur_stage_off = 0, cur_bar = bar_full, cur_empty = bar_empty, cur_parity = 1;
    int blocks_left = nblk, loads_left = nblk - kAhead;
    while (blocks_left > 0 && !failed) {
#pragma unroll
      for (int a = 0; a < kAhead; ++a) {
        if (blocks_left > 0 && !failed) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(cur_empty, cur_parity)) {  // the tensor pipe is done with what this stage held
              failed = true;
              break;
            }
            if (valid) {
              // dense weights of this lane: rows g and g+8, two 16-byte chunks per row
#pragma unroll
              for (int jj = 2 * h; jj < 2 * h + 2; ++jj) {
                const int gi = (GS == 32) ? jj : 0;
                uint4 lo, hi;
                lo.x = dense_pair<B, BF16>(wq[a], 8 * jj + 0, sq_lo[a][gi]);
                lo.y = dense_pair<B, BF16>(wq[a], 8 * jj + 2, sq_lo[a][gi]);
                lo.z = dense_pair<B, BF16>(wq[a], 8 * jj + 4, sq_lo[a][gi]);
                lo.w = dense_pair<B, BF16>(wq[a], 8 * jj + 6, sq_lo[a][gi]);
                hi.x = dense_pair<B, BF16>(wq[a], 8 * jj + 1, sq_hi[a][gi]);
                hi.y = dense_pair<B, BF16>(wq[a], 8 * jj + 3, sq_hi[a][gi]);
                hi.z = dense_pair<B, BF16>(wq[a], 8 * jj + 5, sq_hi[a][gi]);
                hi.w = dense_pair<B, BF16>(wq[a], 8 * jj + 7, sq_hi[a][gi]);
                unsigned char *dst = a_lane + cur_stage_off + (jj & 1) * (4 * kTcChunkStride);
                *reinterpret_cast<uint4 *>(dst) = lo;
                *reinterpret_cast<uint4 *>(dst + 128) = hi;
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor pipe reads
            __syncwarp();
            if (lane == 0) mbar_arrive(cur_bar);
            cur_stage_off += plan.stage_bytes;
            cur_bar += 8;
            cur_empty += 8;
            if (cur_stage_off == ring_bytes) {
              cur_stage_off = 0;
              cur_bar = bar_full;
              cur_empty = bar_empty;
              cur_parity ^= 1;
            }
          }
          // this block's registers are free: fetch the block kAhead ahead
          if (valid && loads_left > 0) load_next(wq[a], sq_lo[a], sq_hi[a]);
          --loads_left;
          --blocks_left;
        }
      }
    }
    if (failed) report_status(kStatusMmaTimeout);
  } else if (warp == 8 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = umma_instr_desc(BF16 ? 1 : 0, p.ncols);
    uint32_t st_off = 0, st_idx8 = 0, parity = 0;
    const uint32_t ring_bytes = static_cast<uint32_t>(stages) * plan.stage_bytes;
    // Activation tiles: iteration j needs rows m0.. and in-features (kb_lo*128 + 64 j ..+64) in the B part of its
    // stage.  They are requested a few iterations ahead, each after the stage has been released.
    uint32_t rq_off = 0, rq_idx8 = 0, rq_parity = 1;
    int rq_x = kb_lo * 128, rq_left = nit;
    auto request_x = [&]() -> bool {
      if (rq_left <= 0) return true;
      if (!mbar_wait(bar_empty + rq_idx8, rq_parity)) return false;
      mbar_arrive_expect_tx(bar_full + rq_idx8, plan.b_stage_bytes);
      tma_load_2d(base_u32 + plan.off_stages + rq_off, &xmap, rq_x, m0, bar_full + rq_idx8);
      rq_x += 64;
      --rq_left;
      rq_off += plan.stage_bytes;
      rq_idx8 += 8;
      if (rq_off == ring_bytes) {
        rq_off = 0;
        rq_idx8 = 0;
        rq_parity ^= 1;
      }
      return true;
    };
    // two stages short of the ring, so that the wait inside request_x() is for MMAs issued two iterations ago
    const int ahead = stages > 3 ? stages - 2 : 1;
    for (int j = 0; j < ahead; ++j)
      if (!request_x()) failed = true;
    for (int it = 0; it < nit && !failed; ++it) {
      if (!request_x()) {
        failed = true;
        report_status(kStatusMmaTimeout);
        break;
      }
      if (!mbar_wait(bar_full + st_idx8, parity)) {
        failed = true;
        report_status(kStatusWeightCopyTimeout);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t stage_b = base_u32 + plan.off_stages + st_off;
      const uint32_t stage_a = stage_b + plan.b_stage_bytes;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t da = umma_smem_desc(stage_a + 2 * k * kTcChunkStride, kTcChunkStride, 128, 0);
        const uint64_t db = umma_smem_desc(stage_b + k * 32, 16, 1024, 2);
        umma_f16(tmem_base, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(bar_empty + st_idx8);
      st_off += plan.stage_bytes;
      st_idx8 += 8;
      if (st_off == ring_bytes) {
        st_off = 0;
        st_idx8 = 0;
        parity ^= 1;
      }
    }
    if (!failed) umma_commit(bar_done);
  }

  // ---------------------------------------------------------------------- epilogue
  if (warp < 8 && !failed) {
    if (!mbar_wait(bar_done, 0)) {
      failed = true;
      report_status(kStatusMmaTimeout);
    }
  }
  if (warp < 8 && !failed) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int q = warp & 3;
    const int n = tile128 * 128 + q * 32 + lane;
    const int nchunks = p.ncols / 16;
    for (int ci = (warp >> 2); ci < nchunks; ci += 2) {
      uint32_t v[16];
      tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ci * 16, v);
      if (n < p.N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + ci * 16 + j;
          if (m < m0 + mrows) {
            const float f = __uint_as_float(v[j]);
            if (p.split > 1) {
              p.partial[(static_cast<size_t>(sk) * p.M + m) * p.N + n] = f;
            } else if (BF16) {
              p.y[static_cast<size_t>(m) * p.ldy + n] = __bfloat16_as_ushort(__float2bfloat16_rn(f));
            } else {
              p.y[static_cast<size_t>(m) * p.ldy + n] = __half_as_ushort(__float2half_rn(f));
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 8) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// partial[split][M][N] fp32 -> y[M][N] (rows ldy elements apart), added in a fixed order
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
    y[m * ldy + (i - m * n_cols)] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(sum)) : __half_as_ushort(__float2half_rn(sum));
  }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static int round_up16(int v) { return (v + 15) / 16 * 16; }

// Up to 128 batch rows the kernel is bound by its producer warps (eight per CTA), so two CTAs share an SM
// whenever three pipeline stages of each fit in half of the SM's shared memory.  Measured on B200: two stages
// are too shallow (256 batch rows: 45 us with one CTA and four stages, 53 us with two CTAs and two stages),
// and at 256 rows sixteen producer warps in one CTA change nothing (the tensor pipe of the 112 to 128 SMs
// that have a tile is then the limit).
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

template <int B, int GS, bool BF16>
static int launch_gemm_tc(GemmParams p, cudaStream_t stream, bool pdl) {
  auto kernel = gemm_tc_kernel<B, GS, BF16>;
  p.ncols = round_up16(p.M < 256 ? p.M : 256);
  CUtensorMap xmap;
  if (make_x_tensor_map(&xmap, p.x, p.M, p.K, p.ncols) != MG_OK) return MG_ERR_CUDA;
  int stages = 8;
  if (tc_two_ctas_per_sm(p.ncols)) {
    while (stages > 3 && tc_plan(p.ncols, stages).total > kTcHalfSmBytes) --stages;
  } else {
    while (stages > 2 && tc_plan(p.ncols, stages).total > 2 * kTcHalfSmBytes) --stages;
  }
  p.stages = stages;
  const TcPlan plan = tc_plan(p.ncols, stages);
  static SharedMemoryOptIn opt_in;  // one per instantiation of this launcher
  {
    const int st = opt_in.ensure(kernel, 224 * 1024);
    if (st != MG_OK) return st;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + 127) / 128, p.split, (p.M + 255) / 256);
  cfg.blockDim = dim3(kTcThreads, 1, 1);
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
  if (cudaLaunchKernelEx(&cfg, kernel, p, xmap) != cudaSuccess) return MG_ERR_CUDA;
  if (p.split > 1) {
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

template <int B, int GS>
static int launch_gemm_tc_type(const GemmParams &p, bool bf16, cudaStream_t stream, bool pdl) {
  if (bf16) return launch_gemm_tc<B, GS, true>(p, stream, pdl);
  return launch_gemm_tc<B, GS, false>(p, stream, pdl);
}

template <int B>
static int launch_gemm_tc_group(const GemmParams &p, int group_size, bool bf16, cudaStream_t stream, bool pdl) {
  switch (group_size) {
    case -1: return launch_gemm_tc_type<B, -1>(p, bf16, stream, pdl);
    case 32: return launch_gemm_tc_type<B, 32>(p, bf16, stream, pdl);
    case 128: return launch_gemm_tc_type<B, 128>(p, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

// workspace: fp32 scratch of at least gemm_tc_workspace_bytes(), or null to run without a K split
int gemm_tc_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                   void *y, void *workspace, long long workspace_bytes, bool bf16, bool pdl, int split_override,
                   cudaStream_t stream, int ldy) {
  int sm_count = 0;  // of the current device: the same value matgptq_b200_matmul_workspace_bytes sized the scratch with
  {
    const int st = current_device_sm_count(&sm_count);
    if (st != MG_OK) return st;
  }
  GemmParams p;
  p.w = static_cast<const uint32_t *>(w);
  p.s = static_cast<const uint16_t *>(s);
  p.x = static_cast<const uint16_t *>(x);
  p.y = static_cast<uint16_t *>(y);
  p.partial = static_cast<float *>(workspace);
  p.N = N;
  p.K = K;
  p.M = M;
  p.ldy = ldy > 0 ? ldy : N;
  p.kblocks = K / 128;
  int split = split_override > 0 ? split_override : gemm_tc_pick_split(N, K, M, sm_count);
  if (split > p.kblocks) split = p.kblocks;
  if (split > 1 && (workspace == nullptr || workspace_bytes < static_cast<long long>(split) * M * N * 4)) {
    if (split_override > 0) return MG_ERR_BAD_ARG;
    split = 1;  // no scratch given: every CTA runs the whole K range
  }
  p.split = split;
  p.ncols = 0;
  p.stages = 0;
  switch (bitwidth) {
    case 2: return launch_gemm_tc_group<2>(p, group_size, bf16, stream, pdl);
    case 3: return launch_gemm_tc_group<3>(p, group_size, bf16, stream, pdl);
    case 4: return launch_gemm_tc_group<4>(p, group_size, bf16, stream, pdl);
    case 6: return launch_gemm_tc_group<6>(p, group_size, bf16, stream, pdl);
    case 8: return launch_gemm_tc_group<8>(p, group_size, bf16, stream, pdl);
    default: return MG_ERR_BAD_ARG;
  }
}

MG_DEFINE_STATUS_ACCESSOR(gemm_tc_device_status)

}  // namespace mg
