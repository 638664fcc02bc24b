// Internal declarations shared by the translation units of libmatgptq_b200.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

// status codes returned through the C ABI (see include/matgptq_b200.h)
#define MG_OK 0
#define MG_ERR_BAD_ARG 1
#define MG_ERR_CUDA 2
#define MG_ERR_UNSUPPORTED 3
#define MG_ERR_ALIGNMENT 4

namespace mg {

// gemv.cu
// z must be null for gemv_launch and non-null for gemv_zp_launch (gemv_zp.cu: the same kernels with zero points)
int gemv_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *z,
                const void *x, void *y, bool bf16, bool pdl, int R_override, int S_override, cudaStream_t stream,
                int ldy = 0);
int gemv_zp_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *z,
                   const void *x, void *y, bool bf16, bool pdl, int R_override, int S_override, cudaStream_t stream,
                   int ldy = 0);

// Row-parallel product fused with its all-reduce over peer memory (gemv.cu).  Every rank runs the same launch on
// its K shard.  In the epilogue every thread stores each of its fp32 partial sums, paired with the epoch of the
// call in ONE 8-byte store, into this rank's slot on every other rank (plain stores to peer memory), then reads
// the other ranks' values of the same outputs from its own memory, polling each 8-byte word until it carries
// the epoch (bounded), and adds them in rank order: every rank computes the same bits.  Value and flag travel
// together, so no fence and no second round trip is needed.  Two slot sets alternate by epoch parity and epochs
// only grow, so nothing is ever reset.
constexpr int kArMaxRanks = 8;
struct ArParams {
  uint2 *data[kArMaxRanks];  // rank q's buffer: [2][nranks][slot_elems] of {value bits, epoch}
  unsigned *ctrl;            // local: [0] epoch of the last finished reduction, [1] CTA tickets
  long long slot_elems;      // elements of one slot (>= M * N)
  int rank, nranks;
  int push_only;             // 1: store only (also into the own slot); matgptq_b200_allreduce_finish adds up (single-GPU emulation of ranks)
};
constexpr int kStatusPeerTimeout = 105;
int gemv_allreduce_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                          void *y, bool bf16, bool pdl, const ArParams &ar, cudaStream_t stream);
int allreduce_finish_launch(const ArParams &ar, void *y, int N, int M, bool bf16, cudaStream_t stream);

// Grouped launch (gemv.cu): nseg products over the same activations, outputs side by side in y[M, ldy].
// MG_ERR_UNSUPPORTED (nothing launched) when the segments cannot share one launch shape.
struct GroupedSegment {
  const void *w;
  const void *s;
  int n_out;
  int bitwidth;
};
int gemv_grouped_launch(const GroupedSegment *segments, int nseg, int group_size, int K, int M, const void *x, void *y,
                        int ldy, bool bf16, bool pdl, cudaStream_t stream);

int gemv_device_status(int *status_out, int reset);
int gemv_zp_device_status(int *status_out, int reset);

// gemm_tc.cu
int gemm_tc_pick_split(int N, int K, int M, int sm_count);
long long gemm_tc_workspace_bytes(int N, int K, int M, int sm_count);
int gemm_tc_launch(int bitwidth, int group_size, int N, int K, int M, const void *w, const void *s, const void *x,
                   void *y, void *workspace, long long workspace_bytes, bool bf16, bool pdl, int split_override,
                   cudaStream_t stream, int ldy = 0, bool scratch_reduce = false);
int gemm_tc_device_status(int *status_out, int reset);

// selftest.cu
int selftest_device_status(int *status_out, int reset);

// pack.cu
int slice_launch(const uint8_t *in, uint8_t *out, long long numel, int master_bitwidth, int bitwidth,
                 cudaStream_t stream);
int pack_launch(const uint8_t *codes, uint32_t *packed, int N, int K, int bitwidth, int slice_from_master,
                cudaStream_t stream);
int pack_host(const uint8_t *codes, uint32_t *packed, int N, int K, int bitwidth, int slice_from_master);
int unpack_host(const uint32_t *packed, uint8_t *codes, int N, int K, int bitwidth);
int reorder_scales_launch(const uint16_t *in, uint16_t *out, int N, int K, int group_size, cudaStream_t stream);
int reorder_scales_host(const uint16_t *in, uint16_t *out, int N, int K, int group_size);

// dequant.cu
int dequant_launch(const uint32_t *packed, const uint16_t *scales, const uint16_t *zeros, uint16_t *w_out, int N,
                   int K, int bitwidth, int group_size, bool bf16, cudaStream_t stream);

}  // namespace mg
