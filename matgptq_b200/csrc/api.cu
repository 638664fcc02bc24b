// extern "C" entry points of libmatgptq_b200 (declared in include/matgptq_b200.h):
// argument checks, then one launch.  Checks mirror csrc/bindings.cpp:50-59,88-95,
// 153-168 of the reference; failures come back as status codes, never exit().
#include <cuda_runtime.h>

#include "../../include/matgptq_b200.h"
#include "kernels.h"

namespace {

bool valid_bitwidth(int64_t b) { return b == 2 || b == 3 || b == 4 || b == 6 || b == 8; }
bool valid_group(int64_t g) { return g == -1 || g == 32 || g == 128; }

int check_shape(int64_t n_out, int64_t n_in, int64_t bitwidth, int64_t group_size) {
  if (!valid_bitwidth(bitwidth) || !valid_group(group_size)) return MG_ERR_BAD_ARG;
  if (n_out <= 0 || n_in <= 0 || n_out > (1 << 24) || n_in > (1 << 24)) return MG_ERR_BAD_ARG;
  if (n_out % 16 != 0) return MG_ERR_BAD_ARG;
  if (n_in % 64 != 0) return MG_ERR_BAD_ARG;
  if (n_in % 128 != 0) return MG_ERR_UNSUPPORTED;  // the reference also takes K % 128 == 64
  if (group_size != -1 && n_in % group_size != 0) return MG_ERR_BAD_ARG;
  return MG_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

int matgptq_b200_version(void) { return 100; }

const char *matgptq_b200_strerror(int status) {
  switch (status) {
    case MG_OK: return "ok";
    case MG_ERR_BAD_ARG: return "bad argument (bitwidth must be 2,3,4,6,8; group size -1,32,128; N % 16 == 0; K % 64 == 0; non-null pointers)";
    case MG_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
    case MG_ERR_UNSUPPORTED:
      return "unsupported: K must be a multiple of 128, or the forced kernel does not take this shape or scratch size";
    case MG_ERR_ALIGNMENT: return "pointer is not 16-byte aligned";
    case MATGPTQ_B200_ERR_SCRATCH_TOO_SMALL:
      return "this shape needs more split-K scratch than the built-in array holds: pass scratch through matgptq_b200_matmul_ws";
    case MATGPTQ_B200_ERR_SCRATCH_UNAVAILABLE:
      return "the built-in scratch array could not be set up on this device (no memory left for it when first used?)";
    default: return "unknown status";
  }
}

// The row-parallel product with the fused all-reduce serves batches below this size (two passes of the GEMV from 17
// rows on); larger batches take the tensor-core path and a library all-reduce.
static const int64_t kTensorCoreMinBatch = 32;

// Automatic choice between the GEMV family and the tensor-core path.  The GEMV handles 16 activation rows per
// pass, so from 17 rows on it reads the weights twice (from L2) and doubles its tensor work, while the time of
// the tensor-core path hardly depends on the batch; measured on B200 (bf16, 4 bits, group 128, cold L2, GEMV
// against tensor cores in us): q/o 16 rows 8.0 / 7.8, 24 rows 14.1 / 8.4; gate/up 16 rows 14.7 / 18.1, 24 rows
// 26.9 / 19.9; down 16 rows 17.7 / 17.0, 24 rows 31.9 / 18.5.  Layers with few row tiles (k/v, N = 1024) are
// level at 24 rows (5.7 / 5.8) and better off on the tensor cores from 32 (6.5 / 5.9).
static bool uses_tensor_cores(int64_t n_out, int64_t batch) {
  if (n_out >= 2048) return batch > 16;
  return batch > 24;
}

static int sm_count_of_current_device(int *out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
  if (cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MG_ERR_CUDA;
  return MG_OK;
}

static int matmul_impl(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch, const void *w,
                       const void *s, const void *x, void *y, void *stream, uint32_t flags, void *workspace,
                       int64_t workspace_bytes, int path, int warps_per_cta, int split_k, const void *z = nullptr) {
  const int st = check_shape(n_out, n_in, bitwidth, group_size);
  if (st != MG_OK) return st;
  if (batch < 0 || batch > (1 << 24) || path < 0 || path > 2 || workspace_bytes < 0) return MG_ERR_BAD_ARG;
  if (batch == 0) return MG_OK;
  if (!w || !s || !x || !y) return MG_ERR_BAD_ARG;
  if (!aligned16(w) || !aligned16(x) || !aligned16(s) || !aligned16(z) || (reinterpret_cast<uintptr_t>(y) & 1u) ||
      (workspace && !aligned16(workspace)))
    return MG_ERR_ALIGNMENT;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const bool bf16 = (flags & MATGPTQ_B200_FLAG_BF16) != 0;
  const bool pdl = (flags & MATGPTQ_B200_FLAG_PDL) != 0;
  const bool tensor_core = path == 2 || (path == 0 && uses_tensor_cores(n_out, batch));
  int r;
  if (z) {
    // zero points: every batch size runs on the GEMV family (more than 16 rows in passes of 16); the tensor-core
    // path has the implicit zero point only
    if (path > 1) return MG_ERR_UNSUPPORTED;
    r = mg::gemv_zp_launch(static_cast<int>(bitwidth), static_cast<int>(group_size), static_cast<int>(n_out),
                           static_cast<int>(n_in), static_cast<int>(batch), w, s, z, x, y, bf16, pdl, warps_per_cta, split_k, cs);
  } else if (tensor_core) {
    r = mg::gemm_tc_launch(static_cast<int>(bitwidth), static_cast<int>(group_size), static_cast<int>(n_out),
                           static_cast<int>(n_in), static_cast<int>(batch), w, s, x, y, workspace, workspace_bytes, bf16,
                           pdl, split_k, cs, 0, (flags & MATGPTQ_B200_FLAG_SCRATCH_REDUCE) != 0);
  } else {
    r = mg::gemv_launch(static_cast<int>(bitwidth), static_cast<int>(group_size), static_cast<int>(n_out),
                        static_cast<int>(n_in), static_cast<int>(batch), w, s, nullptr, x, y, bf16, pdl, warps_per_cta, split_k, cs);
  }
  if (r != MG_OK) return r;
  if (!(flags & MATGPTQ_B200_FLAG_ASYNC)) {
    // the reference synchronises the whole device in this mode (csrc/matgptq_gemm.cu:1060-1062)
    if (cudaStreamSynchronize(cs) != cudaSuccess) return MG_ERR_CUDA;
  }
  return MG_OK;
}

int matgptq_b200_matmul_tuned(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                              const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                              int warps_per_cta, int split_k) {
  return matmul_impl(bitwidth, group_size, n_out, n_in, batch, w, s, x, y, stream, flags, nullptr, 0, 1, warps_per_cta,
                     split_k);
}

int matgptq_b200_matmul(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                        const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags) {
  return matmul_impl(bitwidth, group_size, n_out, n_in, batch, w, s, x, y, stream, flags, nullptr, 0, 0, 0, 0);
}

int matgptq_b200_matmul_zp(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                           const void *w, const void *s, const void *z, const void *x, void *y, void *stream,
                           uint32_t flags) {
  return matmul_impl(bitwidth, group_size, n_out, n_in, batch, w, s, x, y, stream, flags, nullptr, 0, 0, 0, 0, z);
}

int matgptq_b200_matmul_ws(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                           const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                           void *workspace, int64_t workspace_bytes, int path, int split_k) {
  return matmul_impl(bitwidth, group_size, n_out, n_in, batch, w, s, x, y, stream, flags, workspace, workspace_bytes, path,
                     0, split_k);
}

int matgptq_b200_matmul_grouped(const matgptq_b200_segment *segments, int n_segments, int64_t group_size, int64_t n_in,
                                int64_t batch, const void *x, void *y, void *stream, uint32_t flags, void *workspace,
                                int64_t workspace_bytes) {
  if (!segments || n_segments < 1 || n_segments > 8 || workspace_bytes < 0) return MG_ERR_BAD_ARG;
  int64_t total = 0;
  for (int i = 0; i < n_segments; ++i) {
    const int st = check_shape(segments[i].n_out, n_in, segments[i].bitwidth, group_size);
    if (st != MG_OK) return st;
    if (!segments[i].w || !segments[i].s) return MG_ERR_BAD_ARG;
    if (!aligned16(segments[i].w) || !aligned16(segments[i].s)) return MG_ERR_ALIGNMENT;
    total += segments[i].n_out;
  }
  if (batch < 0 || batch > (1 << 24) || total > (1 << 24)) return MG_ERR_BAD_ARG;
  if (batch == 0) return MG_OK;
  if (!x || !y) return MG_ERR_BAD_ARG;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 1u) || (workspace && !aligned16(workspace))) return MG_ERR_ALIGNMENT;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const bool bf16 = (flags & MATGPTQ_B200_FLAG_BF16) != 0;
  const bool pdl = (flags & MATGPTQ_B200_FLAG_PDL) != 0;
  int r = MG_ERR_UNSUPPORTED;
  mg::GroupedSegment segs[8];
  for (int i = 0; i < n_segments; ++i)
    segs[i] = mg::GroupedSegment{segments[i].w, segments[i].s, static_cast<int>(segments[i].n_out),
                                 static_cast<int>(segments[i].bitwidth)};
  if (batch <= 16) {  // one pass of the GEMV: all segments in one launch
    r = mg::gemv_grouped_launch(segs, n_segments, static_cast<int>(group_size), static_cast<int>(n_in),
                                static_cast<int>(batch), x, y, static_cast<int>(total), bf16, pdl, cs);
  }
  if (r == MG_ERR_UNSUPPORTED) {
    // One launch per segment into its column block: segments that cannot share a launch shape, and batches of more
    // than 16 rows, where each segment goes the way matgptq_b200_matmul would send it (a grouped launch of the
    // tensor-core path was measured: level with launches that overlap through programmatic dependent
    // launch up to 64 rows and at 256, 5 % ahead at 128 for gate and up of Llama-3.1-8B; not kept).
    int64_t col = 0;
    for (int i = 0; i < n_segments; ++i) {
      unsigned char *yi = static_cast<unsigned char *>(y) + col * 2;
      if (uses_tensor_cores(segments[i].n_out, batch))
        r = mg::gemm_tc_launch(static_cast<int>(segments[i].bitwidth), static_cast<int>(group_size),
                               static_cast<int>(segments[i].n_out), static_cast<int>(n_in), static_cast<int>(batch),
                               segments[i].w, segments[i].s, x, yi, workspace, workspace_bytes, bf16, pdl, 0, cs,
                               static_cast<int>(total), (flags & MATGPTQ_B200_FLAG_SCRATCH_REDUCE) != 0);
      else
        r = mg::gemv_launch(static_cast<int>(segments[i].bitwidth), static_cast<int>(group_size),
                            static_cast<int>(segments[i].n_out), static_cast<int>(n_in), static_cast<int>(batch),
                            segments[i].w, segments[i].s, nullptr, x, yi, bf16, pdl, 0, 0, cs, static_cast<int>(total));
      if (r != MG_OK) return r;
      col += segments[i].n_out;
    }
  }
  if (r != MG_OK) return r;
  if (!(flags & MATGPTQ_B200_FLAG_ASYNC)) {
    if (cudaStreamSynchronize(cs) != cudaSuccess) return MG_ERR_CUDA;
  }
  return MG_OK;
}

static int to_ar_params(const matgptq_b200_comm *comm, mg::ArParams *ar) {
  if (!comm || comm->nranks < 1 || comm->nranks > mg::kArMaxRanks || comm->rank < 0 || comm->rank >= comm->nranks ||
      !comm->ctrl || comm->slot_elems <= 0)
    return MG_ERR_BAD_ARG;
  for (int q = 0; q < comm->nranks; ++q) {
    if (!comm->data[q] || (reinterpret_cast<uintptr_t>(comm->data[q]) & 7u)) return MG_ERR_BAD_ARG;
    ar->data[q] = static_cast<uint2 *>(comm->data[q]);
  }
  ar->ctrl = static_cast<unsigned *>(comm->ctrl);
  ar->slot_elems = comm->slot_elems;
  ar->rank = comm->rank;
  ar->nranks = comm->nranks;
  ar->push_only = comm->push_only ? 1 : 0;
  return MG_OK;
}

int matgptq_b200_matmul_allreduce(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in_shard, int64_t batch,
                                  const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                                  const matgptq_b200_comm *comm) {
  const int st = check_shape(n_out, n_in_shard, bitwidth, group_size);
  if (st != MG_OK) return st;
  mg::ArParams ar = {};
  const int sc = to_ar_params(comm, &ar);
  if (sc != MG_OK) return sc;
  if (batch <= 0 || batch > (1 << 24) || !w || !s || !x || !y) return MG_ERR_BAD_ARG;
  if (!aligned16(w) || !aligned16(x) || !aligned16(s) || (reinterpret_cast<uintptr_t>(y) & 1u)) return MG_ERR_ALIGNMENT;
  if (batch >= kTensorCoreMinBatch) return MG_ERR_UNSUPPORTED;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int r = mg::gemv_allreduce_launch(static_cast<int>(bitwidth), static_cast<int>(group_size), static_cast<int>(n_out),
                                          static_cast<int>(n_in_shard), static_cast<int>(batch), w, s, x, y,
                                          (flags & MATGPTQ_B200_FLAG_BF16) != 0, (flags & MATGPTQ_B200_FLAG_PDL) != 0, ar, cs);
  if (r != MG_OK) return r;
  if (!(flags & MATGPTQ_B200_FLAG_ASYNC) && cudaStreamSynchronize(cs) != cudaSuccess) return MG_ERR_CUDA;
  return MG_OK;
}

int matgptq_b200_allreduce_finish(const matgptq_b200_comm *comm, void *y, int64_t n_out, int64_t batch, void *stream,
                                  uint32_t flags) {
  mg::ArParams ar = {};
  const int sc = to_ar_params(comm, &ar);
  if (sc != MG_OK) return sc;
  if (!y || n_out <= 0 || batch <= 0 || batch * n_out > comm->slot_elems) return MG_ERR_BAD_ARG;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int r = mg::allreduce_finish_launch(ar, y, static_cast<int>(n_out), static_cast<int>(batch),
                                            (flags & MATGPTQ_B200_FLAG_BF16) != 0, cs);
  if (r != MG_OK) return r;
  if (!(flags & MATGPTQ_B200_FLAG_ASYNC) && cudaStreamSynchronize(cs) != cudaSuccess) return MG_ERR_CUDA;
  return MG_OK;
}

int64_t matgptq_b200_matmul_workspace_bytes(int64_t n_out, int64_t n_in, int64_t batch) {
  if (n_out <= 0 || n_in <= 0 || batch <= 0) return 0;
  int sms = 0;
  if (sm_count_of_current_device(&sms) != MG_OK) sms = 148;
  if (!uses_tensor_cores(n_out, batch)) return 0;
  return mg::gemm_tc_workspace_bytes(static_cast<int>(n_out), static_cast<int>(n_in), static_cast<int>(batch), sms);
}

int matgptq_b200_slice(const uint8_t *master_codes, uint8_t *sliced_codes, int64_t numel, int master_bitwidth,
                       int bitwidth, void *stream) {
  if (!valid_bitwidth(bitwidth) || master_bitwidth < bitwidth || master_bitwidth > 8 || numel < 0) return MG_ERR_BAD_ARG;
  if (numel == 0) return MG_OK;
  if (!master_codes || !sliced_codes) return MG_ERR_BAD_ARG;
  return mg::slice_launch(master_codes, sliced_codes, numel, master_bitwidth, bitwidth, static_cast<cudaStream_t>(stream));
}

int matgptq_b200_pack_qweights(const uint8_t *codes, uint32_t *packed, int64_t n_out, int64_t n_in, int bitwidth,
                               int slice_from_master, void *stream) {
  const int st = check_shape(n_out, n_in, bitwidth, -1);
  if (st != MG_OK) return st;
  if (!codes || !packed) return MG_ERR_BAD_ARG;
  if (slice_from_master != 0 && (slice_from_master < bitwidth || slice_from_master > 8)) return MG_ERR_BAD_ARG;
  return mg::pack_launch(codes, packed, static_cast<int>(n_out), static_cast<int>(n_in), bitwidth, slice_from_master,
                         static_cast<cudaStream_t>(stream));
}

int matgptq_b200_pack_qweights_host(const uint8_t *codes, uint32_t *packed, int64_t n_out, int64_t n_in, int bitwidth,
                                    int slice_from_master) {
  const int st = check_shape(n_out, n_in, bitwidth, -1);
  if (st != MG_OK) return st;
  if (!codes || !packed) return MG_ERR_BAD_ARG;
  if (slice_from_master != 0 && (slice_from_master < bitwidth || slice_from_master > 8)) return MG_ERR_BAD_ARG;
  return mg::pack_host(codes, packed, static_cast<int>(n_out), static_cast<int>(n_in), bitwidth, slice_from_master);
}

int matgptq_b200_unpack_qweights_host(const uint32_t *packed, uint8_t *codes, int64_t n_out, int64_t n_in,
                                      int bitwidth) {
  const int st = check_shape(n_out, n_in, bitwidth, -1);
  if (st != MG_OK) return st;
  if (!codes || !packed) return MG_ERR_BAD_ARG;
  return mg::unpack_host(packed, codes, static_cast<int>(n_out), static_cast<int>(n_in), bitwidth);
}

int matgptq_b200_reorder_scales(const void *scales, void *reordered, int64_t n_out, int64_t n_in, int64_t group_size,
                                void *stream) {
  const int st = check_shape(n_out, n_in, 8, group_size);
  if (st != MG_OK) return st;
  if (!scales || !reordered || scales == reordered) return MG_ERR_BAD_ARG;
  return mg::reorder_scales_launch(static_cast<const uint16_t *>(scales), static_cast<uint16_t *>(reordered),
                                   static_cast<int>(n_out), static_cast<int>(n_in), static_cast<int>(group_size),
                                   static_cast<cudaStream_t>(stream));
}

int matgptq_b200_reorder_scales_host(const void *scales, void *reordered, int64_t n_out, int64_t n_in,
                                     int64_t group_size) {
  const int st = check_shape(n_out, n_in, 8, group_size);
  if (st != MG_OK) return st;
  if (!scales || !reordered || scales == reordered) return MG_ERR_BAD_ARG;
  return mg::reorder_scales_host(static_cast<const uint16_t *>(scales), static_cast<uint16_t *>(reordered),
                                 static_cast<int>(n_out), static_cast<int>(n_in), static_cast<int>(group_size));
}

int matgptq_b200_dequantize(const uint32_t *packed, const void *scales, const void *zeros, void *w_out, int64_t n_out,
                            int64_t n_in, int bitwidth, int64_t group_size, uint32_t flags, void *stream) {
  const int st = check_shape(n_out, n_in, bitwidth, group_size);
  if (st != MG_OK) return st;
  if (!packed || !scales || !w_out) return MG_ERR_BAD_ARG;
  if (!aligned16(packed) || (reinterpret_cast<uintptr_t>(w_out) & 7u)) return MG_ERR_ALIGNMENT;
  return mg::dequant_launch(packed, static_cast<const uint16_t *>(scales), static_cast<const uint16_t *>(zeros),
                            static_cast<uint16_t *>(w_out), static_cast<int>(n_out), static_cast<int>(n_in), bitwidth,
                            static_cast<int>(group_size), (flags & MATGPTQ_B200_FLAG_BF16) != 0,
                            static_cast<cudaStream_t>(stream));
}

int matgptq_b200_device_status(int *status_out, int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) return MG_ERR_CUDA;
  int a = 0, b = 0;
  int r = mg::gemv_device_status(&a, reset);
  if (r != MG_OK) return r;
  r = mg::gemm_tc_device_status(&b, reset);
  if (r != MG_OK) return r;
  int d = 0;
  r = mg::gemv_zp_device_status(&d, reset);
  if (r != MG_OK) return r;
  int e = 0;
  r = mg::selftest_device_status(&e, reset);
  if (r != MG_OK) return r;
  if (status_out) *status_out = a ? a : (b ? b : (d ? d : e));
  return MG_OK;
}

}  // extern "C"
