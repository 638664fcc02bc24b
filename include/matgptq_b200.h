/*
 * C ABI of libmatgptq_b200: the B200 (sm_100a) implementation of MatGPTQ's
 * bit-sliced mixed-precision linear layer.
 *
 * Plain pointers and sizes only.  Device pointers are CUDA device addresses in the
 * current context; `stream` is a cudaStream_t passed as void* (NULL = default
 * stream).  Every function returns 0 on success or one of the MATGPTQ_B200_ERR_*
 * codes; none of them calls exit() or prints.  Functions are thread-safe as long
 * as concurrent calls do not write the same buffers.  Nothing is allocated on the
 * device by any function in this header.
 *
 * Notation: N = out features, K = in features, M = activation rows (tokens),
 * b = inference bitwidth in {2,3,4,6,8}, g = group size in {-1, 32, 128},
 * G = K/g groups per row (1 when g = -1).
 * Shape limits: N % 16 == 0, K % 128 == 0 (and K % g == 0).
 */
#ifndef MATGPTQ_B200_H
#define MATGPTQ_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MATGPTQ_B200_OK 0
#define MATGPTQ_B200_ERR_BAD_ARG 1     /* bitwidth, group size, shape or null pointer */
#define MATGPTQ_B200_ERR_CUDA 2        /* a CUDA runtime call or a kernel launch failed */
#define MATGPTQ_B200_ERR_UNSUPPORTED 3 /* valid in the reference but not provided here */
#define MATGPTQ_B200_ERR_ALIGNMENT 4   /* a pointer is not 16-byte aligned */
#define MATGPTQ_B200_ERR_SCRATCH_TOO_SMALL 5 /* the shape needs more scratch than the built-in array holds */
#define MATGPTQ_B200_ERR_SCRATCH_UNAVAILABLE 6 /* the built-in scratch array could not be set up on this device */

/* feature flags: bits 0 and 1 are the reference's (csrc/include/common.cuh:78-86,
 * matgptq_cuda/matgptq_linear.py:6-9); bits 2 and 3 are additions. */
#define MATGPTQ_B200_FLAG_ASYNC 1 /* do not synchronise the device after the launch */
#define MATGPTQ_B200_FLAG_BF16 2  /* activations, scales and output are bfloat16 (else float16) */
#define MATGPTQ_B200_FLAG_PDL 4   /* launch with programmatic dependent launch: weight prefetch overlaps the previous kernel */
#define MATGPTQ_B200_FLAG_SCRATCH_REDUCE 8 /* tensor-core path: add the sums of a split K through scratch memory and a second
                                            * kernel instead of inside a thread-block cluster (needs the scratch) */

/* Library version (major*10000 + minor*100 + patch). */
int matgptq_b200_version(void);

/* Text for a status code (static storage). */
const char *matgptq_b200_strerror(int status);

/*
 * y[M,N] = x[M,K] . Wdq^T,  Wdq[n,k] = (q[n,k] - 2^(b-1)) * s[n, k/g] * 2^(8-b),
 * fp32 accumulation, output rounded to fp16 (or bf16 with FLAG_BF16).
 * Replaces matmul_matgptq_host (csrc/include/gemm.h:22-32, csrc/matgptq_gemm.cu:1026-1065);
 * argument order follows it (the reference calls N `m`, K `n` and M `k`).
 *   w: device, packed by matgptq_b200_pack_qweights, b*N*K/32 uint32
 *   s: device, reordered by matgptq_b200_reorder_scales, N*G 16-bit floats
 *   x: device, [M,K] row-major, 16-byte aligned;  y: device, [M,N] row-major
 * Any M >= 1 is accepted (the reference is only correct for M in {1,2,4} and multiples of 8).
 */
int matgptq_b200_matmul(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                        const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags);

/*
 * Extension (no counterpart in the reference's operator, whose zero point is the implicit 2^(b-1)): the same
 * product with per-group zero points, Wdq = s * (code * 2^(8-b) - zero), the formula of dequantize()
 * (src/quant_utils_matgpqt.py:19-22).  `z` holds the zero points in master (8-bit) units, in the type of the
 * scales and in their reordered layout (matgptq_b200_reorder_scales on the [N, G] zero points).  z == NULL is
 * matgptq_b200_matmul.  Every batch size runs on the GEMV family (more than 16 rows in passes of 16).
 */
int matgptq_b200_matmul_zp(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                           const void *w, const void *s, const void *z, const void *x, void *y, void *stream,
                           uint32_t flags);

/* Same, with the launch shape of the GEMV forced (0 = choose).  For tuning and tests.
 *   warps_per_cta: low byte = warps per CTA (1..16); next byte = how many of them share one row tile and split
 *                  the CTA's K range between them (0 or 1 = none; must divide the warps; needs the CTA's whole K
 *                  slice of the activations in shared memory, else MATGPTQ_B200_ERR_UNSUPPORTED)
 *   split_k:       CTAs per thread-block cluster along K, one of 1, 2, 4, 8 */
int matgptq_b200_matmul_tuned(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                              const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                              int warps_per_cta, int split_k);

/*
 * The same product with optional scratch memory and a forced path.  Batches of more than 16 rows run
 * on the tensor cores (tcgen05) (from 25 rows for layers with fewer than 2048 out-features, which
 * the GEMV serves faster until then); for shapes with few 128-row tiles that path splits K over
 * up to eight CTAs, which form a thread-block cluster and add their fp32 sums through distributed
 * shared memory, so that no scratch is needed.  Scratch of matgptq_b200_matmul_workspace_bytes(...)
 * bytes (16-byte aligned; contents may be anything before the call and are undefined after it; one
 * buffer per stream in flight) is used in two cases only: with FLAG_SCRATCH_REDUCE the sums go through
 * it and a second kernel, and when the device cannot place the cluster (a partitioned GPU) the launch
 * falls back to that form if the scratch is there (else MATGPTQ_B200_ERR_CUDA).  Both forms add in the
 * order of the K ranges and give identical bits.
 *   path: 0 = choose by batch size and out-features as above,
 *         1 = cluster GEMV, 2 = tensor-core path (any batch size)
 *   split_k: 0 = choose; otherwise the number of CTAs along K (tensor-core path: at most 8; with
 *            FLAG_SCRATCH_REDUCE it needs split_k*M*N*4 bytes of scratch)
 * The reference has one kernel pair for all batch sizes and no scratch
 * (csrc/matgptq_gemm.cu:955-964); this entry has no counterpart there.
 */
int matgptq_b200_matmul_ws(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in, int64_t batch,
                           const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                           void *workspace, int64_t workspace_bytes, int path, int split_k);

/*
 * Grouped product: n_segments weight matrices over the SAME activations, y[M, sum N_i] = x[M,K] . [W_0; W_1; ...]^T,
 * each segment with its own packed weights, scales, out-features N_i and bitwidth b_i (all with the same K and
 * group size); segment i fills the columns [sum_{j<i} N_j, +N_i) of y.  This is the fused qkv / gate_up layer
 * of a model whose checkpoint layers carry different bitwidths (vLLM fuses them into one layer,
 * inference_lib/vllm_matgptq.py:113-121; the bitwidth file of evo_quant_search.py:659-671 gives each its own b).
 * Batches of up to 16 rows run as ONE kernel launch (every CTA looks its segment up in a table); larger batches
 * run one launch per segment into the column block of that segment, each the way matgptq_b200_matmul would run
 * it (the tensor-core path from 17 or 25 rows; workspace as for matgptq_b200_matmul_ws, sized for the largest
 * segment; may be NULL).  Up to 8 segments.  The reference has no
 * counterpart: its operator takes one bitwidth per call.
 */
typedef struct {
  const void *w;    /* device, packed by matgptq_b200_pack_qweights at this segment's bitwidth */
  const void *s;    /* device, reordered scales of this segment */
  int64_t n_out;    /* out-features of this segment, a multiple of 16 */
  int64_t bitwidth; /* 2, 3, 4, 6 or 8 */
} matgptq_b200_segment;
int matgptq_b200_matmul_grouped(const matgptq_b200_segment *segments, int n_segments, int64_t group_size, int64_t n_in,
                                int64_t batch, const void *x, void *y, void *stream, uint32_t flags, void *workspace,
                                int64_t workspace_bytes);

/*
 * Row-parallel product fused with the all-reduce of its output over peer memory (tensor parallelism: every rank
 * holds a K shard of the layer and calls this with its shard; all ranks pass the same n_out, batch, bitwidth and
 * a K shard of the same size).  In the reference this step is vLLM's: RowParallelLinear all-reduces what
 * MatGPTQLinearMethod.apply returns (inference_lib/vllm_matgptq.py:180-200 holds no collective), so the entry has
 * no counterpart there.  One kernel: in the epilogue every fp32 partial sum is stored, paired with the epoch of the
 * call in one 8-byte store, into this rank's slot in every other rank's buffer (plain stores over NVLink to
 * peer-mapped memory); the same thread then reads the other ranks' values of that output from its own buffer,
 * polling until each carries the epoch, and adds them in rank order, so all ranks get the same bits and y needs no
 * further collective.  Waits are bounded (about a second): a rank that never arrives leaves status 105 in
 * matgptq_b200_device_status instead of a hung GPU.
 *   comm.data[q]: device address, valid on THIS device, of rank q's buffer (this rank's own for q == rank, a peer
 *       mapping otherwise): 2*nranks*slot_elems 8-byte words, all zero before the first call, 8-byte aligned.  Two
 *       slot sets alternate from call to call, so one buffer serves every layer.
 *   comm.ctrl: 4 uint32 in this rank's own memory, zero before the first call.
 *   comm.slot_elems >= batch * n_out.
 *   comm.push_only: store only (also into the own slot); matgptq_b200_allreduce_finish then adds up.  For running all
 *       ranks one after the other on one GPU (tests): kernels that wait for each other must not be separate launches.
 * Batches of 32 rows and more and group sizes other than 128 return MATGPTQ_B200_ERR_UNSUPPORTED with nothing
 * launched: run matgptq_b200_matmul and a library all-reduce instead.  Calls on one communicator must be made in
 * the same order on every rank, on one stream per rank.
 */
typedef struct {
  void *data[8];
  void *ctrl;
  int64_t slot_elems;
  int rank, nranks;
  int push_only;
} matgptq_b200_comm;
int matgptq_b200_matmul_allreduce(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in_shard, int64_t batch,
                                  const void *w, const void *s, const void *x, void *y, void *stream, uint32_t flags,
                                  const matgptq_b200_comm *comm);
/* Adds up what launches with comm.push_only stored (status 105 if a value of some rank is missing) into
 * y[batch, n_out] and closes the epoch. */
int matgptq_b200_allreduce_finish(const matgptq_b200_comm *comm, void *y, int64_t n_out, int64_t batch, void *stream,
                                  uint32_t flags);

/* Scratch bytes matgptq_b200_matmul_ws wants for this shape on the current device (0 = none). */
int64_t matgptq_b200_matmul_workspace_bytes(int64_t n_out, int64_t n_in, int64_t batch);

/*
 * matgptq_b200_matmul_ws for callers that cannot allocate: hosts whose memory pool already
 * owns the whole device, plugins without access to their host's allocator, loops in which
 * cudaMalloc is forbidden because it synchronises the device.  The scratch of a K split (used as
 * matgptq_b200_matmul_ws describes: with FLAG_SCRATCH_REDUCE, or when the device cannot place the
 * cluster) is a fixed array of MATGPTQ_B200_STATIC_SCRATCH_BYTES inside the library image; once set up
 * on a GPU it occupies that much of its memory until the process exits.  This entry point has no
 * counterpart in the reference.
 *   - It calls no cudaMalloc, cudaFree or any other allocating routine.
 *   - Shapes whose scratch need (matgptq_b200_matmul_workspace_bytes) exceeds the array run without
 *     scratch; with FLAG_SCRATCH_REDUCE they return MATGPTQ_B200_ERR_SCRATCH_TOO_SMALL and launch nothing.
 *   - The first call on a device for a shape that splits K resolves the array's device address
 *     (cudaGetSymbolAddress, with that device current) and remembers it.  The CUDA runtime loads
 *     device code lazily, so it is THIS first call that brings the array into the device's memory:
 *     the driver takes the MATGPTQ_B200_STATIC_SCRATCH_BYTES then, not when the library is loaded.
 *     Make that first call (any shape with a batch of 32 or more and few row tiles, e.g. the one you
 *     will run) early: before a host that sizes its pool from the free memory does so, and before
 *     any stream capture starts.  If the device has no room left at that moment the call returns
 *     MATGPTQ_B200_ERR_SCRATCH_UNAVAILABLE and launches nothing.  Every later call on that device
 *     leaves the amount of free device memory unchanged.
 *   - All calls on a device share the one array and it keeps whatever the last call left in it;
 *     nothing in it needs clearing, because each call writes every partial sum before reading
 *     it.  Two calls whose kernels overlap on the GPU (different streams) race on it: serialise
 *     them, or give one of them its own scratch through matgptq_b200_matmul_ws.
 */
#define MATGPTQ_B200_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int matgptq_b200_matmul_static_scratch(int64_t bitwidth, int64_t group_size, int64_t n_out, int64_t n_in,
                                       int64_t batch, const void *w, const void *s, const void *x, void *y,
                                       void *stream, uint32_t flags);

/*
 * MSB slicing of 8-bit master codes to b bits with round-to-nearest and saturation.
 * Replaces matryoshka_slice (src/quant_utils_matgpqt.py:9-17).  In and out are
 * device buffers of numel bytes and may be the same buffer.
 */
int matgptq_b200_slice(const uint8_t *master_codes, uint8_t *sliced_codes, int64_t numel, int master_bitwidth,
                       int bitwidth, void *stream);

/*
 * Pack codes[N,K] (uint8, device) into the layout the kernels read: b*N*K/32 uint32.
 * Replaces pack_matgptq_qweights (csrc/bindings.cpp:43-84) and the CPU packers behind
 * it (csrc/utils.cpp:22-217).  With slice_from_master == 0 the codes are already
 * b-bit (what the reference op receives); with slice_from_master == m > 0 they are
 * m-bit master codes and the slicing above is fused into the pack.
 */
int matgptq_b200_pack_qweights(const uint8_t *codes, uint32_t *packed, int64_t n_out, int64_t n_in, int bitwidth,
                               int slice_from_master, void *stream);

/* The same packing on the CPU (host pointers), and its inverse.  The reference packs
 * on the host only (csrc/bindings.cpp:63-83); these serve hosts without a GPU and tests. */
int matgptq_b200_pack_qweights_host(const uint8_t *codes, uint32_t *packed, int64_t n_out, int64_t n_in, int bitwidth,
                                    int slice_from_master);
int matgptq_b200_unpack_qweights_host(const uint32_t *packed, uint8_t *codes, int64_t n_out, int64_t n_in,
                                      int bitwidth);

/*
 * Scales [N,G] -> [N/16, G, 16] (16-bit elements, fp16 or bf16), device or host.
 * Replaces reorder_matgptq_scales (csrc/bindings.cpp:86-142).  In and out must differ.
 */
int matgptq_b200_reorder_scales(const void *scales, void *reordered, int64_t n_out, int64_t n_in, int64_t group_size,
                                void *stream);
int matgptq_b200_reorder_scales_host(const void *scales, void *reordered, int64_t n_out, int64_t n_in,
                                     int64_t group_size);

/*
 * Packed weights -> dense W[N,K] in fp16/bf16, bit-exact with the reference's
 * dequantize (src/quant_utils_matgpqt.py:19-22): W = round(s * ((code << (8-b)) - zero)).
 * `zeros` is NULL (zero = 128, what the three-op path implies, csrc/matgptq_gemm.cu:552,631)
 * or per-group zero points in master units, reordered like the scales.
 */
int matgptq_b200_dequantize(const uint32_t *packed, const void *scales, const void *zeros, void *w_out, int64_t n_out,
                            int64_t n_in, int bitwidth, int64_t group_size, uint32_t flags, void *stream);

/*
 * Helpers of the decode harness (matgptq_b200/decode.py); the reference leaves these steps to
 * vLLM / transformers and has no counterpart.  All tensors are device, contiguous, fp16 or bf16
 * (FLAG_BF16); arithmetic is fp32.  With FLAG_PDL they are launched with programmatic dependent launch as
 * well: each lets the kernel behind it start its prologue at once and waits for the kernel before it.
 *   add_rmsnorm: x[rows,hidden] += delta (when delta != NULL); h = rmsnorm(x) * weight
 *   rope_kv:     qkv[B,S,(H+2KV)*d] -> q_out[B,H,S,d] rotated (pairs 2i,2i+1); rotated k and v are
 *                written into the caches [B,KV,max_seq,d] at positions[s]; cos/sin are [max_seq,d/2] fp32
 *   silu_mul:    gate_up[rows,2*I] -> out[rows,I] = silu(gate) * up
 *   argmax:      logits[rows,cols] (cols % 8 == 0) -> out[rows] int64: the first index of the row's maximum (greedy sampling)
 */
int matgptq_b200_add_rmsnorm(void *x, const void *delta, const void *weight, void *h, int64_t rows, int64_t hidden,
                             float eps, uint32_t flags, void *stream);
int matgptq_b200_rope_kv(const void *qkv, const int64_t *positions, const float *cos_table, const float *sin_table,
                         void *q_out, void *k_cache, void *v_cache, int64_t batch, int64_t seq, int64_t n_heads,
                         int64_t n_kv_heads, int64_t head_dim, int64_t max_seq, uint32_t flags, void *stream);
int matgptq_b200_silu_mul(const void *gate_up, void *out, int64_t rows, int64_t intermediate, uint32_t flags, void *stream);
int matgptq_b200_argmax(const void *logits, int64_t *out, int64_t rows, int64_t cols, uint32_t flags, void *stream);

/*
 * Waits inside the kernels (on asynchronous copies) are bounded: a kernel that gives
 * up records a non-zero code instead of hanging, and its output is then undefined.
 * This call synchronises with the device, returns the first code recorded on the
 * current device since the last reset (0 = none; 101 weight copy, 102 activation
 * copy, 103 tensor-core completion, 105 a peer rank's partial sums) and clears it when reset != 0.  The reference has
 * no counterpart: its only error path is exit(1) in CHECK_CUDA (csrc/include/common.cuh:44-51).
 */
int matgptq_b200_device_status(int *status_out, int reset);

/*
 * Self-test of that mechanism: launches one warp that waits, with a short poll limit, on a barrier that
 * nothing will ever complete, so the wait runs out, `status_code` (101, 102 or 103) is recorded for
 * matgptq_b200_device_status to report and *gave_up_flag (device int, may be NULL) is set to 1.  The kernel
 * then ends normally; the device is not faulted or hung.  No counterpart in the reference.
 */
int matgptq_b200_selftest_wait_timeout(int status_code, int *gave_up_flag, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MATGPTQ_B200_H */
