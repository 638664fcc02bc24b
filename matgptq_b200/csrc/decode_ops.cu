// Small fused kernels of the decode harness around the packed linears: residual add + RMSNorm,
// rotary embedding + KV-cache write, SiLU(gate) * up.  The reference leaves these to vLLM /
// transformers (inference_lib/inference_demo_vllm.py, inference_demo_transformers.py:141-173); they are
// here so that a decode step is a few launches per layer instead of dozens of elementwise ones.
// T is __half or __nv_bfloat16; arithmetic is fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/matgptq_b200.h"
#include "kernels.h"

namespace mg {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// x[row] += delta[row] (when delta != null), then h[row] = rmsnorm(x[row]) * weight.  One CTA per row.
// Programmatic dependent launch: let the next kernel of the stream start its prologue now (the packed products
// prefetch their weights there), then wait until the previous kernel's results are complete and visible.  Both
// are no-ops for a kernel that was launched without the attribute and has no dependents.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename Kernel, typename... Args>
static int launch_helper(Kernel kernel, unsigned grid, unsigned block, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, args...) == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(T *__restrict__ x, const T *__restrict__ delta, const T *__restrict__ weight,
                                                          T *__restrict__ h, int hidden, float eps) {
  pdl_prologue();
  __shared__ float red[8];
  T *xr = x + static_cast<size_t>(blockIdx.x) * hidden;
  const T *dr = delta ? delta + static_cast<size_t>(blockIdx.x) * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f(xr[i]);
    if (dr) {
      v = to_f(from_f<T>(v + to_f(dr[i])));  // the residual stream stays in the model dtype
      xr[i] = from_f<T>(v);
    }
    ss += v * v;
  }
  for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / hidden + eps);
  T *hr = h + static_cast<size_t>(blockIdx.x) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    hr[i] = from_f<T>(to_f(from_f<T>(to_f(xr[i]) * inv)) * to_f(weight[i]));
}

// The same with 16-byte accesses and the row kept in registers: hidden % 8 == 0, hidden <= 512 * 8 * kRowVecs.
constexpr int kNormThreads = 512, kRowVecs = 4;
template <typename T>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_vec_kernel(T *__restrict__ x, const T *__restrict__ delta,
                                                                       const T *__restrict__ weight, T *__restrict__ h, int hidden,
                                                                       float eps) {
  pdl_prologue();
  __shared__ float red[kNormThreads / 32];
  const int nvec = hidden >> 3;
  uint4 *xr = reinterpret_cast<uint4 *>(x + static_cast<size_t>(blockIdx.x) * hidden);
  const uint4 *dr = delta ? reinterpret_cast<const uint4 *>(delta + static_cast<size_t>(blockIdx.x) * hidden) : nullptr;
  const uint4 *wr = reinterpret_cast<const uint4 *>(weight);
  uint4 xv[kRowVecs], dv[kRowVecs], wv[kRowVecs];
#pragma unroll
  for (int j = 0; j < kRowVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      xv[j] = xr[v];
      if (dr) dv[j] = dr[v];
      wv[j] = wr[v];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRowVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      T *xe = reinterpret_cast<T *>(&xv[j]);
      const T *de = reinterpret_cast<const T *>(&dv[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (dr) xe[e] = from_f<T>(to_f(xe[e]) + to_f(de[e]));
        const float f = to_f(xe[e]);
        ss += f * f;
      }
      if (dr) xr[v] = xv[j];
    }
  }
  for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / hidden + eps);
  uint4 *hr = reinterpret_cast<uint4 *>(h + static_cast<size_t>(blockIdx.x) * hidden);
#pragma unroll
  for (int j = 0; j < kRowVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      uint4 o;
      T *oe = reinterpret_cast<T *>(&o);
      const T *xe = reinterpret_cast<const T *>(&xv[j]);
      const T *we = reinterpret_cast<const T *>(&wv[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) oe[e] = from_f<T>(to_f(from_f<T>(to_f(xe[e]) * inv)) * to_f(we[e]));
      hr[v] = o;
    }
  }
}

// qkv [B, S, (H + 2*KV) * d] -> q_out [B, H, S, d] rotated; k rotated and v written into the caches
// [B, KV, max_seq, d] at positions[s].  cos/sin are [max_seq, d/2] fp32.  Pairs are (2i, 2i+1).
template <typename T>
__global__ void rope_kv_kernel(const T *__restrict__ qkv, const long long *__restrict__ positions, const float *__restrict__ cos_t,
                               const float *__restrict__ sin_t, T *__restrict__ q_out, T *__restrict__ k_cache, T *__restrict__ v_cache,
                               int B, int S, int H, int KV, int d, int max_seq) {
  pdl_prologue();
  const int heads = H + 2 * KV, half = d / 2;
  const long long total = static_cast<long long>(B) * S * heads * half;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    long long r = idx / half;
    const int head = static_cast<int>(r % heads);
    r /= heads;
    const int s = static_cast<int>(r % S), b = static_cast<int>(r / S);
    const long long pos = positions[s];
    const T *src = qkv + ((static_cast<size_t>(b) * S + s) * heads + head) * d + 2 * i;
    const float a = to_f(src[0]), c = to_f(src[1]);
    if (head < H + KV) {
      const float cs = cos_t[pos * half + i], sn = sin_t[pos * half + i];
      const T r0 = from_f<T>(a * cs - c * sn), r1 = from_f<T>(a * sn + c * cs);
      T *dst = (head < H) ? q_out + ((static_cast<size_t>(b) * H + head) * S + s) * d + 2 * i
                          : k_cache + ((static_cast<size_t>(b) * KV + (head - H)) * max_seq + pos) * d + 2 * i;
      dst[0] = r0;
      dst[1] = r1;
    } else {
      T *dst = v_cache + ((static_cast<size_t>(b) * KV + (head - H - KV)) * max_seq + pos) * d + 2 * i;
      dst[0] = src[0];
      dst[1] = src[1];
    }
  }
}

// gu [rows, 2*inter] -> out [rows, inter] = silu(gate) * up, both factors rounded to the model dtype first
template <typename T>
__global__ void silu_mul_kernel(const T *__restrict__ gu, T *__restrict__ out, long long rows, int inter) {
  pdl_prologue();
  const long long total = rows * inter;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / inter;
    const int c = static_cast<int>(idx - r * inter);
    const float gte = to_f(gu[r * 2 * inter + c]), up = to_f(gu[r * 2 * inter + inter + c]);
    const float act = to_f(from_f<T>(gte / (1.f + __expf(-gte))));
    out[idx] = from_f<T>(act * up);
  }
}

// Greedy sampling: index of the largest logit of every row (the first one on ties), one CTA per row.  Logits
// [rows, cols] in the model dtype; `cols` a multiple of 8 and rows 16-byte aligned for the vector loads.
template <typename T>
__global__ void __launch_bounds__(1024, 1) argmax_kernel(const T *__restrict__ logits, long long *__restrict__ out, int cols) {
  pdl_prologue();
  const T *row = logits + static_cast<long long>(blockIdx.x) * cols;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4 *>(row + c);
    const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float f = to_f(e[k]);
      if (f > best) {  // strictly greater: within a thread the columns ascend, so the first maximum stays
        best = f;
        best_i = c + k;
      }
    }
  }
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  auto better = [](float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); };
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_down_sync(0xffffffffu, best, off);
    const int oi = __shfl_down_sync(0xffffffffu, best_i, off);
    if (better(ov, oi, best, best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_val[threadIdx.x >> 5] = best;
    s_idx[threadIdx.x >> 5] = best_i;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? s_val[threadIdx.x] : -INFINITY;
    best_i = threadIdx.x < nw ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, best, off);
      const int oi = __shfl_down_sync(0xffffffffu, best_i, off);
      if (better(ov, oi, best, best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

static unsigned grid_for(long long total, int threads) {
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (blocks < 1) blocks = 1;
  return static_cast<unsigned>(blocks);
}

}  // namespace mg

extern "C" {

int matgptq_b200_add_rmsnorm(void *x, const void *delta, const void *weight, void *h, int64_t rows, int64_t hidden,
                             float eps, uint32_t flags, void *stream) {
  if (!x || !weight || !h || rows < 0 || hidden <= 0) return MG_ERR_BAD_ARG;
  if (rows == 0) return MG_OK;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const bool vec = hidden % 8 == 0 && hidden <= static_cast<int64_t>(mg::kNormThreads) * 8 * mg::kRowVecs &&
                   (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
                    reinterpret_cast<uintptr_t>(h)) % 16 == 0;
  const unsigned grid = static_cast<unsigned>(rows);
  const int hd = static_cast<int>(hidden);
  const bool pdl = (flags & MATGPTQ_B200_FLAG_PDL) != 0;
  if (flags & MATGPTQ_B200_FLAG_BF16) {
    using T = __nv_bfloat16;
    if (vec)
      return mg::launch_helper(mg::add_rmsnorm_vec_kernel<T>, grid, mg::kNormThreads, cs, pdl, static_cast<T *>(x),
                               static_cast<const T *>(delta), static_cast<const T *>(weight), static_cast<T *>(h), hd, eps);
    else
      return mg::launch_helper(mg::add_rmsnorm_kernel<T>, grid, 256, cs, pdl, static_cast<T *>(x), static_cast<const T *>(delta),
                               static_cast<const T *>(weight), static_cast<T *>(h), hd, eps);
  } else {
    using T = __half;
    if (vec)
      return mg::launch_helper(mg::add_rmsnorm_vec_kernel<T>, grid, mg::kNormThreads, cs, pdl, static_cast<T *>(x),
                               static_cast<const T *>(delta), static_cast<const T *>(weight), static_cast<T *>(h), hd, eps);
    else
      return mg::launch_helper(mg::add_rmsnorm_kernel<T>, grid, 256, cs, pdl, static_cast<T *>(x), static_cast<const T *>(delta),
                               static_cast<const T *>(weight), static_cast<T *>(h), hd, eps);
  }
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

int matgptq_b200_rope_kv(const void *qkv, const int64_t *positions, const float *cos_table, const float *sin_table, void *q_out,
                         void *k_cache, void *v_cache, int64_t batch, int64_t seq, int64_t n_heads, int64_t n_kv_heads,
                         int64_t head_dim, int64_t max_seq, uint32_t flags, void *stream) {
  if (!qkv || !positions || !cos_table || !sin_table || !q_out || !k_cache || !v_cache || head_dim % 2) return MG_ERR_BAD_ARG;
  const long long total = batch * seq * (n_heads + 2 * n_kv_heads) * (head_dim / 2);
  if (total <= 0) return MG_OK;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const unsigned grid = mg::grid_for(total, 256);
  const long long *pos = reinterpret_cast<const long long *>(positions);
  if (flags & MATGPTQ_B200_FLAG_BF16)
    return mg::launch_helper(mg::rope_kv_kernel<__nv_bfloat16>, grid, 256, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
        static_cast<const __nv_bfloat16 *>(qkv), pos, cos_table, sin_table, static_cast<__nv_bfloat16 *>(q_out),
        static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), static_cast<int>(batch), static_cast<int>(seq),
        static_cast<int>(n_heads), static_cast<int>(n_kv_heads), static_cast<int>(head_dim), static_cast<int>(max_seq));
  else
    return mg::launch_helper(mg::rope_kv_kernel<__half>, grid, 256, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
        static_cast<const __half *>(qkv), pos, cos_table, sin_table, static_cast<__half *>(q_out), static_cast<__half *>(k_cache),
        static_cast<__half *>(v_cache), static_cast<int>(batch), static_cast<int>(seq), static_cast<int>(n_heads),
        static_cast<int>(n_kv_heads), static_cast<int>(head_dim), static_cast<int>(max_seq));
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

int matgptq_b200_argmax(const void *logits, int64_t *out, int64_t rows, int64_t cols, uint32_t flags, void *stream) {
  if (!logits || !out || rows < 0 || cols <= 0 || cols % 8 != 0 || cols > (1 << 30)) return MG_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(logits) & 15u) return MG_ERR_ALIGNMENT;
  if (rows == 0) return MG_OK;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  static_assert(sizeof(long long) == sizeof(int64_t), "int64_t is long long here");
  if (flags & MATGPTQ_B200_FLAG_BF16)
    return mg::launch_helper(mg::argmax_kernel<__nv_bfloat16>, static_cast<unsigned>(rows), 1024, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
        static_cast<const __nv_bfloat16 *>(logits), reinterpret_cast<long long *>(out), static_cast<int>(cols));
  else
    return mg::launch_helper(mg::argmax_kernel<__half>, static_cast<unsigned>(rows), 1024, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
                             static_cast<const __half *>(logits), reinterpret_cast<long long *>(out), static_cast<int>(cols));
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

int matgptq_b200_silu_mul(const void *gate_up, void *out, int64_t rows, int64_t intermediate, uint32_t flags, void *stream) {
  if (!gate_up || !out || rows < 0 || intermediate <= 0) return MG_ERR_BAD_ARG;
  if (rows == 0) return MG_OK;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const unsigned grid = mg::grid_for(rows * intermediate, 256);
  if (flags & MATGPTQ_B200_FLAG_BF16)
    return mg::launch_helper(mg::silu_mul_kernel<__nv_bfloat16>, grid, 256, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
                             static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(out),
                             static_cast<long long>(rows), static_cast<int>(intermediate));
  else
    return mg::launch_helper(mg::silu_mul_kernel<__half>, grid, 256, cs, (flags & MATGPTQ_B200_FLAG_PDL) != 0,
                             static_cast<const __half *>(gate_up), static_cast<__half *>(out), static_cast<long long>(rows),
                             static_cast<int>(intermediate));
  return cudaGetLastError() == cudaSuccess ? MG_OK : MG_ERR_CUDA;
}

}  // extern "C"
