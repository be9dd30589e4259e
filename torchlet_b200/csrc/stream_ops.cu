// Small kernels around the float32 residual stream for block arrangements whose sub-layers
// do not add into the stream one after the other:
//
//   scaled_add        acc += m * delta            (a parallel block's one residual sum; optionally
//                                                  the updated stream is also written in bfloat16)
//   rms_scaled_add    acc += m * y / sqrt(mean(y^2) + eps) * w      (a normed side branch)
//   gated_token_embed out = gelu_tanh(gate) * table[token]          (gate of a per-token input)
//   clamped_glu       out = g sigmoid(alpha g) (u + 1),  g = min(gate, limit), u = clamp(up, +-limit)
//   glu_act           out = act(gate) * up (* one number a token), act = silu or the tanh form of gelu
//   scale             x *= alpha                  (logit scale)
//   fill_zero
//
// All arithmetic is float32; T is the storage type of activations.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

__global__ void fill_zero_kernel(float4* __restrict__ p, size_t quads) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < quads) p[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// The same one element a thread, for sizes or addresses the 16-byte forms do not take.
__global__ void fill_zero_scalar_kernel(float* __restrict__ p, size_t n) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 0.f;
}

__global__ void scaled_add_scalar_kernel(float* __restrict__ acc, float* __restrict__ delta, float m,
                                         __nv_bfloat16* __restrict__ cast, size_t n, int clear) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = fmaf(m, delta[i], acc[i]);
  acc[i] = a;
  if (cast) cast[i] = __float2bfloat16_rn(a);
  if (clear) delta[i] = 0.f;  // behind the store that needed its old value
}

__global__ void scale_kernel(float* __restrict__ p, float alpha, size_t n) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] *= alpha;
}

// acc += m * delta over float4; cast (optional) receives the updated stream in bfloat16; clear: delta is left zeroed
// (for the next branch to add into).
__global__ void scaled_add_kernel(float4* __restrict__ acc, float4* __restrict__ delta, float m,
                                  uint2* __restrict__ cast, size_t quads, int clear) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= quads) return;
  float4 a = acc[i];
  const float4 d = delta[i];
  a.x = fmaf(m, d.x, a.x);
  a.y = fmaf(m, d.y, a.y);
  a.z = fmaf(m, d.z, a.z);
  a.w = fmaf(m, d.w, a.w);
  acc[i] = a;
  if (cast) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    cast[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
  if (clear) delta[i] = make_float4(0.f, 0.f, 0.f, 0.f);  // behind the store that needed its old value
}

// One block per row: acc[r] += m * y[r] * rsqrt(mean(y[r]^2) + eps) * w.  The order of the
// additions depends only on the width.
template <int NT>
__global__ void __launch_bounds__(NT)
rms_scaled_add_kernel(float* __restrict__ acc, float* __restrict__ y, const float* __restrict__ w, float m,
                      float eps, int hidden, int clear) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float scratch[32];
  float* row = y + (size_t)blockIdx.x * hidden;
  float* out = acc + (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int j = threadIdx.x; j < hidden; j += NT) {
    const float v = row[j];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<NT>(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int j = threadIdx.x; j < hidden; j += NT) {
    out[j] = fmaf(m, row[j] * inv * w[j], out[j]);
    if (clear) row[j] = 0.f;  // the side stream is left zeroed for the next sub-layer to add into
  }
}

// The same for a sub-layer output of which a product left ``splits`` partial sums [splits][rows][hidden]:
// v = y + their sum in ascending order, acc[r] += m * v * rsqrt(mean(v^2) + eps) * w; ``clear``: y is left zeroed.  The sums are taken twice
// (once for the mean square, once for the output) rather than kept: the partial sums of a step of few tokens
// lie in the L2; the first eight entries a thread owns are kept in registers instead.
template <int NT>
__global__ void __launch_bounds__(NT)
rms_scaled_add_partials_kernel(float* __restrict__ acc, float* __restrict__ y, const float* __restrict__ partials,
                               int splits, int rows, const float* __restrict__ w, float m, float eps, int hidden,
                               int clear) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float scratch[32];
  const size_t plane = (size_t)rows * hidden;
  const float* row = partials + (size_t)blockIdx.x * hidden;
  float* yrow = y + (size_t)blockIdx.x * hidden;
  float* out = acc + (size_t)blockIdx.x * hidden;
  constexpr int KEEP = 8;
  float kept[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int j = threadIdx.x + i * NT;
    float v = 0.f;
    if (j < hidden) {
      v = yrow[j];
      for (int s = 0; s < splits; ++s) v += row[(size_t)s * plane + j];
    }
    kept[i] = v;
    ss = fmaf(v, v, ss);
  }
  for (int j = threadIdx.x + KEEP * NT; j < hidden; j += NT) {
    float v = yrow[j];
    for (int s = 0; s < splits; ++s) v += row[(size_t)s * plane + j];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<NT>(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int j = threadIdx.x + i * NT;
    if (j < hidden) {
      out[j] = fmaf(m, kept[i] * inv * w[j], out[j]);
      yrow[j] = clear ? 0.f : kept[i];  // else y holds the finished sum, as after a finishing pass of its own
    }
  }
  for (int j = threadIdx.x + KEEP * NT; j < hidden; j += NT) {
    float v = yrow[j];
    for (int s = 0; s < splits; ++s) v += row[(size_t)s * plane + j];
    out[j] = fmaf(m, v * inv * w[j], out[j]);
    yrow[j] = clear ? 0.f : v;
  }
}

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void gated_token_embed_kernel(const float* __restrict__ gate, const T* __restrict__ table, int table_stride,
                                         const int* __restrict__ ids, int vocab, T* __restrict__ out, int dim,
                                         size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / dim;
  const int j = (int)(idx - t * dim);
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  TL_DEBUG_OK(ok, TL_DEBUG_TOKEN, id);
  const float e = ok ? to_float(table[(size_t)id * table_stride + j]) : 0.f;
  out[idx] = from_float<T>(gelu_tanh(gate[idx]) * e);
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, float limit,
                                   float alpha) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int j = (int)(idx - t * inter);
  const float g = fminf(to_float(gu[t * 2 * inter + j]), limit);
  const float u = fminf(fmaxf(to_float(gu[t * 2 * inter + inter + j]), -limit), limit);
  out[idx] = from_float<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// act: 0 silu(g) = g sigmoid(g); 1 the tanh form of gelu, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))).
// row_scale (optional, float32 [tokens]): the row is multiplied by its token's number before it is rounded.
template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, int act,
                               const float* __restrict__ row_scale) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int j = (int)(idx - t * inter);
  const float g = to_float(gu[t * 2 * inter + j]);
  const float u = to_float(gu[t * 2 * inter + inter + j]);
  const float a = act == 1 ? 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)))
                           : g / (1.f + expf(-g));
  out[idx] = from_float<T>(a * u * (row_scale ? row_scale[t] : 1.f));
}

}  // namespace

TL_DEBUG_READER(tl_stream_ops_debug_error)

extern "C" {

int tl_fill_zero(float* p, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 || (reinterpret_cast<uintptr_t>(p) & 15)) {
    tl::launch_kernel(fill_zero_scalar_kernel, (unsigned)(((size_t)n + 255) / 256), 256, 0, stream, p, (size_t)n);
    return TL_LAUNCH_CHECK();
  }
  const size_t quads = (size_t)n / 4;
  tl::launch_kernel(fill_zero_kernel, (unsigned)((quads + 255) / 256), 256, 0, stream, (float4*)p, quads);
  return TL_LAUNCH_CHECK();
}

int tl_scale(float* p, float alpha, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  tl::launch_kernel(scale_kernel, (unsigned)(((size_t)n + 255) / 256), 256, 0, stream, p, alpha, (size_t)n);
  return TL_LAUNCH_CHECK();
}

int tl_scaled_add(float* acc, float* delta, float m, void* cast, long long n, int clear, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 || ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(delta)) & 15) ||
      (reinterpret_cast<uintptr_t>(cast) & 7)) {
    tl::launch_kernel(scaled_add_scalar_kernel, (unsigned)(((size_t)n + 255) / 256), 256, 0, stream, acc, delta, m,
                      (__nv_bfloat16*)cast, (size_t)n, clear);
    return TL_LAUNCH_CHECK();
  }
  const size_t quads = (size_t)n / 4;
  tl::launch_kernel(scaled_add_kernel, (unsigned)((quads + 255) / 256), 256, 0, stream, (float4*)acc,
                    (float4*)delta, m, (uint2*)cast, quads, clear);
  return TL_LAUNCH_CHECK();
}

int tl_rms_scaled_add(float* acc, float* y, const float* w, float m, float eps, int rows, int hidden, int clear,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 1024)
    tl::launch_kernel(rms_scaled_add_kernel<128>, rows, 128, 0, stream, acc, y, w, m, eps, hidden, clear);
  else
    tl::launch_kernel(rms_scaled_add_kernel<512>, rows, 512, 0, stream, acc, y, w, m, eps, hidden, clear);
  return TL_LAUNCH_CHECK();
}

int tl_rms_scaled_add_partials(float* acc, float* y, const float* partials, int splits, const float* w, float m, float eps,
                               int rows, int hidden, int clear, cudaStream_t stream) {
  if (rows <= 0 || hidden <= 0) return 0;
  if (splits <= 0) return TL_ERR_UNSUPPORTED;
  if (hidden <= 1024)
    tl::launch_kernel(rms_scaled_add_partials_kernel<128>, rows, 128, 0, stream, acc, y, partials, splits, rows, w, m, eps,
                      hidden, clear);
  else
    tl::launch_kernel(rms_scaled_add_partials_kernel<512>, rows, 512, 0, stream, acc, y, partials, splits, rows, w, m, eps,
                      hidden, clear);
  return TL_LAUNCH_CHECK();
}

int tl_gated_token_embed(const float* gate, const void* table, int table_stride, int dtype, const int* ids, int vocab,
                         void* out, int tokens, int dim, cudaStream_t stream) {
  const size_t total = (size_t)tokens * dim;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(gated_token_embed_kernel<float>, blocks, 256, 0, stream, gate, (const float*)table, table_stride,
                      ids, vocab, (float*)out, dim, total);
  else
    tl::launch_kernel(gated_token_embed_kernel<__nv_bfloat16>, blocks, 256, 0, stream, gate,
                      (const __nv_bfloat16*)table, table_stride, ids, vocab, (__nv_bfloat16*)out, dim, total);
  return TL_LAUNCH_CHECK();
}

int tl_clamped_glu(const void* gate_up, void* out, int dtype, int tokens, int inter, float limit, float alpha,
                   cudaStream_t stream) {
  const size_t total = (size_t)tokens * inter;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(clamped_glu_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter,
                      total, limit, alpha);
  else
    tl::launch_kernel(clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up,
                      (__nv_bfloat16*)out, inter, total, limit, alpha);
  return TL_LAUNCH_CHECK();
}

int tl_glu_act(const void* gate_up, void* out, int dtype, int tokens, int inter, int act, const float* row_scale,
               cudaStream_t stream) {
  const size_t total = (size_t)tokens * inter;
  if (total == 0) return 0;
  if (act < 0 || act > 1) return TL_ERR_UNSUPPORTED;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(glu_act_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total,
                      act, row_scale);
  else
    tl::launch_kernel(glu_act_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up,
                      (__nv_bfloat16*)out, inter, total, act, row_scale);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
