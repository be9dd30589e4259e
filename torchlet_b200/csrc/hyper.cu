// Several residual streams a token ("hyper-connections"), a causal convolution over time in front of a
// sub-layer, and a layer norm.  z is the float32 stream tensor [tokens, n, width]; a sub-layer q with
// vectors a (in), b (out) and a matrix M (mix, indexed [from, to]) runs as
//
//   u = sum_s a_s z_s;   h = norm(u);   x = h + conv(h);   y = sublayer(x);   z_t <- sum_s M[s, t] z_s + b_t y
//
// Kernels (all float32 inside; T is the type of what a sub-layer reads):
//   fanout        z[t, s] = acc[t] for every s                       (the streams start equal)
//   collapse      acc[t] = sum_s z[t, s], ascending s
//   read_norm     one block a token: u, then (u - mean) / sqrt(var + eps) * w + b (``centre``) or
//                 u / sqrt(mean(u^2) + eps) * w (no centring); h float32, or T when no convolution follows
//   conv          x[t] = h[t] + sum_j w[:, j] h[t - taps + 1 + j] over a request's tokens; rows before the step's
//                 first token of a request come from the request's slot (the last taps - 1 rows of h that
//                 earlier steps left; zeros at a sequence's start, which is what a cleared slot holds)
//   conv_state    the slot's rows after the step: the last taps - 1 rows of h of the request (old rows
//                 shift down where the step brought fewer tokens than that); one thread a (request, channel)
//   write         z_t <- sum_s M[s, t] z_s + b_t y, all streams from the old ones; y is left zeroed
//   layer_norm    rows of a float32 [tokens, width] stream (optionally gathered) -> T, with weight and bias
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int MAX_STREAMS = 8;
constexpr int MAX_TAPS = 8;
constexpr int NORM_NT = 256;

__global__ void fanout_kernel(const float* __restrict__ acc, float* __restrict__ z, int n, int width, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over tokens * width
  if (i >= total) return;
  const size_t t = i / width, c = i - t * width;
  const float v = acc[i];
  for (int s = 0; s < n; ++s) z[(t * n + s) * width + c] = v;
}

__global__ void collapse_kernel(const float* __restrict__ z, float* __restrict__ acc, int n, int width, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width, c = i - t * width;
  float v = 0.f;
  for (int s = 0; s < n; ++s) v += z[(t * n + s) * width + c];
  acc[i] = v;
}

// One block a row.  ``z`` rows are [n, width] (n = 1 and a = nullptr: a plain stream); ``rows`` gathers.
// The row is kept in shared memory between the passes; mean and variance are two block sums whose order
// depends on the width alone.
template <typename OutT>
__global__ void __launch_bounds__(NORM_NT)
read_norm_kernel(const float* __restrict__ z, const float* __restrict__ a, const float* __restrict__ weight,
                 const float* __restrict__ bias, const int* __restrict__ rows, OutT* __restrict__ out, int n, int width,
                 float eps, int centre) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float u[];  // width
  __shared__ float scratch[32];
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* row = z + src * n * width;
  float sum = 0.f;
  for (int c = threadIdx.x; c < width; c += NORM_NT) {
    float v;
    if (a) {
      v = 0.f;
      for (int s = 0; s < n; ++s) v = fmaf(a[s], row[(size_t)s * width + c], v);
    } else {
      v = row[c];
    }
    u[c] = v;
    sum += v;
  }
  float mean = 0.f;
  if (centre) mean = block_sum<NORM_NT>(sum, scratch) / (float)width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += NORM_NT) {
    const float d = u[c] - mean;
    ss = fmaf(d, d, ss);
  }
  const float inv = 1.f / sqrtf(block_sum<NORM_NT>(ss, scratch) / (float)width + eps);
  OutT* o = out + (size_t)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += NORM_NT) {
    float v = (u[c] - mean) * inv * weight[c];
    if (bias) v += bias[c];
    o[c] = from_float<OutT>(v);
  }
}

// h [tokens, width] float32; w [width, taps]; state [max_slots, taps - 1, width] (row r: the input taps - 1 - r
// tokens before the request's next one); out [tokens, width].  One thread a (token, channel).
template <typename T>
__global__ void conv_kernel(const float* __restrict__ h, const float* __restrict__ w, const float* __restrict__ state,
                            const int* __restrict__ token_req, const int* __restrict__ req_indptr,
                            const int* __restrict__ slots, T* __restrict__ out, int tokens, int width, int taps,
                            int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)tokens * width) return;
  const int t = (int)(i / width), c = (int)(i - (size_t)t * width);
  const int req = token_req[t];
  const int first = req_indptr[req];
  const int slot = slots[req];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  const float* mine = state + (size_t)(live ? slot : 0) * (taps - 1) * width;
  const float centre = h[i];
  float sum = 0.f;
  for (int j = 0; j < taps; ++j) {  // ascending j: the oldest input first
    const int back = taps - 1 - j;  // how many tokens before t
    float v;
    if (t - back >= first) v = h[(size_t)(t - back) * width + c];
    else if (live) v = mine[(size_t)(taps - 1 - (first - (t - back))) * width + c];  // first - (t - back) rows before the step
    else v = 0.f;
    sum = fmaf(w[(size_t)c * taps + j], v, sum);
  }
  out[i] = from_float<T>(centre + sum);
}

__global__ void conv_state_kernel(const float* __restrict__ h, float* __restrict__ state, const int* __restrict__ req_indptr,
                                  const int* __restrict__ slots, int requests, int width, int taps, int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)requests * width) return;
  const int req = (int)(i / width), c = (int)(i - (size_t)req * width);
  const int slot = slots[req];
  if (!(TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0)) return;
  const int first = req_indptr[req], count = req_indptr[req + 1] - first;
  const int keep = taps - 1;
  float* mine = state + (size_t)slot * keep * width;
  float rows[MAX_TAPS];
  for (int r = 0; r < keep; ++r) {
    // row r of the new state: the input keep - r tokens before the request's NEXT token
    const int at = count - (keep - r);  // index among the step's tokens; negative: an old row
    rows[r] = at >= 0 ? h[(size_t)(first + at) * width + c] : mine[(size_t)(r + count) * width + c];
  }
  for (int r = 0; r < keep; ++r) mine[(size_t)r * width + c] = rows[r];
}

__global__ void write_kernel(float* __restrict__ z, float* __restrict__ y, const float* __restrict__ mix,
                             const float* __restrict__ b, int n, int width, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width, c = i - t * width;
  float old[MAX_STREAMS];
  for (int s = 0; s < n; ++s) old[s] = z[(t * n + s) * width + c];
  const float add = y[i];
  y[i] = 0.f;
  for (int to = 0; to < n; ++to) {
    float v = 0.f;
    for (int s = 0; s < n; ++s) v = fmaf(mix[s * n + to], old[s], v);
    z[(t * n + to) * width + c] = fmaf(b[to], add, v);
  }
}

}  // namespace

TL_DEBUG_READER(tl_hyper_debug_error)

extern "C" {

int tl_hyper_fanout(const float* acc, float* z, int tokens, int n, int width, cudaStream_t stream) {
  const size_t total = (size_t)tokens * width;
  if (total == 0) return 0;
  if (n <= 0) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(fanout_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, acc, z, n, width, total);
  return TL_LAUNCH_CHECK();
}

int tl_hyper_collapse(const float* z, float* acc, int tokens, int n, int width, cudaStream_t stream) {
  const size_t total = (size_t)tokens * width;
  if (total == 0) return 0;
  if (n <= 0) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(collapse_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, z, acc, n, width, total);
  return TL_LAUNCH_CHECK();
}

// a: nullptr with n = 1 reads a plain stream; rows: nullptr or the rows to gather; bias: may be nullptr.
int tl_hyper_read_norm(const float* z, const float* a, const float* weight, const float* bias, const int* rows, void* out,
                       int out_dtype, int count, int n, int width, float eps, int centre, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (n <= 0 || n > MAX_STREAMS || width <= 0 || (size_t)width * sizeof(float) > 200 * 1024) return TL_ERR_UNSUPPORTED;
  const size_t smem = (size_t)width * sizeof(float);
  if (out_dtype == TL_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(read_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    tl::launch_kernel(read_norm_kernel<float>, (unsigned)count, NORM_NT, smem, stream, z, a, weight, bias, rows,
                      (float*)out, n, width, eps, centre);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(read_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    tl::launch_kernel(read_norm_kernel<__nv_bfloat16>, (unsigned)count, NORM_NT, smem, stream, z, a, weight, bias, rows,
                      (__nv_bfloat16*)out, n, width, eps, centre);
  }
  return TL_LAUNCH_CHECK();
}

int tl_hyper_conv(const float* h, const float* w, const float* state, const int* token_req, const int* req_indptr,
                  const int* slots, void* out, int out_dtype, int tokens, int width, int taps, int max_slots,
                  cudaStream_t stream) {
  const size_t total = (size_t)tokens * width;
  if (total == 0) return 0;
  if (taps < 1 || taps > MAX_TAPS || (taps > 1 && state == nullptr)) return TL_ERR_UNSUPPORTED;  // one tap: no history
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == TL_DTYPE_F32)
    tl::launch_kernel(conv_kernel<float>, blocks, 256, 0, stream, h, w, state, token_req, req_indptr, slots, (float*)out,
                      tokens, width, taps, max_slots);
  else
    tl::launch_kernel(conv_kernel<__nv_bfloat16>, blocks, 256, 0, stream, h, w, state, token_req, req_indptr, slots,
                      (__nv_bfloat16*)out, tokens, width, taps, max_slots);
  return TL_LAUNCH_CHECK();
}

int tl_hyper_conv_state(const float* h, float* state, const int* req_indptr, const int* slots, int requests, int width,
                        int taps, int max_slots, cudaStream_t stream) {
  const size_t total = (size_t)requests * width;
  if (total == 0) return 0;
  if (taps < 2 || taps > MAX_TAPS) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(conv_state_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, h, state, req_indptr, slots,
                    requests, width, taps, max_slots);
  return TL_LAUNCH_CHECK();
}

int tl_hyper_write(float* z, float* y, const float* mix, const float* b, int tokens, int n, int width,
                   cudaStream_t stream) {
  const size_t total = (size_t)tokens * width;
  if (total == 0) return 0;
  if (n <= 0 || n > MAX_STREAMS) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(write_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, z, y, mix, b, n, width, total);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
