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
//                 u / sqrt(mean(u^2) + eps) * w (no centring); h float32, or T when no convolution follows.
//                 It can take the WRITE of the sub-layer before into the same pass, and, in a step of single tokens,
//                 the convolution and the slot's new rows: a decode step then runs ONE kernel a sub-layer here
//   conv          x[t] = h[t] + sum_j w[:, j] h[t - taps + 1 + j] over a request's tokens; rows before the step's
//                 first token of a request come from the request's slot (the last taps - 1 rows of h that
//                 earlier steps left; zeros at a sequence's start, which is what a cleared slot holds)
//   conv_state    the slot's rows after the step: the last taps - 1 rows of h of the request (old rows
//                 shift down where the step brought fewer tokens than that); one thread a (request, channel)
//   write         z_t <- sum_s M[s, t] z_s + b_t y, all streams from the old ones; y is left zeroed
//   layer_norm    rows of a float32 [tokens, width] stream (optionally gathered) -> T, with weight and bias
#include <math.h>

#include <type_traits>

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
//   y != nullptr: the WRITE of the sub-layer before comes first, z_t <- sum_s M[s, t] z_s + b_t y (y left zeroed),
//                 and the read takes the new streams from registers: one pass over z instead of two.
//   conv_w != nullptr: every request of the step brings ONE token, so a token's history is in its request's slot
//                 alone: x = h + conv(h) is written instead of h, and the slot's rows move up by one.
// Every sum is written as in write_kernel, conv_kernel and conv_state_kernel, so the results are theirs bit for bit.
// V consecutive channels of a row at once (V = 4 where the width allows: 16-byte loads, and a thread of a 2,048-wide
// row walks its channels in ONE round, which is what a step of few tokens, a chain of dependent loads, is made of).
template <int V> __device__ __forceinline__ void load_v(const float* p, float (&out)[V]) {
  if constexpr (V == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
    out[0] = *p;
  }
}
template <int V> __device__ __forceinline__ void store_v(float* p, const float (&v)[V]) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}
template <int V> __device__ __forceinline__ void store_v(__nv_bfloat16* p, const float (&v)[V]) {
  if constexpr (V == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
  } else {
    *p = __float2bfloat16_rn(v[0]);
  }
}

// NT threads a block: 256, or 512 for wide rows, where a thread then walks few channels (a step of few tokens is a
// chain of dependent loads; the fewer rounds, the shorter).
// N: the number of streams where it is 1, 2 or 4 (loops without guards, few registers), else 0 (any number up to 8).
template <typename OutT, int NT, int N, int V>
__global__ void __launch_bounds__(NT, N > 0 ? 1024 / NT : 1)  // 64 registers: 1,024 threads an SM and more (48 % -> of the DRAM peak)
read_norm_kernel(float* z, const float* __restrict__ a, const float* __restrict__ weight, const float* __restrict__ bias,
                 const int* __restrict__ rows, OutT* __restrict__ out, int n, int width, float eps, int centre,
                 float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ b,
                 const float* __restrict__ conv_w, float* __restrict__ conv_state, const int* __restrict__ token_req,
                 const int* __restrict__ slots, int taps, int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  constexpr int S = N > 0 ? N : MAX_STREAMS;  // the unrolled loops' bound
  if (N > 0) n = N;
  extern __shared__ __align__(16) float u[];  // width
  __shared__ float scratch[32];
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_b[MAX_STREAMS], s_a[MAX_STREAMS];
  if (y) {
    if (threadIdx.x < n * n) s_mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < n) s_b[threadIdx.x] = b[threadIdx.x];
  }
  if (a && threadIdx.x < n) s_a[threadIdx.x] = a[threadIdx.x];
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* row = z + src * n * width;
  float sum = 0.f;
  if (y) {
    float* add_row = y + src * width;
    // A round's loads are asked for one round ahead, the first ones before the coefficients have arrived: in a step
    // of few tokens the kernel is a chain of dependent trips to memory, and this takes one out.
    float old[S][V], add[V];
    int c = threadIdx.x * V;
    auto fetch = [&](int at) {
#pragma unroll
      for (int s = 0; s < S; ++s)
        if (s < n) load_v<V>(row + (size_t)s * width + at, old[s]);
      load_v<V>(add_row + at, add);
    };
    if (c < width) fetch(c);
    __syncthreads();
    while (c < width) {
      float v[V];
#pragma unroll
      for (int e = 0; e < V; ++e) v[e] = 0.f;
#pragma unroll
      for (int to = 0; to < S; ++to) {
        if (to < n) {
          float w[V];
#pragma unroll
          for (int e = 0; e < V; ++e) {
            float t = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s)
              if (s < n) t = fmaf(s_mix[s * n + to], old[s][e], t);
            w[e] = fmaf(s_b[to], add[e], t);
            v[e] = a ? fmaf(s_a[to], w[e], v[e]) : w[e];
          }
          store_v<V>(row + (size_t)to * width + c, w);
        }
      }
      // cleared only now: a store issued right behind the load of the same address, while that load is still in
      // flight, made the whole pass five times slower (measured: 146 -> 31 us for 2,048 tokens x 4 streams x 2,048)
      float zero[V];
#pragma unroll
      for (int e = 0; e < V; ++e) zero[e] = 0.f;
      store_v<V>(add_row + c, zero);
      store_v<V>(u + c, v);
#pragma unroll
      for (int e = 0; e < V; ++e) sum += v[e];
      c += NT * V;
      if (c < width) fetch(c);
    }
  } else {
    __syncthreads();
    for (int c = threadIdx.x * V; c < width; c += NT * V) {
      float v[V];
      if (a) {
        float old[S][V];
#pragma unroll
        for (int s = 0; s < S; ++s)
          if (s < n) load_v<V>(row + (size_t)s * width + c, old[s]);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          v[e] = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s)
            if (s < n) v[e] = fmaf(s_a[s], old[s][e], v[e]);
        }
      } else {
        load_v<V>(row + c, v);
      }
      store_v<V>(u + c, v);
#pragma unroll
      for (int e = 0; e < V; ++e) sum += v[e];
    }
  }
  float mean = 0.f;
  if (centre) mean = block_sum<NT>(sum, scratch) / (float)width;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < width; c += NT * V) {  // a thread reads back what it wrote itself
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float d = u[c + e] - mean;
      ss = fmaf(d, d, ss);
    }
  }
  const float inv = 1.f / sqrtf(block_sum<NT>(ss, scratch) / (float)width + eps);
  OutT* o = out + (size_t)blockIdx.x * width;
  const int keep = taps - 1;
  int slot = -1;
  if (conv_w) slot = slots[token_req[blockIdx.x]];
  const bool live = conv_w && TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  float* mine = conv_state + (size_t)(live ? slot : 0) * keep * width;
  for (int c = threadIdx.x * V; c < width; c += NT * V) {
    float w[V], bv[V], v[V];
    load_v<V>(weight + c, w);
    if (bias) load_v<V>(bias + c, bv);
    float hist[MAX_TAPS - 1][V];
    if (conv_w) {
#pragma unroll
      for (int r = 0; r < MAX_TAPS - 1; ++r) {
        if (r < keep) {
          if (live) load_v<V>(mine + (size_t)r * width + c, hist[r]);
          else
#pragma unroll
            for (int e = 0; e < V; ++e) hist[r][e] = 0.f;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      v[e] = __fmul_rn(__fmul_rn(u[c + e] - mean, inv), w[e]);
      if (bias) v[e] = __fadd_rn(v[e], bv[e]);
    }
    if (!conv_w) {
      store_v<V>(o + c, v);
      continue;
    }
    float x[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < MAX_TAPS; ++j)  // ascending j: the oldest input first, the token itself last
        if (j < taps) acc = fmaf(conv_w[(size_t)(c + e) * taps + j], j < keep ? hist[j < MAX_TAPS - 1 ? j : 0][e] : v[e], acc);
      x[e] = __fadd_rn(v[e], acc);
    }
    store_v<V>(o + c, x);
    if (live) {
#pragma unroll
      for (int r = 0; r < MAX_TAPS - 1; ++r)
        if (r < keep) store_v<V>(mine + (size_t)r * width + c, r + 1 < keep ? hist[r + 1 < MAX_TAPS - 1 ? r + 1 : 0] : v);
    }
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

__global__ void __launch_bounds__(256)
write_kernel(float* __restrict__ z, float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ b, int n,
             int width, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_b[MAX_STREAMS];
  if (threadIdx.x < n * n) s_mix[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < n) s_b[threadIdx.x] = b[threadIdx.x];
  __syncthreads();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width, c = i - t * width;
  float old[MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < MAX_STREAMS; ++s)
    if (s < n) old[s] = z[(t * n + s) * width + c];
  const float add = y[i];
#pragma unroll
  for (int to = 0; to < MAX_STREAMS; ++to) {
    if (to < n) {
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < n) v = fmaf(s_mix[s * n + to], old[s], v);
      z[(t * n + to) * width + c] = fmaf(s_b[to], add, v);
    }
  }
  y[i] = 0.f;  // behind the stores that needed its old value (see read_norm_kernel)
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
// y, mix, b (or nullptr): the write of the sub-layer before, z_t <- sum_s mix[s, t] z_s + b_t y, in the same pass
// (rows must be nullptr).  conv_w [width, taps] (or nullptr), conv_state [max_slots, taps - 1, width], token_req,
// slots: the convolution of a step whose requests bring one token each; out is then h + conv(h).
int tl_hyper_read_norm(float* z, const float* a, const float* weight, const float* bias, const int* rows, void* out,
                       int out_dtype, int count, int n, int width, float eps, int centre, float* y, const float* mix,
                       const float* b, const float* conv_w, float* conv_state, const int* token_req, const int* slots,
                       int taps, int max_slots, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (n <= 0 || n > MAX_STREAMS || width <= 0 || (size_t)width * sizeof(float) > 200 * 1024) return TL_ERR_UNSUPPORTED;
  if (y && (rows || !mix || !b)) return TL_ERR_UNSUPPORTED;
  if (conv_w && (taps < 1 || taps > MAX_TAPS || !token_req || !slots || (taps > 1 && !conv_state))) return TL_ERR_UNSUPPORTED;
  const size_t smem = (size_t)width * sizeof(float);
  // four channels a thread where rows, weights and slots' rows start on 16-byte boundaries (and the stream count has
  // its own instance: the any-count kernel would spill)
  const bool vec = width % 4 == 0 && (n == 1 || n == 2 || n == 4);
  const bool wide = width / (vec ? 4 : 1) > 256;
  auto run = [&](auto kernel, auto* typed, int threads) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    tl::launch_kernel(kernel, (unsigned)count, threads, smem, stream, z, a, weight, bias, rows, typed, n, width, eps, centre, y,
                      mix, b, conv_w, conv_state, token_req, slots, taps, max_slots);
  };
  auto pick = [&](auto* typed) {
    using OutT = std::remove_pointer_t<decltype(typed)>;
#define TL_READ_NORM(NT, V)                                                         \
  switch (n) {                                                                      \
    case 1: run(read_norm_kernel<OutT, NT, 1, V>, typed, NT); break;                \
    case 2: run(read_norm_kernel<OutT, NT, 2, V>, typed, NT); break;                \
    case 4: run(read_norm_kernel<OutT, NT, 4, V>, typed, NT); break;                \
    default: run(read_norm_kernel<OutT, NT, 0, 1>, typed, NT); break;               \
  }
    if (vec && wide) {
      TL_READ_NORM(512, 4)
    } else if (vec) {
      TL_READ_NORM(NORM_NT, 4)
    } else if (wide) {
      TL_READ_NORM(512, 1)
    } else {
      TL_READ_NORM(NORM_NT, 1)
    }
#undef TL_READ_NORM
  };
  if (out_dtype == TL_DTYPE_F32) pick((float*)out);
  else pick((__nv_bfloat16*)out);
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
