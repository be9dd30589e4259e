// The kernels around a selective state-space mixer (state-space duality) and around linear attention with
// an activation on q, k, v.  The recurrence itself is the scan of gla.cu (a D x V float32 state per head with one
// decay number per token and head); here is everything before and behind it, all float32 inside:
//
//   conv        the causal convolution over time of the channels [x | B | C] (weights [channels, taps], the LAST
//               column is the current token's; a bias), silu, the step size dt = softplus(dt_raw + bias) and the decay
//               exp(-exp(A_log) dt) of every head; writes the scan's rows [C (G N) | B (G N) | dt x (H V)], the
//               activated x and the decays.  Inputs before a step's first token of a request come from the request's
//               slot (the last taps - 1 raw inputs), zeros before the start of a sequence;
//   conv_state  moves the last taps - 1 raw inputs of every request into its slot (in a step of single tokens ``conv``
//               does that itself);
//   gated_norm  out = norm(y) * w with y = o (+ D_h x) and a gate: either y * act(gate) before the norm, or the norm
//               first and the gate behind it; the norm is an RMS norm over ``groups`` equal parts of the row;
//   activate    silu, in place, on the first columns of float32 rows;
//   gate_mul    rows *= sigmoid(gate rows), in the compute type;
//   token_gate  one number a token: sigmoid(w . x), float32.
//
// proj[t] = [ z (inner) | x B C (inner + 2 G N) | dt (H) ] are the float32 rows of the input product.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int NT = 256;
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (ceil(tokens / CONV_TOKENS), ceil(channels / NT)).  channels = inner + 2 G N.  A thread takes one channel through
// CONV_TOKENS consecutive tokens: its taps and bias stay in registers, and the last taps - 1 inputs slide along while the
// tokens belong to one request (a request's tokens are consecutive in a step), so an input is loaded once; where a
// request's portion begins inside the tile they are fetched anew, from the portion or from the request's slot.  The
// step sizes of the block's heads are taken once a (token, head) into shared memory, not once a channel.
constexpr int CONV_TOKENS = 8;

__global__ void __launch_bounds__(NT)
ssm_conv_kernel(const float* __restrict__ proj, int proj_stride, int xbc_offset, int dt_offset,
                const float* __restrict__ weight, const float* __restrict__ bias, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, float* state, const int* __restrict__ token_req,
                const int* __restrict__ req_indptr, const int* __restrict__ slots, float* __restrict__ scan_in,
                float* __restrict__ x_out, float* __restrict__ decay, int tokens, int channels, int taps, int heads,
                int vdim, int gn, int max_slots, int update_state, int tile) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float step[CONV_TOKENS][NT + 1];  // dt of (token of the tile, head of the block)
  __shared__ int tile_req[CONV_TOKENS], tile_slot[CONV_TOKENS], tile_place[CONV_TOKENS];
  const int t0 = blockIdx.x * tile;  // ``tile`` tokens a block: CONV_TOKENS, or 1 where a step has few tokens
  const int count = tokens - t0 < tile ? tokens - t0 : tile;
  if (threadIdx.x < count) {  // the tokens' request, slot and place in their request's portion, once a block
    const int req = token_req[t0 + threadIdx.x];
    tile_req[threadIdx.x] = req;
    tile_slot[threadIdx.x] = slots[req];
    tile_place[threadIdx.x] = t0 + threadIdx.x - req_indptr[req];
  }
  const int c_lo = blockIdx.y * NT, c = c_lo + threadIdx.x;
  const int inner = heads * vdim;
  const int scan_row = 2 * gn + inner;
  // the heads whose x channels this block holds (none where it holds only B and C)
  const int h_lo = c_lo < inner ? c_lo / vdim : 0;
  const int h_hi = c_lo < inner ? ((c_lo + NT - 1 < inner ? c_lo + NT - 1 : inner - 1) / vdim) : -1;
  const int nh = h_hi - h_lo + 1;
  for (int e = threadIdx.x; e < count * nh; e += NT) {
    const int tt = e / nh, h = h_lo + e - tt * nh;
    step[tt][h - h_lo] = softplus_f(proj[(size_t)(t0 + tt) * proj_stride + dt_offset + h] + dt_bias[h]);
  }
  if (blockIdx.y == 0) {  // the decays of all heads, once
    for (int e = threadIdx.x; e < count * heads; e += NT) {
      const int tt = e / heads, h = e - tt * heads;
      const int slot = slots[token_req[t0 + tt]];  // (before the barrier: not from shared memory)
      const float dt = softplus_f(proj[(size_t)(t0 + tt) * proj_stride + dt_offset + h] + dt_bias[h]);
      decay[(size_t)(t0 + tt) * heads + h] = slot >= 0 ? expf(-expf(a_log[h]) * dt) : 1.f;
    }
  }
  __syncthreads();
  if (c >= channels) return;
  float w[MAX_TAPS], win[MAX_TAPS];  // win[j]: the input taps - 1 - j tokens back; win[taps - 1]: the token's own
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    w[j] = j < taps ? weight[(size_t)c * taps + j] : 0.f;
    win[j] = 0.f;
  }
  const float b = bias[c];
  const int my_head = c < inner ? c / vdim - h_lo : 0;  // where this channel's step size lies in ``step``
  float own[CONV_TOKENS];  // the tokens' own inputs: all loads of the tile in flight at once
#pragma unroll
  for (int tt = 0; tt < CONV_TOKENS; ++tt)
    own[tt] = tt < count ? proj[(size_t)(t0 + tt) * proj_stride + xbc_offset + c] : 0.f;
  int prev_req = -1;
#pragma unroll
  for (int tt = 0; tt < CONV_TOKENS; ++tt) {
    if (tt >= count) break;
    const int t = t0 + tt;
    const int req = tile_req[tt];
    const int slot = tile_slot[tt];
    const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
    float act = 0.f;
    if (live) {
      const int i = tile_place[tt];  // the token's place in its request's portion
      float* old = state + (size_t)slot * (taps - 1) * channels;
      const float cur = own[tt];
      if (req == prev_req) {  // the same request as the token before: the inputs slide by one
#pragma unroll
        for (int j = 0; j < MAX_TAPS - 1; ++j)
          if (j < taps - 1) win[j] = win[j + 1];
      } else {
#pragma unroll
        for (int j = 0; j < MAX_TAPS - 1; ++j) {
          if (j >= taps - 1) continue;
          const int back = taps - 1 - j;
          win[j] = i - back >= 0 ? proj[(size_t)(t - back) * proj_stride + xbc_offset + c]
                                 : old[(size_t)(taps - 1 + i - back) * channels + c];
        }
      }
      float sum = b;
#pragma unroll
      for (int j = 0; j < MAX_TAPS; ++j) {  // ascending j: oldest input first
        if (j >= taps) continue;
        if (j == taps - 1) win[j] = cur;
        sum = fmaf(w[j], win[j], sum);
      }
      // a step of single tokens: this thread alone reads and writes the channel's rows of the slot, so it also moves
      // them up by one (the last row takes the token's own input)
      if (update_state) {
#pragma unroll
        for (int j = 1; j < MAX_TAPS; ++j)
          if (j < taps) old[(size_t)(j - 1) * channels + c] = win[j];
      }
      act = silu_f(sum);
      prev_req = req;
    } else {
      prev_req = -1;
    }
    if (c < inner) {
      x_out[(size_t)t * inner + c] = act;
      scan_in[(size_t)t * scan_row + 2 * gn + c] = step[tt][my_head] * act;
    } else if (c < inner + gn) {
      scan_in[(size_t)t * scan_row + gn + (c - inner)] = act;  // B: the scan's k
    } else {
      scan_in[(size_t)t * scan_row + (c - inner - gn)] = act;  // C: the scan's q
    }
  }
}

// grid (requests, ceil(channels / NT)); a thread moves one channel's rows, oldest first, so that a row of the old state
// is read before the same thread overwrites it.
__global__ void __launch_bounds__(NT)
ssm_conv_state_kernel(const float* __restrict__ proj, int proj_stride, int xbc_offset, float* __restrict__ state,
                      const int* __restrict__ req_indptr, const int* __restrict__ slots, int channels, int taps,
                      int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int req = blockIdx.x;
  const int c = blockIdx.y * NT + threadIdx.x;
  const int slot = slots[req];
  if (!(TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0) || c >= channels) return;
  const int first = req_indptr[req], n = req_indptr[req + 1] - first;
  float* rows = state + (size_t)slot * (taps - 1) * channels;
  for (int j = 0; j < taps - 1; ++j) {
    const int from = n - (taps - 1) + j;  // index into the portion; negative: a row of the old state
    rows[(size_t)j * channels + c] = from >= 0 ? proj[(size_t)(first + from) * proj_stride + xbc_offset + c]
                                               : rows[(size_t)(taps - 1 + from) * channels + c];
  }
}

// grid (tokens, groups).  y = o + skip[h] x (skip, x optional); gate_first: y *= act(gate), then the norm and the weight;
// else the norm and the weight, then *= act(gate).  gate_act: 0 silu, 1 sigmoid.  The gate is float32 rows.
// CACHED: the part's values (and, where the gate comes last, its factors) are kept in shared memory between the sum of
// squares and the output, so memory is read once; every thread has four elements' loads in flight at a time.  Parts too
// long for shared memory are read twice.
template <typename T, bool CACHED>
__global__ void __launch_bounds__(NT)
gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ x, const float* __restrict__ skip,
                  const float* __restrict__ gate, int gate_stride, const float* __restrict__ weight,
                  T* __restrict__ out, int width, int groups, int vdim, int gate_first, int gate_act, float eps) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float kept[];  // CACHED: part values, then (gate last) part factors
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = width / groups, c0 = blockIdx.y * part;
  const float* row = o + (size_t)t * width;
  const float* xr = x ? x + (size_t)t * width : nullptr;
  const float* g = gate + (size_t)t * gate_stride;
  float* factor = kept + part;
  float ss = 0.f;
  for (int base = threadIdx.x; base < part; base += 4 * NT) {
    float y[4], gv[4], xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {  // the loads of four elements first
      const int i = base + u * NT;
      const bool in = i < part;
      y[u] = in ? row[c0 + i] : 0.f;
      gv[u] = in ? g[c0 + i] : 0.f;
      xv[u] = (in && skip) ? xr[c0 + i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * NT;
      if (i >= part) break;
      float v = skip ? fmaf(skip[(c0 + i) / vdim], xv[u], y[u]) : y[u];
      const float a = gate_act ? sigmoid_f(gv[u]) : silu_f(gv[u]);
      if (gate_first) v *= a;
      ss = fmaf(v, v, ss);
      if (CACHED) {
        kept[i] = v;
        if (!gate_first) factor[i] = a;
      }
    }
  }
  ss = block_sum<NT>(ss, scratch);  // (its barriers also order the shared-memory writes before the reads below)
  const float inv = 1.f / sqrtf(ss / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += NT) {
    const int c = c0 + i;
    float v, a = 1.f;
    if (CACHED) {
      v = kept[i];
      if (!gate_first) a = factor[i];
    } else {
      v = skip ? fmaf(skip[c / vdim], xr[c], row[c]) : row[c];
      const float ga = gate_act ? sigmoid_f(g[c]) : silu_f(g[c]);
      if (gate_first) v *= ga; else a = ga;
    }
    out[(size_t)t * width + c] = from_float<T>(v * inv * weight[c] * a);
  }
}

// Four consecutive elements a thread where rows and columns allow 16-byte accesses, else one.
template <bool VEC>
__global__ void activate_kernel(float* __restrict__ rows, int stride, int cols, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
  if (e >= total) return;
  float* at = rows + (e / cols) * stride + e % cols;
  if (VEC) {
    float4 v = *reinterpret_cast<float4*>(at);
    v.x = silu_f(v.x); v.y = silu_f(v.y); v.z = silu_f(v.z); v.w = silu_f(v.w);
    *reinterpret_cast<float4*>(at) = v;
  } else {
    *at = silu_f(*at);
  }
}

template <typename T, bool VEC>
__global__ void gate_mul_kernel(T* __restrict__ rows, const float* __restrict__ gate, int gate_stride, int cols,
                                size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
  if (e >= total) return;
  const size_t t = e / cols;
  const int c = (int)(e % cols);
  if (VEC) {
    const float4 g = *reinterpret_cast<const float4*>(gate + t * gate_stride + c);
    T* at = rows + e;
    at[0] = from_float<T>(to_float(at[0]) * sigmoid_f(g.x));
    at[1] = from_float<T>(to_float(at[1]) * sigmoid_f(g.y));
    at[2] = from_float<T>(to_float(at[2]) * sigmoid_f(g.z));
    at[3] = from_float<T>(to_float(at[3]) * sigmoid_f(g.w));
  } else {
    rows[e] = from_float<T>(to_float(rows[e]) * sigmoid_f(gate[t * gate_stride + c]));
  }
}

// One warp a token: out[t] = sigmoid(w . x[t]); each lane sums its 32nd in ascending k.
template <typename T>
__global__ void __launch_bounds__(128)
token_gate_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, float* __restrict__ out, int tokens,
                  int hidden) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const T* row = x + (size_t)t * ldx;
  float p[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = 0.f;
  int k = lane;
  for (; k + 224 < hidden; k += 256) {  // eight independent chains, eight loads in flight a lane
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = fmaf(to_float(row[k + 32 * i]), w[k + 32 * i], p[i]);
  }
  for (; k < hidden; k += 32) p[0] = fmaf(to_float(row[k]), w[k], p[0]);
  float sum = warp_sum(((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7])));
  if (lane == 0) out[t] = sigmoid_f(sum);
}

}  // namespace

TL_DEBUG_READER(tl_ssm_debug_error)

extern "C" {

// scan_in float32 [tokens, 2 G N + H V]; x_out float32 [tokens, H V]; decay float32 [tokens, H];
// state float32 [max_slots, taps - 1, channels] (unused when taps == 1).
int tl_ssm_conv(const float* proj, int proj_stride, int xbc_offset, int dt_offset, const float* weight, const float* bias,
                const float* dt_bias, const float* a_log, const float* state, const int* token_req,
                const int* req_indptr, const int* slots, float* scan_in, float* x_out, float* decay, int tokens,
                int taps, int heads, int vdim, int gn, int max_slots, int update_state, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  // few tokens (a step of single tokens): a block a token, so that the tokens run side by side
  if (taps < 1 || taps > MAX_TAPS || heads <= 0 || vdim <= 0 || gn <= 0) return TL_ERR_UNSUPPORTED;
  const int channels = heads * vdim + 2 * gn;
  const int tile = tokens <= 8 * CONV_TOKENS ? 1 : CONV_TOKENS;
  dim3 grid((tokens + tile - 1) / tile, (channels + NT - 1) / NT);
  tl::launch_kernel(ssm_conv_kernel, grid, NT, 0, stream, proj, proj_stride, xbc_offset, dt_offset, weight, bias, dt_bias,
                    a_log, (float*)state, token_req, req_indptr, slots, scan_in, x_out, decay, tokens, channels, taps, heads,
                    vdim, gn, max_slots, update_state, tile);
  return TL_LAUNCH_CHECK();
}

int tl_ssm_conv_state(const float* proj, int proj_stride, int xbc_offset, float* state, const int* req_indptr,
                      const int* slots, int requests, int channels, int taps, int max_slots, cudaStream_t stream) {
  if (requests <= 0 || taps <= 1) return 0;
  if (taps > MAX_TAPS) return TL_ERR_UNSUPPORTED;
  dim3 grid(requests, (channels + NT - 1) / NT);
  tl::launch_kernel(ssm_conv_state_kernel, grid, NT, 0, stream, proj, proj_stride, xbc_offset, state, req_indptr, slots,
                    channels, taps, max_slots);
  return TL_LAUNCH_CHECK();
}

int tl_gated_norm(const float* o, const float* x, const float* skip, const float* gate, int gate_stride,
                  const float* weight, void* out, int out_dtype, int tokens, int width, int groups, int vdim,
                  int gate_first, int gate_act, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (groups <= 0 || width % groups || groups > 65535 || vdim <= 0) return TL_ERR_UNSUPPORTED;
  dim3 grid(tokens, groups);
  const size_t smem = (size_t)(width / groups) * (gate_first ? 1 : 2) * sizeof(float);
  const bool cached = smem <= 40 * 1024;
#define TL_NORM(T, CACHED)                                                                                          \
  tl::launch_kernel(gated_norm_kernel<T, CACHED>, grid, NT, CACHED ? smem : 0, stream, o, x, skip, gate, gate_stride, \
                    weight, (T*)out, width, groups, vdim, gate_first, gate_act, eps)
  if (out_dtype == TL_DTYPE_F32) {
    if (cached) TL_NORM(float, true); else TL_NORM(float, false);
  } else {
    if (cached) TL_NORM(__nv_bfloat16, true); else TL_NORM(__nv_bfloat16, false);
  }
#undef TL_NORM
  return TL_LAUNCH_CHECK();
}

int tl_activate_silu(float* rows, int stride, int tokens, int cols, cudaStream_t stream) {
  const size_t total = (size_t)tokens * cols;
  if (total == 0) return 0;
  if (cols % 4 == 0 && stride % 4 == 0 && (reinterpret_cast<uintptr_t>(rows) & 15) == 0)
    tl::launch_kernel(activate_kernel<true>, (unsigned)((total / 4 + 255) / 256), 256, 0, stream, rows, stride, cols, total);
  else
    tl::launch_kernel(activate_kernel<false>, (unsigned)((total + 255) / 256), 256, 0, stream, rows, stride, cols, total);
  return TL_LAUNCH_CHECK();
}

int tl_gate_mul(void* rows, int dtype, const float* gate, int gate_stride, int tokens, int cols, cudaStream_t stream) {
  const size_t total = (size_t)tokens * cols;
  if (total == 0) return 0;
  const bool vec = cols % 4 == 0 && gate_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0;
  const unsigned blocks = (unsigned)(((vec ? total / 4 : total) + 255) / 256);
#define TL_GATE(T, VEC) \
  tl::launch_kernel(gate_mul_kernel<T, VEC>, blocks, 256, 0, stream, (T*)rows, gate, gate_stride, cols, total)
  if (dtype == TL_DTYPE_F32) {
    if (vec) TL_GATE(float, true); else TL_GATE(float, false);
  } else {
    if (vec) TL_GATE(__nv_bfloat16, true); else TL_GATE(__nv_bfloat16, false);
  }
#undef TL_GATE
  return TL_LAUNCH_CHECK();
}

int tl_token_gate(const void* x, int ldx, int dtype, const float* w, float* out, int tokens, int hidden,
                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const unsigned blocks = (unsigned)((tokens + 3) / 4);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(token_gate_kernel<float>, blocks, 128, 0, stream, (const float*)x, ldx, w, out, tokens, hidden);
  else
    tl::launch_kernel(token_gate_kernel<__nv_bfloat16>, blocks, 128, 0, stream, (const __nv_bfloat16*)x, ldx, w, out,
                      tokens, hidden);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
