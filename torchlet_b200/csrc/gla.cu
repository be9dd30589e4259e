// Gated linear attention: a recurrent mixer whose per-request state is one D x V float32 matrix
// per head (key channel i, value channel j), carried from token to token:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t * qscale
//
// with a decay per key channel a = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau), z = W2 l + b, where
// l is a low-rank projection of the layer's input.  Everything here is float32, also in the bfloat16
// engine: the projections arrive as float32 rows
//   proj[t] = [ q (H D) | k (H D) | v (H V) | g (H V) | l (rank) ].
//
// Three kernels:
//   decay   one block per (8 tokens, 128 channels): a of every key channel;
//   scan    one block per (request, head, 32 value channels): the columns of S are independent of one
//           another; four lanes share a column, each keeps a quarter of it in registers, and the block
//           walks the request's tokens of this step in order; q, k, a, v of a few tokens at a time are
//           staged in shared memory (four stages, asynchronous copies).  The state row of the request's slot
//           is read at the start and written back at the end, so a prompt cut into portions, or
//           decoded token by token, runs the same additions in the same order as the whole prompt;
//   finish  one warp per (token, head): o / rms(o) * weight * silu(g) in the compute type (the
//           weight covers one head and is shared by all).
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int DECAY_TOKENS = 8;
constexpr int DECAY_NT = 128;

// w2t: W2 transposed, [rank, channels]; out: [tokens, channels].
__global__ void __launch_bounds__(DECAY_NT)
gla_decay_kernel(const float* __restrict__ proj, int proj_stride, int low_offset, const float* __restrict__ w2t,
                 const float* __restrict__ bias, float* __restrict__ out, int tokens, int channels, int rank,
                 float inv_tau) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float low[];  // DECAY_TOKENS x rank
  const int t0 = blockIdx.x * DECAY_TOKENS;
  const int count = tokens - t0 < DECAY_TOKENS ? tokens - t0 : DECAY_TOKENS;
  for (int e = threadIdx.x; e < DECAY_TOKENS * rank; e += DECAY_NT) {
    const int tt = e / rank, j = e - tt * rank;
    low[e] = tt < count ? proj[(size_t)(t0 + tt) * proj_stride + low_offset + j] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * DECAY_NT + threadIdx.x;
  if (c >= channels) return;
  float z[DECAY_TOKENS];
#pragma unroll
  for (int tt = 0; tt < DECAY_TOKENS; ++tt) z[tt] = 0.f;
#pragma unroll 8
  for (int j = 0; j < rank; ++j) {  // ascending j: the order depends on the rank alone
    const float w = w2t[(size_t)j * channels + c];
#pragma unroll
    for (int tt = 0; tt < DECAY_TOKENS; ++tt) z[tt] = fmaf(w, low[tt * rank + j], z[tt]);
  }
  const float b = bias[c];
#pragma unroll
  for (int tt = 0; tt < DECAY_TOKENS; ++tt) {
    if (tt >= count) break;
    const float x = z[tt] + b;
    // log(sigmoid(x)) = min(x, 0) - log1p(exp(-|x|))
    const float logsig = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
    out[(size_t)(t0 + tt) * channels + c] = expf(logsig * inv_tau);
  }
}

__device__ __forceinline__ void copy16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void copy4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One block per (request, head, COLS value channels), KS * COLS threads.  KS (four or eight) lanes share a
// column of S (value channel j): lane part p keeps the key channels i with (i / 4) % KS == p, DK / KS of them
// (DK: the key size rounded up to 16, 32, 64, 128 or 256), and the sum over i of a token's S^T q meets
// by two or three shuffles.  Every warp reads the same staged q, k, a of CHUNK tokens, STAGES stages deep: while
// the block walks one chunk, the next three are on their way (a chunk's copies take longer than its
// arithmetic).  A token costs a block 3 DK / 4 shared-memory reads of 16 bytes a warp, which is what bounds
// a block of many warps; hence few columns a block, and more blocks.
// Lanes that share a column: four, or eight at key sizes from 128 on (a lane's share of the column, and with it the
// chain of additions a token, stays at most 32 long, and a block has eight warps to hide the chain's waits behind).
__host__ __device__ constexpr int lanes_a_column(int dk) { return dk >= 128 ? 8 : 4; }
constexpr int COLS = 32;
constexpr int STAGES = 4;

// MODE says what ``decay`` holds: DECAY_ROWS a row [heads * dim] per token (one number a key channel), DECAY_HEAD one
// constant per head (``heads`` numbers; a retention), DECAY_TOKEN one number per (token, head) for all of the head's
// key channels (a selective state space).  ``qk_heads``: q and k have that many heads (a divisor of ``heads``), head h
// reading q/k head h / (heads / qk_heads); the rows are [ q (qk_heads D) | k (qk_heads D) | v (heads V) | ... ].
constexpr int DECAY_ROWS = 0, DECAY_HEAD = 1, DECAY_TOKEN = 2;
template <int DK, bool VEC, int MODE>
__global__ void __launch_bounds__(lanes_a_column(DK) * COLS)
gla_scan_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ decay,
                const int* __restrict__ req_indptr, const int* __restrict__ slots, float* __restrict__ state,
                float* __restrict__ out, int heads, int qk_heads, int dim, int vdim, int max_slots, float qscale) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  constexpr bool FIXED = MODE != DECAY_ROWS;  // no decay row is staged
  constexpr int KS = lanes_a_column(DK);
  constexpr int PER = DK / KS;
  // a staged token: q, k, (a: only where the decay is a row a token), v, the token's decay number.  Without the a
  // row a stage holds twice as many tokens of the larger key sizes, and the walk meets half as many barriers.
  constexpr int VOFF = (FIXED ? 2 : 3) * DK;
  constexpr int CHUNK = FIXED ? (DK <= 128 ? 8 : 4) : (DK <= 64 ? 8 : (DK <= 128 ? 4 : 2));
  constexpr int row = VOFF + COLS + 4;
  __shared__ __align__(16) float stage[STAGES * CHUNK * row];  // [STAGES][CHUNK]
  constexpr int NT = KS * COLS;
  const int req = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int col0 = blockIdx.z * COLS;  // this block's value channels: col0 .. col0 + COLS
  const int cols_here = vdim - col0 < COLS ? vdim - col0 : COLS;
  const int part = tid % KS, col = col0 + tid / KS;
  const bool on = col < vdim;
  const int hd = qk_heads * dim, hv = heads * vdim;
  const int hq = h / (heads / qk_heads);  // the q/k head this head reads
  const int first = req_indptr[req], last = req_indptr[req + 1];
  const int slot = slots[req];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  if (!live) {  // a padding lane of a captured step: no state is touched
    if (part == 0 && on)
      for (int t = first; t < last; ++t) out[(size_t)t * hv + h * vdim + col] = 0.f;
    return;
  }
  // entries past dim (and past vdim) stay zero in both stages
  for (int e = tid; e < STAGES * CHUNK * row; e += NT) stage[e] = 0.f;
  __syncthreads();
  auto fetch = [&](int base, int buf) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    float* dst = stage + (size_t)buf * CHUNK * row;
    if (VEC) {
      const int qd = dim >> 2, qv = cols_here >> 2, per_token = (FIXED ? 2 : 3) * qd + qv + (MODE == DECAY_TOKEN ? 1 : 0);
      for (int e = tid; e < count * per_token; e += NT) {
        const int tt = e / per_token, rest = e - tt * per_token;
        const int t = base + tt;
        const float* src;
        float* to;
        if (rest < 2 * qd) {  // q, k
          const int what = rest / qd, q4 = rest - what * qd;
          src = proj + (size_t)t * proj_stride + what * hd + hq * dim + 4 * q4;
          to = dst + tt * row + what * DK + 4 * q4;
        } else if (!FIXED && rest < 3 * qd) {
          const int q4 = rest - 2 * qd;
          src = decay + (size_t)t * heads * dim + h * dim + 4 * q4;
          to = dst + tt * row + 2 * DK + 4 * q4;
        } else if (MODE == DECAY_TOKEN && rest == per_token - 1) {
          copy4(dst + tt * row + VOFF + COLS, decay + (size_t)t * heads + h);
          continue;
        } else {
          const int q4 = rest - (FIXED ? 2 : 3) * qd;
          src = proj + (size_t)t * proj_stride + 2 * hd + h * vdim + col0 + 4 * q4;
          to = dst + tt * row + VOFF + 4 * q4;
        }
        copy16(to, src);
      }
    } else {
      const int per_token = (FIXED ? 2 : 3) * dim + cols_here + (MODE == DECAY_TOKEN ? 1 : 0);
      for (int e = tid; e < count * per_token; e += NT) {
        const int tt = e / per_token, rest = e - tt * per_token;
        const int t = base + tt;
        const float* src;
        float* to;
        if (rest < 2 * dim) {
          const int what = rest / dim, i = rest - what * dim;
          src = proj + (size_t)t * proj_stride + what * hd + hq * dim + i;
          to = dst + tt * row + what * DK + i;
        } else if (!FIXED && rest < 3 * dim) {
          const int i = rest - 2 * dim;
          src = decay + (size_t)t * heads * dim + h * dim + i;
          to = dst + tt * row + 2 * DK + i;
        } else if (MODE == DECAY_TOKEN && rest == per_token - 1) {
          src = decay + (size_t)t * heads + h;
          to = dst + tt * row + VOFF + COLS;
        } else {
          const int i = rest - (FIXED ? 2 : 3) * dim;
          src = proj + (size_t)t * proj_stride + 2 * hd + h * vdim + col0 + i;
          to = dst + tt * row + VOFF + i;
        }
        copy4(to, src);
      }
    }
    copies_commit();
  };
  for (int s = 0; s < STAGES - 1; ++s) {  // always STAGES - 1 groups in flight (some of them empty)
    if (first + s * CHUNK < last) fetch(first + s * CHUNK, s);
    else copies_commit();
  }

  // this lane's key channels: i = 4 (n / 4 * KS + part) + n % 4
  float* mine = state + ((size_t)slot * heads + h) * dim * vdim;
  float S[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = 4 * ((n >> 2) * KS + part) + (n & 3);
    S[n] = (on && i < dim) ? mine[(size_t)i * vdim + col] : 0.f;
  }

  const float head_decay = MODE == DECAY_HEAD ? decay[h] : 0.f;
  int buf = 0;
  for (int base = first; base < last; base += CHUNK, buf = (buf + 1) % STAGES) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    // the stage that the chunk before this one used is free (the barrier at the end of its walk)
    if (base + (STAGES - 1) * CHUNK < last) fetch(base + (STAGES - 1) * CHUNK, (buf + STAGES - 1) % STAGES);
    else copies_commit();
    copies_wait<STAGES - 1>();  // all but the newest STAGES - 1 groups: this chunk has landed
    __syncthreads();
    const float* chunk = stage + (size_t)buf * CHUNK * row;
    for (int tt = 0; tt < count; ++tt) {
      const float* tok = chunk + tt * row;
      const float4* q4 = reinterpret_cast<const float4*>(tok);
      const float4* k4 = reinterpret_cast<const float4*>(tok + DK);
      const float4* a4 = reinterpret_cast<const float4*>(tok + 2 * DK);
      const float v = tok[VOFF + (on ? col - col0 : 0)];
      const float fixed = MODE == DECAY_TOKEN ? tok[VOFF + COLS] : head_decay;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int n = 0; n < PER / 4; ++n) {
        const float4 a = FIXED ? make_float4(fixed, fixed, fixed, fixed) : a4[n * KS + part];
        const float4 k = k4[n * KS + part], q = q4[n * KS + part];
        S[4 * n] = fmaf(k.x, v, a.x * S[4 * n]);
        S[4 * n + 1] = fmaf(k.y, v, a.y * S[4 * n + 1]);
        S[4 * n + 2] = fmaf(k.z, v, a.z * S[4 * n + 2]);
        S[4 * n + 3] = fmaf(k.w, v, a.w * S[4 * n + 3]);
        o0 = fmaf(q.x, S[4 * n], o0);
        o1 = fmaf(q.y, S[4 * n + 1], o1);
        o2 = fmaf(q.z, S[4 * n + 2], o2);
        o3 = fmaf(q.w, S[4 * n + 3], o3);
      }
      float o = (o0 + o1) + (o2 + o3);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (KS == 8) o += __shfl_xor_sync(0xffffffffu, o, 4);
      if (on && part == 0) out[(size_t)(base + tt) * hv + h * vdim + col] = o * qscale;
    }
    __syncthreads();  // the stage is free for the chunk after the next
  }
  if (on) {
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = 4 * ((n >> 2) * KS + part) + (n & 3);
      if (i < dim) mine[(size_t)i * vdim + col] = S[n];
    }
  }
}

constexpr int FINISH_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(FINISH_WARPS * 32)
gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int proj_stride, int gate_offset,
                  const float* __restrict__ weight, T* __restrict__ out, long long items, int heads, int vdim,
                  float eps) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * FINISH_WARPS + warp;
  if (item >= items) return;
  const long long t = item / heads;
  const int h = (int)(item % heads);
  const int hv = heads * vdim;
  const float* row = o + (size_t)t * hv + h * vdim;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(row[i], row[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  const float* gate = proj + (size_t)t * proj_stride + gate_offset + h * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float g = gate[i];
    out[(size_t)t * hv + h * vdim + i] = from_float<T>(row[i] * inv * (weight ? weight[i] : 1.f) * (g / (1.f + expf(-g))));
  }
}

// Split-half rotation of the first ``dims`` entries of ``heads`` consecutive heads of ``dim`` entries in float32
// rows, in place: entry i (< dims / 2) pairs with i + dims / 2, angle = float(position) * inv_freq[i].
__global__ void rotate_heads_kernel(float* __restrict__ rows, int stride, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int heads, int dim, int half, size_t total) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int i = (int)(e % half);
  const int h = (int)((e / half) % heads);
  const size_t t = e / ((size_t)half * heads);
  float s, c;
  sincosf((float)positions[t] * inv_freq[i], &s, &c);
  float* head = rows + t * stride + (size_t)h * dim;
  const float u = head[i], v = head[i + half];
  head[i] = u * c - v * s;
  head[i + half] = v * c + u * s;
}

}  // namespace

TL_DEBUG_READER(tl_gla_debug_error)

extern "C" {

// decay: float32 [tokens, channels] scratch; w2t: [rank, channels]; the low-rank input is
// proj[t, low_offset : low_offset + rank].
int tl_gla_decay(const float* proj, int proj_stride, int low_offset, const float* w2t, const float* bias, float* decay,
                 int tokens, int channels, int rank, float tau, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || rank <= 0 || rank > 1024 || !(tau > 0.f)) return TL_ERR_UNSUPPORTED;
  dim3 grid((tokens + DECAY_TOKENS - 1) / DECAY_TOKENS, (channels + DECAY_NT - 1) / DECAY_NT);
  if (grid.y > 65535) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(gla_decay_kernel, grid, DECAY_NT, (size_t)DECAY_TOKENS * rank * sizeof(float), stream, proj,
                    proj_stride, low_offset, w2t, bias, decay, tokens, channels, rank, 1.f / tau);
  return TL_LAUNCH_CHECK();
}

// state: float32 [max_slots, heads, dim, vdim]; out: float32 [tokens, heads * vdim].
// decay_mode: 0 ``decay`` holds [tokens, heads * dim] rows, 1 one constant per head, 2 [tokens, heads] (one number per
// token and head).  qk_heads: how many heads q and k have (divides heads).
int tl_gla_scan(const float* proj, int proj_stride, const float* decay, const int* req_indptr, const int* slots,
                float* state, float* out, int requests, int heads, int qk_heads, int dim, int vdim, int max_slots,
                float qscale, int decay_mode, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (dim <= 0 || dim > 256 || vdim <= 0 || vdim > 256 || heads > 65535) return TL_ERR_UNSUPPORTED;
  if (qk_heads <= 0 || heads % qk_heads || decay_mode < 0 || decay_mode > 2) return TL_ERR_UNSUPPORTED;
  const bool fixed_decay = decay_mode != DECAY_ROWS;
  dim3 grid(requests, heads, (vdim + COLS - 1) / COLS);
  const bool vec = dim % 4 == 0 && vdim % 4 == 0 && proj_stride % 4 == 0 && (qk_heads * dim) % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(proj) & 15) == 0 &&
                   (fixed_decay || (reinterpret_cast<uintptr_t>(decay) & 15) == 0);
#define TL_SCAN_ONE(DK, VEC, MODE)                                                                                 \
  tl::launch_kernel(gla_scan_kernel<DK, VEC, MODE>, grid, lanes_a_column(DK) * COLS, 0, stream, proj, proj_stride, decay, req_indptr, \
                    slots, state, out, heads, qk_heads, dim, vdim, max_slots, qscale)
#define TL_SCAN(DK)                                                                \
  {                                                                                \
    if (vec && decay_mode == DECAY_HEAD) TL_SCAN_ONE(DK, true, DECAY_HEAD);        \
    else if (vec && decay_mode == DECAY_TOKEN) TL_SCAN_ONE(DK, true, DECAY_TOKEN); \
    else if (vec) TL_SCAN_ONE(DK, true, DECAY_ROWS);                               \
    else if (decay_mode == DECAY_HEAD) TL_SCAN_ONE(DK, false, DECAY_HEAD);         \
    else if (decay_mode == DECAY_TOKEN) TL_SCAN_ONE(DK, false, DECAY_TOKEN);       \
    else TL_SCAN_ONE(DK, false, DECAY_ROWS);                                       \
  }
  if (dim <= 16) TL_SCAN(16)
  else if (dim <= 32) TL_SCAN(32)
  else if (dim <= 64) TL_SCAN(64)
  else if (dim <= 128) TL_SCAN(128)
  else TL_SCAN(256)
#undef TL_SCAN
#undef TL_SCAN_ONE
  return TL_LAUNCH_CHECK();
}

int tl_rotate_heads_f32(float* rows, int stride, const int* positions, const float* inv_freq, int tokens, int heads,
                        int dim, int dims, cudaStream_t stream) {
  if (tokens <= 0 || dims <= 0) return 0;
  if (dims % 2 || dims > dim || heads <= 0) return TL_ERR_UNSUPPORTED;
  const size_t total = (size_t)tokens * heads * (dims / 2);
  tl::launch_kernel(rotate_heads_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, rows, stride, positions,
                    inv_freq, heads, dim, dims / 2, total);
  return TL_LAUNCH_CHECK();
}

int tl_gla_finish(const float* o, const float* proj, int proj_stride, int gate_offset, const float* weight, void* out,
                  int out_dtype, int tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  const long long items = (long long)tokens * heads;
  if (items <= 0) return 0;
  const unsigned blocks = (unsigned)((items + FINISH_WARPS - 1) / FINISH_WARPS);
  if (out_dtype == TL_DTYPE_F32)
    tl::launch_kernel(gla_finish_kernel<float>, blocks, FINISH_WARPS * 32, 0, stream, o, proj, proj_stride,
                      gate_offset, weight, (float*)out, items, heads, vdim, eps);
  else
    tl::launch_kernel(gla_finish_kernel<__nv_bfloat16>, blocks, FINISH_WARPS * 32, 0, stream, o, proj, proj_stride,
                      gate_offset, weight, (__nv_bfloat16*)out, items, heads, vdim, eps);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
