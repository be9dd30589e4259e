// Latent attention: every token keeps ONE row [c (rank) | k_rot (rot)] in the cache, shared by
// all heads; a head's key is [W_uk,h c | k_rot] and its value W_uv,h c.  The kernels here run
// the attention in the latent space, which needs no expanded key or value of any cached token:
//
//   score(t, s, h) = scale * ( (W_uk,h^T q_plain[t,h]) . c_s + q_rot[t,h] . k_rot,s )
//   out[t, h]      = W_uv,h ( sum_s softmax_s(score) c_s )
//
// so that all heads read the same cached rows (a multi-query attention with key size rank + rot
// and value size rank over the cache, between two small per-head products).
//
//   prepare     one block per token: RMS norm of the query latent (-> compute type), RMS norm
//               of the key/value latent and rotation of the shared key part, both written into
//               the token's cache row; float32 inside;
//   absorb_q    one block per (8 tokens, head): rotate q_rot; fold W_uk,h into q_plain;
//   attention   one warp per (token, head), keys in tiles of 32 consecutive ABSOLUTE positions,
//               float32 scores, online softmax and sums: the order of every sum depends only on
//               the token's position, never on the cut, the batch or the pages (the true 32-bit
//               kernel and the any-size kernel);
//   expand_o    one block per (8 tokens, head): out[t, h] = W_uv,h o_lat[t, h].
// For many tokens the two per-head products run on the tensor cores instead (the mixer's choice).
//
// Rotation: entry i of the first ``dims`` entries pairs with i + dims/2, angle = float(p) *
// inv_freq[i] in float32; entries past ``dims`` pass unchanged.
// Cache layer: [page][slot in page][rank + rot] in the compute type T.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

template <typename T, int NT>
__global__ void __launch_bounds__(NT)
latent_prepare_kernel(const float* __restrict__ down, int down_stride, int q_rank, int kv_rank, int rot_dim,
                      int rot_dims, const float* __restrict__ q_norm, const float* __restrict__ kv_norm,
                      const float* __restrict__ inv_freq, float eps, const int* __restrict__ positions,
                      const int* __restrict__ token_req, const int* __restrict__ block_table, int table_width,
                      T* __restrict__ pages, int page_size, int num_pages, T* __restrict__ q_latent, int write_kv) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const float* row = down + (size_t)t * down_stride;
  if (q_rank > 0) {  // 0: the queries come straight from the layer's input, there is no query latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += NT) ss = fmaf(row[i], row[i], ss);
    ss = block_sum<NT>(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += NT)
      q_latent[(size_t)t * q_rank + i] = from_float<T>(row[i] * inv * q_norm[i]);
  }
  if (!write_kv) return;
  const float* kv = row + q_rank;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += NT) ss = fmaf(kv[i], kv[i], ss);
  ss = block_sum<NT>(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)kv_rank + eps);
  const int pos = positions[t];
  if (!TL_DEBUG_OK(pos >= 0 && pos / page_size < table_width, TL_DEBUG_POSITION, pos)) return;
  const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
  if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) return;
  T* dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot_dim);
  for (int i = threadIdx.x; i < kv_rank; i += NT) dst[i] = from_float<T>(kv[i] * inv * kv_norm[i]);
  const float* kr = kv + kv_rank;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < rot_dim; i += NT) {
    float v = kr[i];
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      float s, c;
      sincosf((float)pos * inv_freq[f], &s, &c);
      v = i < half ? kr[i] * c - kr[i + half] * s : kr[i] * c + kr[i - half] * s;
    }
    dst[kv_rank + i] = from_float<T>(v);
  }
}

// q: float32 [T, heads * (dim + rot_dim)];  uk: T [heads * dim, kv_rank];
// q_abs: T [T, heads, kv_rank + rot_dim].  A block takes up to TOKENS tokens of one head, so that a
// weight is read once for all of them.  ``fold`` 0: only the rotated part is written (the folded
// part comes from a tensor-core product) and ``plain_out`` (optional) receives q_plain in T.
constexpr int TOKENS = 8;

template <typename T, int NT>
__global__ void __launch_bounds__(NT)
latent_absorb_q_kernel(const float* __restrict__ q, int q_stride, const T* __restrict__ uk,
                       const float* __restrict__ inv_freq, const int* __restrict__ positions, T* __restrict__ q_abs,
                       T* __restrict__ plain_out, int tokens, int heads, int dim, int rot_dim, int rot_dims,
                       int kv_rank, int fold) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float plain[];  // TOKENS x dim floats
  const int t0 = blockIdx.x * TOKENS, h = blockIdx.y;
  const int count = tokens - t0 < TOKENS ? tokens - t0 : TOKENS;
  for (int e = threadIdx.x; e < TOKENS * dim; e += NT) {
    const int tt = e / dim, i = e - tt * dim;
    const float v = tt < count ? q[(size_t)(t0 + tt) * q_stride + (size_t)h * (dim + rot_dim) + i] : 0.f;
    plain[e] = v;
    if (plain_out && tt < count && blockIdx.z == 0) plain_out[((size_t)(t0 + tt) * heads + h) * dim + i] = from_float<T>(v);
  }
  __syncthreads();
  const int row = kv_rank + rot_dim;
  if (fold) {
    const T* w = uk + (size_t)h * dim * kv_rank;
    for (int r = blockIdx.z * NT + threadIdx.x; r < kv_rank; r += NT * gridDim.z) {
      float sum[TOKENS];
#pragma unroll
      for (int tt = 0; tt < TOKENS; ++tt) sum[tt] = 0.f;
#pragma unroll 4
      for (int d = 0; d < dim; ++d) {  // (unrolled by 16 it was slower: 197 against 150 us in a decode step of four such layers)
        const float wv = to_float(w[(size_t)d * kv_rank + r]);
#pragma unroll
        for (int tt = 0; tt < TOKENS; ++tt) sum[tt] = fmaf(plain[tt * dim + d], wv, sum[tt]);
      }
#pragma unroll
      for (int tt = 0; tt < TOKENS; ++tt)
        if (tt < count) q_abs[((size_t)(t0 + tt) * heads + h) * row + r] = from_float<T>(sum[tt]);
    }
  }
  if (blockIdx.z) return;
  const int half = rot_dims / 2;
  for (int e = threadIdx.x; e < count * rot_dim; e += NT) {
    const int tt = e / rot_dim, i = e - tt * rot_dim;
    const float* qr = q + (size_t)(t0 + tt) * q_stride + (size_t)h * (dim + rot_dim) + dim;
    float v = qr[i];
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      float sn, cs;
      sincosf((float)positions[t0 + tt] * inv_freq[f], &sn, &cs);
      v = i < half ? qr[i] * cs - qr[i + half] * sn : qr[i] * cs + qr[i - half] * sn;
    }
    q_abs[((size_t)(t0 + tt) * heads + h) * row + kv_rank + i] = from_float<T>(v);
  }
}

constexpr int WARPS = 4;
constexpr int MAX_DV = 1024;

template <typename T, bool VEC>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const T* __restrict__ q_abs, const T* __restrict__ pages, const int* __restrict__ block_table,
                        int table_width, const int* __restrict__ token_req, const int* __restrict__ positions,
                        T* __restrict__ out, int tokens, int heads, int dk, int dv, int page_size, float scale,
                        int num_pages) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  extern __shared__ float qs_all[];  // WARPS x dk
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = qs_all + (size_t)warp * dk;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)tokens * heads) return;
  const int t = (int)(item / heads);
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_req[t] * table_width;
  const T* qrow = q_abs + (size_t)item * dk;
  for (int i = lane; i < dk; i += 32) qs[i] = to_float(qrow[i]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[MAX_DV / 32];
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) acc[c] = 0.f;

  for (int start = 0; start <= pos; start += 32) {
    const int key = start + lane;
    const bool valid = key <= pos;
    float s = -INFINITY;
    size_t row_off = 0;
    if (valid) {
      int page = 0;
      if (TL_DEBUG_OK(key / page_size < table_width, TL_DEBUG_POSITION, key)) page = table[key / page_size];
      if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) page = 0;
      row_off = ((size_t)page * page_size + key % page_size) * dk;
      const T* krow = pages + row_off;
      float dot = 0.f;
      if (VEC) {
        for (int i = 0; i < dk; i += 8) {
          float kv[8];
          load8(krow + i, kv);
#pragma unroll
          for (int j = 0; j < 8; ++j) dot = fmaf(qs[i + j], kv[j], dot);
        }
      } else {
        for (int i = 0; i < dk; ++i) dot = fmaf(qs[i], to_float(krow[i]), dot);
      }
      s = dot * scale;
    }
    const float new_m = fmaxf(m, warp_max(s));
    const float corr = expf(m - new_m);  // first tile: exp(-inf) = 0
    const float p = valid ? expf(s - new_m) : 0.f;
    l = l * corr + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int c = 0; c < MAX_DV / 32; ++c) acc[c] *= corr;
    const int last = pos - start < 31 ? pos - start : 31;
    for (int j = 0; j <= last; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, j);
      const T* vrow = pages + off;
#pragma unroll
      for (int c = 0; c < MAX_DV / 32; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
      }
    }
  }
  T* orow = out + (size_t)item * dv;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < MAX_DV / 32; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) orow[i] = from_float<T>(acc[c] * inv);
  }
}

// o_lat: T [T, heads, kv_rank];  uv: T [heads * vdim, kv_rank];  out: T [T, heads * vdim].
// A block takes up to TOKENS tokens of one head; a warp a value channel at a time, lanes over
// the latent (8 consecutive entries a load where kv_rank is a multiple of 8).
constexpr int EXPAND_WARPS = 8;

template <typename T, bool VEC>
__global__ void __launch_bounds__(EXPAND_WARPS * 32)
latent_expand_o_kernel(const T* __restrict__ o_lat, const T* __restrict__ uv, T* __restrict__ out, int tokens,
                       int heads, int vdim, int kv_rank, const float* __restrict__ gate, int gate_stride) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float latent[];  // TOKENS x kv_rank floats
  const int t0 = blockIdx.x * TOKENS, h = blockIdx.y;
  const int count = tokens - t0 < TOKENS ? tokens - t0 : TOKENS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < TOKENS * kv_rank; e += EXPAND_WARPS * 32) {
    const int tt = e / kv_rank, i = e - tt * kv_rank;
    latent[e] = tt < count ? to_float(o_lat[((size_t)(t0 + tt) * heads + h) * kv_rank + i]) : 0.f;
  }
  __syncthreads();
  for (int v = blockIdx.z * EXPAND_WARPS + warp; v < vdim; v += EXPAND_WARPS * gridDim.z) {
    const T* w = uv + ((size_t)h * vdim + v) * kv_rank;
    float sum[TOKENS];
#pragma unroll
    for (int tt = 0; tt < TOKENS; ++tt) sum[tt] = 0.f;
    if (VEC) {
      for (int r = lane * 8; r < kv_rank; r += 256) {
        float wv[8];
        load8(w + r, wv);
#pragma unroll
        for (int tt = 0; tt < TOKENS; ++tt)
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[tt] = fmaf(latent[tt * kv_rank + r + j], wv[j], sum[tt]);
      }
    } else {
      for (int r = lane; r < kv_rank; r += 32) {
        const float wv = to_float(w[r]);
#pragma unroll
        for (int tt = 0; tt < TOKENS; ++tt) sum[tt] = fmaf(latent[tt * kv_rank + r], wv, sum[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < TOKENS; ++tt) {
      const float total = warp_sum(sum[tt]);
      if (lane == 0 && tt < count) {
        // gate (optional, float32 rows [tokens, heads * vdim]): the output is multiplied by sigmoid(gate)
        const float g = gate ? 1.f / (1.f + expf(-gate[(size_t)(t0 + tt) * gate_stride + (size_t)h * vdim + v])) : 1.f;
        out[(size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + v] = from_float<T>(total * g);
      }
    }
  }
}

}  // namespace

TL_DEBUG_READER(tl_latent_attention_debug_error)

extern "C" {

int tl_latent_prepare(const float* down, int down_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                      const float* q_norm, const float* kv_norm, const float* inv_freq, float eps,
                      const int* positions, const int* token_req, const int* block_table, int table_width, void* pages,
                      int dtype, int page_size, int num_pages, void* q_latent, int write_kv, int tokens,
                      cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims % 2 || rot_dims > rot_dim) return TL_ERR_UNSUPPORTED;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(latent_prepare_kernel<float, 128>, tokens, 128, 0, stream, down, down_stride, q_rank, kv_rank,
                      rot_dim, rot_dims, q_norm, kv_norm, inv_freq, eps, positions, token_req, block_table,
                      table_width, (float*)pages, page_size, num_pages, (float*)q_latent, write_kv);
  else
    tl::launch_kernel(latent_prepare_kernel<__nv_bfloat16, 128>, tokens, 128, 0, stream, down, down_stride, q_rank,
                      kv_rank, rot_dim, rot_dims, q_norm, kv_norm, inv_freq, eps, positions, token_req, block_table,
                      table_width, (__nv_bfloat16*)pages, page_size, num_pages, (__nv_bfloat16*)q_latent, write_kv);
  return TL_LAUNCH_CHECK();
}

int tl_latent_absorb_q(const float* q, int q_stride, const void* uk, int dtype, const float* inv_freq,
                       const int* positions, void* q_abs, void* plain_out, int tokens, int heads, int dim, int rot_dim,
                       int rot_dims, int kv_rank, int fold, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads > 65535 || rot_dims % 2 || rot_dims > rot_dim || dim > 1024) return TL_ERR_UNSUPPORTED;
  // few tokens: the folded entries of a head are spread over several blocks, so that the weights stream through
  // many SMs (64 entries a block); many tokens: the grid is large anyway
  const int chunks = (tokens + TOKENS - 1) / TOKENS;
  const int parts = (fold && chunks * heads < 256) ? (kv_rank + 63) / 64 : 1;
  dim3 grid(chunks, heads, parts);
  const size_t smem = (size_t)TOKENS * dim * sizeof(float);
  if (parts > 1) {
    if (dtype == TL_DTYPE_F32)
      tl::launch_kernel(latent_absorb_q_kernel<float, 64>, grid, 64, smem, stream, q, q_stride, (const float*)uk,
                        inv_freq, positions, (float*)q_abs, (float*)plain_out, tokens, heads, dim, rot_dim, rot_dims,
                        kv_rank, fold);
    else
      tl::launch_kernel(latent_absorb_q_kernel<__nv_bfloat16, 64>, grid, 64, smem, stream, q, q_stride,
                        (const __nv_bfloat16*)uk, inv_freq, positions, (__nv_bfloat16*)q_abs,
                        (__nv_bfloat16*)plain_out, tokens, heads, dim, rot_dim, rot_dims, kv_rank, fold);
    return TL_LAUNCH_CHECK();
  }
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(latent_absorb_q_kernel<float, 256>, grid, 256, smem, stream, q, q_stride, (const float*)uk,
                      inv_freq, positions, (float*)q_abs, (float*)plain_out, tokens, heads, dim, rot_dim, rot_dims,
                      kv_rank, fold);
  else
    tl::launch_kernel(latent_absorb_q_kernel<__nv_bfloat16, 256>, grid, 256, smem, stream, q, q_stride,
                      (const __nv_bfloat16*)uk, inv_freq, positions, (__nv_bfloat16*)q_abs, (__nv_bfloat16*)plain_out,
                      tokens, heads, dim, rot_dim, rot_dims, kv_rank, fold);
  return TL_LAUNCH_CHECK();
}

int tl_latent_attention(const void* q_abs, const void* pages, int dtype, const int* block_table, int table_width,
                        const int* token_req, const int* positions, void* out, int tokens, int heads, int dk, int dv,
                        int page_size, float scale, int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dv <= 0 || dv > MAX_DV || dv > dk || dk > 2048) return TL_ERR_UNSUPPORTED;
  const long long items = (long long)tokens * heads;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  const size_t smem = (size_t)WARPS * dk * sizeof(float);
  const bool vec = dk % 8 == 0;
#define TL_LATENT(T, VEC)                                                                                       \
  tl::launch_kernel(latent_attention_kernel<T, VEC>, blocks, WARPS * 32, smem, stream, (const T*)q_abs,         \
                    (const T*)pages, block_table, table_width, token_req, positions, (T*)out, tokens, heads, dk, \
                    dv, page_size, scale, num_pages)
  if (dtype == TL_DTYPE_F32) {
    if (vec) TL_LATENT(float, true); else TL_LATENT(float, false);
  } else {
    if (vec) TL_LATENT(__nv_bfloat16, true); else TL_LATENT(__nv_bfloat16, false);
  }
#undef TL_LATENT
  return TL_LAUNCH_CHECK();
}

int tl_latent_expand_o(const void* o_lat, const void* uv, void* out, int dtype, int tokens, int heads, int vdim,
                       int kv_rank, const float* gate, int gate_stride, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads > 65535 || kv_rank > 1024) return TL_ERR_UNSUPPORTED;
  const int chunks = (tokens + TOKENS - 1) / TOKENS;
  const int parts = chunks * heads < 256 ? (vdim + EXPAND_WARPS - 1) / EXPAND_WARPS : 1;  // few tokens: a warp a channel
  dim3 grid(chunks, heads, parts);
  const size_t smem = (size_t)TOKENS * kv_rank * sizeof(float);
  const bool vec = kv_rank % 8 == 0;
#define TL_EXPAND(T, VEC)                                                                                          \
  tl::launch_kernel(latent_expand_o_kernel<T, VEC>, grid, EXPAND_WARPS * 32, smem, stream, (const T*)o_lat,        \
                    (const T*)uv, (T*)out, tokens, heads, vdim, kv_rank, gate, gate_stride)
  if (dtype == TL_DTYPE_F32) {
    if (vec) TL_EXPAND(float, true); else TL_EXPAND(float, false);
  } else {
    if (vec) TL_EXPAND(__nv_bfloat16, true); else TL_EXPAND(__nv_bfloat16, false);
  }
#undef TL_EXPAND
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
