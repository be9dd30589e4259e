// Softmax attention over a sliding window of tokens PLUS one pooled key and value for every whole block
// of P tokens that lies before the window, all in one softmax:
//
//   query at position i sees   the tokens j with 0 <= i - j < size, and
//                              the blocks b with b P + P - 1 <= i - size   (nb(i) = floor((i - size + 1) / P) of them),
//   a block's key / value being the mean of its P cached keys / values.
//
// Keys may be wider or narrower than values (d, dv).  A token keeps ONE cache row per KV head, [key (d) | value (dv)],
// in pages [num_pages, 1, kv heads, page_size, d + dv] of the storage type T; pooled rows are float32 and live in
// the request's slot, pooled[slot, block, kv head, d + dv] (a slot has room for the engine's longest sequence).
//
// Kernels:
//   store      one block a token: its key and value rows go to its page; the token that completes a block
//              (position = b P + P - 1) also writes the block's means, summing the P rows in ascending position,
//              rows of this step from the projection (already of type T, as the cache holds them), older ones from
//              the pages, so the mean does not depend on how the sequence was cut into steps;
//   attention  one warp a (token, query head): pooled rows in tiles of 32 blocks, then the window's tokens in tiles
//              of 32 ABSOLUTE positions, online softmax, float32 throughout; the order of every sum depends on the
//              position alone.  The true 32-bit kernel and the any-size kernel of the bfloat16 engine.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(128)
pooled_store_kernel(const T* __restrict__ proj, int proj_stride, int k_offset, int v_offset, T* __restrict__ pages,
                    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
                    const int* __restrict__ positions, const int* __restrict__ req_indptr,
                    const int* __restrict__ slots, float* __restrict__ pooled, int max_blocks, int max_slots, int nkv,
                    int d, int dv, int page_size, int pool, int num_pages) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int t = blockIdx.x;
  const int req = token_req[t], pos = positions[t];
  const int row = d + dv;
  const int* table = block_table + (size_t)req * table_width;
  int page = 0;
  if (TL_DEBUG_OK(pos / page_size < table_width, TL_DEBUG_POSITION, pos)) page = table[pos / page_size];
  if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) page = 0;
  const T* mine = proj + (size_t)t * proj_stride;
  for (int e = threadIdx.x; e < nkv * row; e += blockDim.x) {
    const int g = e / row, c = e - g * row;
    const T v = c < d ? mine[k_offset + g * d + c] : mine[v_offset + g * dv + (c - d)];
    pages[(((size_t)page * nkv + g) * page_size + pos % page_size) * row + c] = v;
  }
  if ((pos + 1) % pool) return;
  const int slot = slots[req];
  if (!(TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0)) return;
  const int block = pos / pool;
  if (block >= max_blocks) return;
  const int first = req_indptr[req];     // the request's first token of this step ...
  const int first_pos = positions[first];  // ... and its position: older rows are in the pages
  float* out = pooled + (((size_t)slot * max_blocks + block) * nkv) * row;
  const float inv = 1.f / (float)pool;
  for (int e = threadIdx.x; e < nkv * row; e += blockDim.x) {
    const int g = e / row, c = e - g * row;
    float sum = 0.f;
    for (int p = pos - pool + 1; p <= pos; ++p) {
      float v;
      if (p >= first_pos) {
        const T* theirs = proj + (size_t)(first + (p - first_pos)) * proj_stride;
        v = to_float(c < d ? theirs[k_offset + g * d + c] : theirs[v_offset + g * dv + (c - d)]);
      } else {
        int pg = 0;
        if (TL_DEBUG_OK(p / page_size < table_width, TL_DEBUG_POSITION, p)) pg = table[p / page_size];
        if (!TL_DEBUG_OK(pg >= 0 && pg < num_pages, TL_DEBUG_PAGE, pg)) pg = 0;
        v = to_float(pages[(((size_t)pg * nkv + g) * page_size + p % page_size) * row + c]);
      }
      sum += v;
    }
    out[e] = sum * inv;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
pooled_attention_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
                        const int* __restrict__ positions, const int* __restrict__ slots,
                        const float* __restrict__ pooled, int max_blocks, int max_slots, T* __restrict__ out,
                        int out_stride, int tokens, int nh, int nkv, int d, int dv, int page_size, int size, int pool,
                        float scale, int num_pages) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int req = token_req[t];
  const int lo = pos - size + 1 > 0 ? pos - size + 1 : 0;
  const int slot = slots[req];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  int blocks = (pool > 0 && live && pos - size + 1 > 0) ? (pos - size + 1) / pool : 0;
  if (blocks > max_blocks) blocks = max_blocks;
  const int* table = block_table + (size_t)req * table_width;
  const int row = d + dv;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = to_float(qrow[i]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) acc[c] = 0.f;

  // the pooled blocks, oldest first
  const float* mine = pooled + ((size_t)(live ? slot : 0) * max_blocks * nkv + kvh) * row;
  for (int start = 0; start < blocks; start += 32) {
    const int b = start + lane;
    const bool valid = b < blocks;
    float s = -INFINITY;
    if (valid) {
      const float* krow = mine + (size_t)b * nkv * row;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[warp][i], krow[i], dot);
      s = dot * scale;
    }
    const float new_m = fmaxf(m, warp_max(s));
    const float corr = expf(m - new_m);
    const float p = valid ? expf(s - new_m) : 0.f;
    l = l * corr + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] *= corr;
    const int last = blocks - start < 32 ? blocks - start : 32;
    for (int j = 0; j < last; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vrow = mine + (size_t)(start + j) * nkv * row + d;
#pragma unroll
      for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] = fmaf(pj, vrow[i], acc[c]);
      }
    }
  }

  // the window's tokens
  for (int start = lo & ~31; start <= pos; start += 32) {
    const int key = start + lane;
    const bool valid = key >= lo && key <= pos;
    float s = -INFINITY;
    size_t row_off = 0;
    if (valid) {
      int page = 0;
      if (TL_DEBUG_OK(key / page_size < table_width, TL_DEBUG_POSITION, key)) page = table[key / page_size];
      if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) page = 0;
      row_off = (((size_t)page * nkv + kvh) * page_size + key % page_size) * row;
      const T* krow = pages + row_off;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[warp][i], to_float(krow[i]), dot);
      s = dot * scale;
    }
    const float new_m = fmaxf(m, warp_max(s));
    const float corr = expf(m - new_m);
    const float p = valid ? expf(s - new_m) : 0.f;
    l = l * corr + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] *= corr;
    const int first = lo > start ? lo - start : 0;
    const int last = pos - start < 31 ? pos - start : 31;
    for (int j = first; j <= last; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, j);
      const T* vrow = pages + off + d;
#pragma unroll
      for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
      }
    }
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) orow[i] = from_float<T>(acc[c] * inv);
  }
}

}  // namespace

TL_DEBUG_READER(tl_pooled_attention_debug_error)

extern "C" {

// proj rows hold the keys at k_offset (nkv x d) and the values at v_offset (nkv x dv).
int tl_pooled_store(const void* proj, int proj_stride, int k_offset, int v_offset, void* pages, int dtype,
                    const int* block_table, int table_width, const int* token_req, const int* positions,
                    const int* req_indptr, const int* slots, float* pooled, int max_blocks, int max_slots, int tokens,
                    int nkv, int d, int dv, int page_size, int pool, int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || pool <= 0) return TL_ERR_UNSUPPORTED;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(pooled_store_kernel<float>, (unsigned)tokens, 128, 0, stream, (const float*)proj, proj_stride,
                      k_offset, v_offset, (float*)pages, block_table, table_width, token_req, positions, req_indptr,
                      slots, pooled, max_blocks, max_slots, nkv, d, dv, page_size, pool, num_pages);
  else
    tl::launch_kernel(pooled_store_kernel<__nv_bfloat16>, (unsigned)tokens, 128, 0, stream,
                      (const __nv_bfloat16*)proj, proj_stride, k_offset, v_offset, (__nv_bfloat16*)pages, block_table,
                      table_width, token_req, positions, req_indptr, slots, pooled, max_blocks, max_slots, nkv, d, dv,
                      page_size, pool, num_pages);
  return TL_LAUNCH_CHECK();
}

int tl_pooled_attention(const void* q, int q_stride, const void* pages, int dtype, const int* block_table,
                        int table_width, const int* token_req, const int* positions, const int* slots,
                        const float* pooled, int max_blocks, int max_slots, void* out, int out_stride, int tokens, int nh,
                        int nkv, int d, int dv, int page_size, int size, int pool, float scale, int num_pages,
                        cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || nkv <= 0 || nh % nkv || page_size <= 0 || size <= 0 || pool < 0)
    return TL_ERR_UNSUPPORTED;
  const long long items = (long long)tokens * nh;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(pooled_attention_kernel<float>, blocks, WARPS * 32, 0, stream, (const float*)q, q_stride,
                      (const float*)pages, block_table, table_width, token_req, positions, slots, pooled, max_blocks,
                      max_slots, (float*)out, out_stride, tokens, nh, nkv, d, dv, page_size, size, pool, scale,
                      num_pages);
  else
    tl::launch_kernel(pooled_attention_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, (const __nv_bfloat16*)q,
                      q_stride, (const __nv_bfloat16*)pages, block_table, table_width, token_req, positions, slots,
                      pooled, max_blocks, max_slots, (__nv_bfloat16*)out, out_stride, tokens, nh, nkv, d, dv, page_size,
                      size, pool, scale, num_pages);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
