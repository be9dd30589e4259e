// Softmax attention over a sliding window of tokens PLUS one pooled key and value for every whole block
// of P tokens that lies before the window, all in one softmax:
//
//   query at position i sees   the tokens j with 0 <= i - j < size, and
//                              the blocks b with b P + P - 1 <= i - size   (nb(i) = floor((i - size + 1) / P) of them),
//   a block's key / value being the mean of its P cached keys / values.
//
// Keys may be wider or narrower than values (d, dv).  A token's cache rows are in pages of the storage type T, in one
// of two layouts: JOINED, one row per KV head, [key (d) | value (dv)], pages [num_pages, 1, kv heads, page_size, d + dv];
// or, where d = dv, SPLIT into a key plane and a value plane, pages [num_pages, 2, kv heads, page_size, d], which is
// what the tensor-core attention kernels read.  Pooled rows are float32 and live in the request's slot,
// pooled[slot, block, kv head, d + dv] (a slot has room for the engine's longest sequence).
//
// Kernels:
//   store      one block a token copies its key and value rows to its page, one more a KV head writes the block's mean
//              row where the token completes a block: the token that completes a block
//              (position = b P + P - 1) also writes the block's means, summing the P rows in ascending position,
//              rows of this step from the projection (already of type T, as the cache holds them), older ones from
//              the pages, so the mean does not depend on how the sequence was cut into steps;
//   attention  one warp a (token, query head): pooled rows in tiles of 32 blocks, then the window's tokens in tiles
//              of 32 ABSOLUTE positions, online softmax, float32 throughout; the order of every sum depends on the
//              position alone.  The true 32-bit kernel and the any-size kernel of the bfloat16 engine.
//   prior      one warp a (token, query head): the softmax state over the pooled rows ALONE (max in log2 units of the
//              scaled score, sum, unnormalized weighted values, float32), which the tensor-core kernels that walk the
//              window's tokens (attention_mma.cu, attention_tc.cu) join where they normalize a row.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

// Where the rows of (page, KV head, place in the page) start, in elements.
struct Layout {
  size_t page_stride, v_base;
  int row;
  __device__ Layout(int split, int nkv, int d, int dv, int page_size) {
    row = split ? d : d + dv;
    page_stride = (size_t)(split ? 2 : 1) * nkv * page_size * row;
    v_base = split ? (size_t)nkv * page_size * d : (size_t)d;
  }
  __device__ size_t key(int page, int g, int place, int page_size) const {
    return (size_t)page * page_stride + ((size_t)g * page_size + place) * row;
  }
  __device__ size_t value(int page, int g, int place, int page_size) const { return key(page, g, place, page_size) + v_base; }
};

// Grid (tokens, 1 + nkv): block (t, 0) copies the token's rows into its page; block (t, 1 + g) leaves at once unless
// the token completes a block of ``pool`` tokens, and then writes the mean row of KV head g.
template <typename T>
__global__ void __launch_bounds__(128)
pooled_store_kernel(const T* __restrict__ proj, int proj_stride, int k_offset, int v_offset, T* __restrict__ pages,
                    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
                    const int* __restrict__ positions, const int* __restrict__ req_indptr,
                    const int* __restrict__ slots, float* __restrict__ pooled, int max_blocks, int max_slots, int nkv,
                    int d, int dv, int page_size, int pool, int num_pages, int split) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const Layout at(split, nkv, d, dv, page_size);
  const int t = blockIdx.x;
  const int req = token_req[t], pos = positions[t];
  const int row = d + dv;
  const int* table = block_table + (size_t)req * table_width;
  const T* mine = proj + (size_t)t * proj_stride;
  if (blockIdx.y == 0) {
    int page = 0;
    if (TL_DEBUG_OK(pos / page_size < table_width, TL_DEBUG_POSITION, pos)) page = table[pos / page_size];
    if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) page = 0;
    for (int e = threadIdx.x; e < nkv * row; e += blockDim.x) {
      const int g = e / row, c = e - g * row;
      if (c < d)
        pages[at.key(page, g, pos % page_size, page_size) + c] = mine[k_offset + g * d + c];
      else
        pages[at.value(page, g, pos % page_size, page_size) + (c - d)] = mine[v_offset + g * dv + (c - d)];
    }
    return;
  }
  if ((pos + 1) % pool) return;
  const int slot = slots[req];
  if (!(TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0)) return;
  const int block = pos / pool;
  if (block >= max_blocks) return;
  const int g = blockIdx.y - 1;
  const int first = req_indptr[req];     // the request's first token of this step ...
  const int first_pos = positions[first];  // ... and its position: older rows are in the pages
  float* out = pooled + (((size_t)slot * max_blocks + block) * nkv + g) * row;
  const float inv = 1.f / (float)pool;
  const int begin = pos - pool + 1;
  const int old_end = first_pos < begin ? begin : (first_pos > pos + 1 ? pos + 1 : first_pos);  // [begin, old_end): in the pages
  for (int c = threadIdx.x; c < row; c += blockDim.x) {
    float sum = 0.f;  // ascending position, whatever the step's cut
    int p = begin;
    for (; p + 8 <= old_end; p += 8) {  // eight loads in flight
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int pg = 0;
        if (TL_DEBUG_OK((p + j) / page_size < table_width, TL_DEBUG_POSITION, p + j)) pg = table[(p + j) / page_size];
        if (!TL_DEBUG_OK(pg >= 0 && pg < num_pages, TL_DEBUG_PAGE, pg)) pg = 0;
        v[j] = to_float(c < d ? pages[at.key(pg, g, (p + j) % page_size, page_size) + c]
                              : pages[at.value(pg, g, (p + j) % page_size, page_size) + (c - d)]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[j];
    }
    for (; p < old_end; ++p) {
      int pg = 0;
      if (TL_DEBUG_OK(p / page_size < table_width, TL_DEBUG_POSITION, p)) pg = table[p / page_size];
      if (!TL_DEBUG_OK(pg >= 0 && pg < num_pages, TL_DEBUG_PAGE, pg)) pg = 0;
      sum += to_float(c < d ? pages[at.key(pg, g, p % page_size, page_size) + c]
                            : pages[at.value(pg, g, p % page_size, page_size) + (c - d)]);
    }
    const T* theirs = proj + (size_t)(first + (p - first_pos)) * proj_stride + (c < d ? k_offset + g * d + c : v_offset + g * dv + (c - d));
    for (; p + 8 <= pos + 1; p += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = to_float(theirs[(size_t)j * proj_stride]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[j];
      theirs += (size_t)8 * proj_stride;
    }
    for (; p <= pos; ++p) {
      sum += to_float(*theirs);
      theirs += proj_stride;
    }
    out[c] = sum * inv;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
pooled_attention_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
                        const int* __restrict__ positions, const int* __restrict__ slots,
                        const float* __restrict__ pooled, int max_blocks, int max_slots, T* __restrict__ out,
                        int out_stride, int tokens, int nh, int nkv, int d, int dv, int page_size, int size, int pool,
                        float scale, int num_pages, int split) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  const Layout at(split, nkv, d, dv, page_size);
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
      row_off = at.key(page, kvh, key % page_size, page_size);
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
      const T* vrow = pages + off + at.v_base;
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

// The softmax state of every (token, query head) over its pooled rows alone.  ml[item] = (max, sum) with the max in
// log2 units (score * scale * log2 e), acc[item][dv] = sum_b 2^(s_b - max) value_b; a row that sees no block: (-inf, 0).
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
pooled_prior_kernel(const T* __restrict__ q, int q_stride, const int* __restrict__ token_req,
                    const int* __restrict__ positions, const int* __restrict__ slots, const float* __restrict__ pooled,
                    int max_blocks, int max_slots, float* __restrict__ ml, float* __restrict__ acc_out, int tokens, int nh,
                    int nkv, int d, int dv, int size, int pool, float scale_log2) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  __shared__ __align__(16) float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int slot = slots[token_req[t]];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  int blocks = (live && pos - size + 1 > 0) ? (pos - size + 1) / pool : 0;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks == 0) {
    if (lane == 0) {
      ml[item * 2] = -INFINITY;
      ml[item * 2 + 1] = 0.f;
    }
    return;
  }
  const int row = d + dv;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = to_float(qrow[i]);
  __syncwarp();
  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) acc[c] = 0.f;
  const float* mine = pooled + ((size_t)slot * max_blocks * nkv + kvh) * row;
  if (blocks <= 64 && (d & 3) == 0 && (row & 3) == 0) {
    // Few rows (which path a row takes depends on its position alone): the WARP walks each row, a lane four entries
    // of it, eight rows' loads in flight, instead of every lane its own row from end to end.  The chain of
    // dependent trips to memory is a third as long, and a row is read in whole lines.
    const int quads = d >> 2;
    float4 q4[MAX_D / 128];
#pragma unroll
    for (int k = 0; k < MAX_D / 128; ++k)
      q4[k] = lane + 32 * k < quads ? *reinterpret_cast<const float4*>(&qs[warp][4 * (lane + 32 * k)]) : make_float4(0.f, 0.f, 0.f, 0.f);
    float s0 = -INFINITY, s1 = -INFINITY;  // lane b's scores of rows b and 32 + b
    for (int b0 = 0; b0 < blocks; b0 += 8) {
      float part[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        part[u] = 0.f;
        if (b0 + u < blocks) {
          const float4* krow = reinterpret_cast<const float4*>(mine + (size_t)(b0 + u) * nkv * row);
#pragma unroll
          for (int k = 0; k < MAX_D / 128; ++k) {
            if (lane + 32 * k < quads) {
              const float4 k4 = krow[lane + 32 * k];
              part[u] = fmaf(q4[k].x, k4.x, part[u]);
              part[u] = fmaf(q4[k].y, k4.y, part[u]);
              part[u] = fmaf(q4[k].z, k4.z, part[u]);
              part[u] = fmaf(q4[k].w, k4.w, part[u]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float total = warp_sum(part[u]);
        const int b = b0 + u;
        if (b < blocks && (b & 31) == lane) {
          if (b < 32) s0 = total * scale_log2;
          else s1 = total * scale_log2;
        }
      }
    }
    m = warp_max(fmaxf(s0, s1));
    const float p0 = s0 == -INFINITY ? 0.f : exp2f(s0 - m), p1 = s1 == -INFINITY ? 0.f : exp2f(s1 - m);
    l = warp_sum(p0 + p1);
#pragma unroll 8
    for (int b = 0; b < blocks; ++b) {
      const float pj = __shfl_sync(0xffffffffu, b < 32 ? p0 : p1, b & 31);
      const float* vrow = mine + (size_t)b * nkv * row + d;
#pragma unroll
      for (int c = 0; c < MAX_D / 32; ++c) {
        const int e = lane + 32 * c;
        if (e < dv) acc[c] = fmaf(pj, vrow[e], acc[c]);
      }
    }
    if (lane == 0) {
      ml[item * 2] = m;
      ml[item * 2 + 1] = l;
    }
    float* dst = acc_out + (size_t)item * dv;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) {
      const int e = lane + 32 * c;
      if (e < dv) dst[e] = acc[c];
    }
    return;
  }
  for (int start = 0; start < blocks; start += 32) {
    const int b = start + lane;
    const bool valid = b < blocks;
    float s = -INFINITY;
    if (valid) {
      const float4* krow = reinterpret_cast<const float4*>(mine + (size_t)b * nkv * row);
      float dot = 0.f;
      if ((row & 3) == 0 && (d & 3) == 0) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;  // four chains instead of one of d dependent steps
#pragma unroll 16
        for (int i = 0; i < d / 4; ++i) {  // sixteen loads of the lane's own row in flight
          const float4 k4 = krow[i];
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[warp][4 * i]);
          d0 = fmaf(q4.x, k4.x, d0);
          d1 = fmaf(q4.y, k4.y, d1);
          d2 = fmaf(q4.z, k4.z, d2);
          d3 = fmaf(q4.w, k4.w, d3);
        }
        dot = (d0 + d1) + (d2 + d3);
      } else {
        const float* k1 = mine + (size_t)b * nkv * row;
        for (int i = 0; i < d; ++i) dot = fmaf(qs[warp][i], k1[i], dot);
      }
      s = dot * scale_log2;
    }
    const float new_m = fmaxf(m, warp_max(s));
    const float corr = exp2f(m - new_m);
    const float p = valid ? exp2f(s - new_m) : 0.f;
    l = l * corr + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] *= corr;
    const int last = blocks - start < 32 ? blocks - start : 32;
#pragma unroll 8
    for (int j = 0; j < last; ++j) {  // eight rows' loads in flight
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vrow = mine + (size_t)(start + j) * nkv * row + d;
#pragma unroll
      for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] = fmaf(pj, vrow[i], acc[c]);
      }
    }
  }
  if (lane == 0) {
    ml[item * 2] = m;
    ml[item * 2 + 1] = l;
  }
  float* dst = acc_out + (size_t)item * dv;
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) dst[i] = acc[c];
  }
}

}  // namespace

TL_DEBUG_READER(tl_pooled_attention_debug_error)

extern "C" {

// proj rows hold the keys at k_offset (nkv x d) and the values at v_offset (nkv x dv).  split != 0: the pages are
// [num_pages, 2, nkv, page_size, d] (d = dv), else [num_pages, 1, nkv, page_size, d + dv].
int tl_pooled_store(const void* proj, int proj_stride, int k_offset, int v_offset, void* pages, int dtype,
                    const int* block_table, int table_width, const int* token_req, const int* positions,
                    const int* req_indptr, const int* slots, float* pooled, int max_blocks, int max_slots, int tokens,
                    int nkv, int d, int dv, int page_size, int pool, int num_pages, int split, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nkv <= 0 || nkv >= 65535 || d <= 0 || dv <= 0 || page_size <= 0 || pool <= 0 || (split && d != dv))
    return TL_ERR_UNSUPPORTED;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(pooled_store_kernel<float>, dim3((unsigned)tokens, 1 + nkv), 128, 0, stream, (const float*)proj, proj_stride,
                      k_offset, v_offset, (float*)pages, block_table, table_width, token_req, positions, req_indptr,
                      slots, pooled, max_blocks, max_slots, nkv, d, dv, page_size, pool, num_pages, split);
  else
    tl::launch_kernel(pooled_store_kernel<__nv_bfloat16>, dim3((unsigned)tokens, 1 + nkv), 128, 0, stream,
                      (const __nv_bfloat16*)proj, proj_stride, k_offset, v_offset, (__nv_bfloat16*)pages, block_table,
                      table_width, token_req, positions, req_indptr, slots, pooled, max_blocks, max_slots, nkv, d, dv,
                      page_size, pool, num_pages, split);
  return TL_LAUNCH_CHECK();
}

int tl_pooled_attention(const void* q, int q_stride, const void* pages, int dtype, const int* block_table,
                        int table_width, const int* token_req, const int* positions, const int* slots,
                        const float* pooled, int max_blocks, int max_slots, void* out, int out_stride, int tokens, int nh,
                        int nkv, int d, int dv, int page_size, int size, int pool, float scale, int num_pages, int split,
                        cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || nkv <= 0 || nh % nkv || page_size <= 0 || size <= 0 || pool < 0 ||
      (split && d != dv))
    return TL_ERR_UNSUPPORTED;
  const long long items = (long long)tokens * nh;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(pooled_attention_kernel<float>, blocks, WARPS * 32, 0, stream, (const float*)q, q_stride,
                      (const float*)pages, block_table, table_width, token_req, positions, slots, pooled, max_blocks,
                      max_slots, (float*)out, out_stride, tokens, nh, nkv, d, dv, page_size, size, pool, scale,
                      num_pages, split);
  else
    tl::launch_kernel(pooled_attention_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, (const __nv_bfloat16*)q,
                      q_stride, (const __nv_bfloat16*)pages, block_table, table_width, token_req, positions, slots,
                      pooled, max_blocks, max_slots, (__nv_bfloat16*)out, out_stride, tokens, nh, nkv, d, dv, page_size,
                      size, pool, scale, num_pages, split);
  return TL_LAUNCH_CHECK();
}

// The softmax state over the pooled rows alone, for the kernels that walk the window's tokens: ml [tokens][nh][2],
// acc [tokens][nh][dv], float32.
int tl_pooled_prior(const void* q, int q_stride, int dtype, const int* token_req, const int* positions, const int* slots,
                    const float* pooled, int max_blocks, int max_slots, float* ml, float* acc, int tokens, int nh, int nkv,
                    int d, int dv, int size, int pool, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || nkv <= 0 || nh % nkv || size <= 0 || pool <= 0)
    return TL_ERR_UNSUPPORTED;
  const long long items = (long long)tokens * nh;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(pooled_prior_kernel<float>, blocks, WARPS * 32, 0, stream, (const float*)q, q_stride, token_req,
                      positions, slots, pooled, max_blocks, max_slots, ml, acc, tokens, nh, nkv, d, dv, size, pool,
                      scale_log2);
  else
    tl::launch_kernel(pooled_prior_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_stride,
                      token_req, positions, slots, pooled, max_blocks, max_slots, ml, acc, tokens, nh, nkv, d, dv, size,
                      pool, scale_log2);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
