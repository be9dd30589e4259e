// A routed feed-forward (mixture of experts): every token goes through ``top`` of ``experts`` small
// gated feed-forwards.  Everything is planned on the device, so a step needs no answer from the GPU
// and a step of single tokens can be captured in a CUDA graph.
//
//   route     one warp per token: router logits z = W_r x in float32 (ascending k), scores
//             sigmoid(z) or softmax(z), the ``top`` largest (the lower index wins a tie), optionally
//             renormalized to sum 1;
//   plan      one block: rows per expert, each expert's rows rounded up to whole row tiles of
//             ``tile`` rows so that a tile of the grouped products belongs to ONE expert; the
//             position of every (token, choice) in that expert-sorted order; the expert of every tile;
//   scatter   the expert-sorted input rows: x[token] (times the choice's weight where the weight
//             multiplies the expert's INPUT);
//   products  out[row] = W_e(row) . in[row] over the sorted rows, CUDA cores, ascending k: with the
//             gated activation g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, +-limit),
//             over [gate; up] stacked weights, or plain (the down projection, float32 output);
//   combine   side[token] += sum over the token's choices, in the order of the choices, of the down
//             rows (times the weight where it multiplies the OUTPUT).
//
// A row's result depends on the row alone (its expert, its input), never on where it stands in the
// sorted order or on which other tokens are in the step.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int ROUTE_WARPS = 16;  // router rows taken side by side (8: ten rows and a gate's row took two rounds of loads)
constexpr int MAX_EXPERTS = 256;

// One router logit by one warp: each lane sums its 32nd of the row in eight independent chains (k = lane,
// lane + 32, ... in turn; eight loads in flight), so a logit's order of additions depends on the width alone.
template <typename Row>
__device__ __forceinline__ float router_logit(const Row* __restrict__ row, const float* __restrict__ w, int hidden, int lane) {
  float p[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = 0.f;
  int k = lane;
  for (; k + 224 < hidden; k += 256) {
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = fmaf(to_float(row[k + 32 * i]), w[k + 32 * i], p[i]);
  }
  for (; k < hidden; k += 32) p[0] = fmaf(to_float(row[k]), w[k], p[0]);
  return warp_sum(((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7])));
}

// One warp: from a token's router logits (``score``, shared memory, overwritten) to its ``top`` experts and
// their weights.
// ``groups`` > 1 with ``keep`` < groups: the experts form ``groups`` equal groups of neighbours, a group is scored by
// its largest member, and only experts of the ``keep`` best groups (the lower index wins a tie) can be chosen.
// ``pick`` (shared memory, ``experts`` floats; may be ``score`` itself): the numbers the choice goes by.  With a
// ``correction`` (one number an expert) they are score + correction, while the weights stay the scores.  The weights
// are multiplied by ``scale`` at the end.
__device__ __forceinline__ void choose_experts(float* score, float* pick, const float* __restrict__ correction,
                                               int experts, int top, int softmax_scores, int renormalize,
                                               int lane, int* __restrict__ choice, float* __restrict__ weight,
                                               int groups, int keep, float renorm_eps, float scale) {
  if (softmax_scores) {
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, score[e]);
    m = warp_max(m);
    float l = 0.f;
    for (int e = lane; e < experts; e += 32) l += expf(score[e] - m);
    l = warp_sum(l);
    for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - m) / l;
  } else {
    for (int e = lane; e < experts; e += 32) score[e] = 1.f / (1.f + expf(-score[e]));
  }
  __syncwarp();
  if (pick != score)
    for (int e = lane; e < experts; e += 32) pick[e] = score[e] + correction[e];
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = experts / groups;
    // lane g (and g + 32, ...) holds group g's score; ``kept`` groups are marked by a bit per group and lane
    unsigned long long mine = 0ull;  // bit i: the group lane + 32 i is kept
    for (int round = 0; round < keep; ++round) {
      float best = -INFINITY;
      int at = groups;
      for (int g = lane, i = 0; g < groups; g += 32, ++i) {
        if (mine >> i & 1ull) continue;
        float top_of = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) top_of = fmaxf(top_of, pick[e]);
        if (top_of > best) { best = top_of; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, o);
        const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
        if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
      }
      if (at < groups && (at & 31) == lane) mine |= 1ull << (at >> 5);
    }
    for (int g = lane, i = 0; g < groups; g += 32, ++i)
      if (!(mine >> i & 1ull))
        for (int e = g * per; e < (g + 1) * per; ++e) pick[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = experts;
    for (int e = lane; e < experts; e += 32) {
      const float s = pick[e];
      if (s > best) { best = s; at = e; }  // ascending e: the lower index keeps a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_at = __shfl_xor_sync(0xffffffffu, at, o);
      if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
    }
    if (at >= experts) at = 0;  // every score was NaN: still a valid expert
    const float chosen = score[at];
    __syncwarp();  // every lane has read the score before it is struck out
    total += chosen;
    if (lane == 0) {
      choice[j] = at;
      weight[j] = chosen;
      pick[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize || scale != 1.f)
    for (int j = lane; j < top; j += 32) weight[j] = (renormalize ? weight[j] / (total + renorm_eps) : weight[j]) * scale;
}

// One block per token.  The token's row is staged in shared memory as floats; warp w takes the
// experts w, w + ROUTE_WARPS, ...; the first warp then chooses.
template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ router, int* __restrict__ choice,
                 float* __restrict__ weight, int tokens, int hidden, int experts, int top, int softmax_scores,
                 int renormalize, int groups, int keep, float renorm_eps, const float* __restrict__ correction,
                 float scale, const float* __restrict__ gate_w, float* __restrict__ gate_out) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float xrow[];  // hidden floats
  __shared__ float all_scores[MAX_EXPERTS];
  __shared__ float picks[MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* row = x + (size_t)t * ldx;
  for (int k = threadIdx.x; k < hidden; k += ROUTE_WARPS * 32) xrow[k] = to_float(row[k]);
  __syncthreads();
  for (int e = warp; e < experts; e += ROUTE_WARPS) {
    const float part = router_logit(xrow, router + (size_t)e * hidden, hidden, lane);
    if (lane == 0) all_scores[e] = part;
  }
  // a gate of one number a token beside the router (an always-on expert's): sigmoid(gate_w . x), by the last warp
  if (gate_w && warp == ROUTE_WARPS - 1) {
    const float z = router_logit(xrow, gate_w, hidden, lane);
    if (lane == 0) gate_out[t] = 1.f / (1.f + expf(-z));
  }
  __syncthreads();
  if (warp != 0) return;
  choose_experts(all_scores, correction ? picks : all_scores, correction, experts, top, softmax_scores, renormalize, lane,
                 choice + (size_t)t * top, weight + (size_t)t * top, groups, keep, renorm_eps, scale);
}

// plan[0] = tiles in use; plan[1 ..] = expert of every tile (-1: none).
constexpr int PLAN_NT = 1024;

__global__ void __launch_bounds__(PLAN_NT)
moe_plan_kernel(const int* __restrict__ choice, int* __restrict__ position, int* __restrict__ plan, int entries,
                int experts, int tile, int max_tiles) {
  // a choice >= experts names an identity expert (its output is its input): it has no row, position -1
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ int count[MAX_EXPERTS], start[MAX_EXPERTS], cursor[MAX_EXPERTS];
  for (int e = threadIdx.x; e < experts; e += PLAN_NT) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += PLAN_NT)
    if (choice[i] < experts) atomicAdd(&count[choice[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = tiles * tile;
      const int mine = (count[e] + tile - 1) / tile;
      for (int j = 0; j < mine && tiles + j < max_tiles; ++j) plan[1 + tiles + j] = e;
      tiles += mine;
    }
    plan[0] = tiles < max_tiles ? tiles : max_tiles;
    for (int j = tiles; j < max_tiles; ++j) plan[1 + j] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += PLAN_NT) {
    const int e = choice[i];
    position[i] = e < experts ? start[e] + atomicAdd(&cursor[e], 1) : -1;
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_scatter_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ position, const float* __restrict__ weight,
                   T* __restrict__ sorted, int hidden, int top, int weighted) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int entry = blockIdx.x;
  const int t = entry / top;
  const float w = weighted ? weight[entry] : 1.f;
  if (position[entry] < 0) return;  // an identity expert has no row
  const T* from = x + (size_t)t * ldx;
  T* to = sorted + (size_t)position[entry] * hidden;
  for (int k = threadIdx.x; k < hidden; k += 128) to[k] = weighted ? from_float<T>(w * to_float(from[k])) : from[k];
}

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// out[row, n] over the rows of tile blockIdx.y, whose expert the plan names.  GLU: w holds, per
// expert, [gate (N rows); up (N rows)] and out = act(gate . x, up . x); else out = w_e . x.
template <typename T, typename OutT, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, OutT* __restrict__ out,
                     const int* __restrict__ plan, int N, int K, float limit, float alpha) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  if ((int)blockIdx.y >= plan[0]) return;
  const int expert = plan[1 + blockIdx.y];
  if (expert < 0) return;
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  __shared__ float us[GLU ? BK : 1][BN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;
  const T* we = w + (size_t)expert * (GLU ? 2 : 1) * N * K;
  float acc[TM][TN], acc_up[GLU ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if constexpr (GLU) acc_up[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / BK, c = e % BK;
      const int k = k0 + c;
      float xv = 0.f, wv = 0.f, uv = 0.f;
      if (k < K) {
        xv = to_float(x[(size_t)(m0 + r) * K + k]);
        if (n0 + r < N) {
          wv = to_float(we[(size_t)(n0 + r) * K + k]);
          if (GLU) uv = to_float(we[(size_t)(N + n0 + r) * K + k]);
        }
      }
      xs[c][r] = xv;
      ws[c][r] = wv;
      if constexpr (GLU) us[c][r] = uv;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float xa[TM], wb[TN], ub[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) xa[i] = xs[c][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        wb[j] = ws[c][tx * TN + j];
        if constexpr (GLU) ub[j] = us[c][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
          if constexpr (GLU) acc_up[i][j] = fmaf(xa[i], ub[j], acc_up[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if constexpr (GLU) {
        if (limit > 0.f) {
          const float g = fminf(v, limit);
          const float u = fminf(fmaxf(acc_up[i][j], -limit), limit);
          v = g / (1.f + expf(-alpha * g)) * (u + 1.f);
        } else {  // no limit: silu(gate) * up
          v = v / (1.f + expf(-v)) * acc_up[i][j];
        }
      }
      out[(size_t)m * N + n] = from_float<OutT>(v);
    }
  }
}

// Four columns a thread (a block of 512 columns of one token): a thread's loads are the choices' positions and
// one 16-byte value each, so nothing waits in a chain, and a long step still moves whole sectors.  VEC: the width
// is a multiple of 4 (else one column a thread).
template <bool VEC>
__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ position, const float* __restrict__ weight,
                   float* __restrict__ side, int hidden, int top, int weighted, const float* __restrict__ x_f32,
                   const __nv_bfloat16* __restrict__ x_bf16, int ldx) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int t = blockIdx.x;
  constexpr int PER = VEC ? 4 : 1;
  const int c = (blockIdx.y * 128 + threadIdx.x) * PER;
  if (c >= hidden) return;
  float sum[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) sum[i] = 0.f;
  for (int j = 0; j < top; ++j) {  // in the order of the choices
    const int at = position[(size_t)t * top + j];
    const float w = weighted ? weight[(size_t)t * top + j] : 1.f;
    if (at < 0) {  // an identity expert: its output is the token's own input row (x_f32 or x_bf16)
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const size_t e = (size_t)t * ldx + c + i;
        const float v = x_bf16 ? to_float(x_bf16[e]) : x_f32[e];
        sum[i] = weighted ? fmaf(w, v, sum[i]) : sum[i] + v;
      }
      continue;
    }
    const float* row = y + (size_t)at * hidden + c;
    if constexpr (VEC) {
      const float4 v = *reinterpret_cast<const float4*>(row);
      sum[0] = weighted ? fmaf(w, v.x, sum[0]) : sum[0] + v.x;
      sum[1] = weighted ? fmaf(w, v.y, sum[1]) : sum[1] + v.y;
      sum[2] = weighted ? fmaf(w, v.z, sum[2]) : sum[2] + v.z;
      sum[3] = weighted ? fmaf(w, v.w, sum[3]) : sum[3] + v.w;
    } else {
      sum[0] = weighted ? fmaf(w, row[0], sum[0]) : sum[0] + row[0];
    }
  }
  float* out = side + (size_t)t * hidden + c;
  if constexpr (VEC) {
    float4 o = *reinterpret_cast<float4*>(out);
    o.x += sum[0]; o.y += sum[1]; o.z += sum[2]; o.w += sum[3];
    *reinterpret_cast<float4*>(out) = o;
  } else {
    out[0] += sum[0];
  }
}

}  // namespace

extern "C" {

int tl_moe_tile_rows() { return BM; }

// choice int32 [tokens, top], weight float32 [tokens, top]; router float32 [experts, hidden].
// correction (optional, float32 [experts]): added to the scores for the choice only.  scale: multiplies the weights.
// gate_w (optional, float32 [hidden]) with gate_out (float32 [tokens]): gate_out[t] = sigmoid(gate_w . x[t]).
int tl_moe_route(const void* x, int ldx, int dtype, const float* router, int* choice, float* weight, int tokens,
                 int hidden, int experts, int top, int softmax_scores, int renormalize, int groups, int keep,
                 float renorm_eps, const float* correction, float scale, const float* gate_w, float* gate_out,
                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (experts <= 0 || experts > MAX_EXPERTS || top <= 0 || top > experts) return TL_ERR_UNSUPPORTED;
  if (groups < 1 || keep < 1 || keep > groups || experts % groups || top > keep * (experts / groups) || groups > 2048)
    return TL_ERR_UNSUPPORTED;
  const unsigned blocks = tokens;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 48 * 1024) return TL_ERR_UNSUPPORTED;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(moe_route_kernel<float>, blocks, ROUTE_WARPS * 32, smem, stream, (const float*)x, ldx, router, choice,
                      weight, tokens, hidden, experts, top, softmax_scores, renormalize, groups, keep, renorm_eps, correction,
                      scale, gate_w, gate_out);
  else
    tl::launch_kernel(moe_route_kernel<__nv_bfloat16>, blocks, ROUTE_WARPS * 32, smem, stream, (const __nv_bfloat16*)x,
                      ldx, router, choice, weight, tokens, hidden, experts, top, softmax_scores, renormalize, groups, keep,
                      renorm_eps, correction, scale, gate_w, gate_out);
  return TL_LAUNCH_CHECK();
}

// position int32 [entries]; plan int32 [1 + max_tiles].
int tl_moe_plan(const int* choice, int* position, int* plan, int entries, int experts, int tile, int max_tiles,
                cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (experts <= 0 || experts > MAX_EXPERTS || tile <= 0) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(moe_plan_kernel, 1, PLAN_NT, 0, stream, choice, position, plan, entries, experts, tile, max_tiles);
  return TL_LAUNCH_CHECK();
}

int tl_moe_scatter(const void* x, int ldx, int dtype, const int* position, const float* weight, void* sorted,
                   int tokens, int hidden, int top, int weighted, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(moe_scatter_kernel<float>, (unsigned)(tokens * top), 128, 0, stream, (const float*)x, ldx, position,
                      weight, (float*)sorted, hidden, top, weighted);
  else
    tl::launch_kernel(moe_scatter_kernel<__nv_bfloat16>, (unsigned)(tokens * top), 128, 0, stream,
                      (const __nv_bfloat16*)x, ldx, position, weight, (__nv_bfloat16*)sorted, hidden, top, weighted);
  return TL_LAUNCH_CHECK();
}

// x [rows, K] sorted rows (rows = max_tiles * 64), w [experts, (2) N, K], out [rows, N].
int tl_moe_gemm_simt(const void* x, const void* w, int dtype, void* out, int out_dtype, const int* plan, int max_tiles,
                     int N, int K, int glu, float limit, float alpha, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || max_tiles > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid((N + BN - 1) / BN, max_tiles);
#define TL_MOE(T, OutT, GLU)                                                                                        \
  tl::launch_kernel(moe_gemm_simt_kernel<T, OutT, GLU>, grid, 256, 0, stream, (const T*)x, (const T*)w, (OutT*)out, \
                    plan, N, K, limit, alpha)
  if (dtype == TL_DTYPE_F32) {
    if (out_dtype != TL_DTYPE_F32) return TL_ERR_UNSUPPORTED;
    if (glu) TL_MOE(float, float, true); else TL_MOE(float, float, false);
  } else if (glu) {
    if (out_dtype != TL_DTYPE_BF16) return TL_ERR_UNSUPPORTED;
    TL_MOE(__nv_bfloat16, __nv_bfloat16, true);
  } else {
    if (out_dtype != TL_DTYPE_F32) return TL_ERR_UNSUPPORTED;
    TL_MOE(__nv_bfloat16, float, false);
  }
#undef TL_MOE
  return TL_LAUNCH_CHECK();
}

// x (optional; its rows in ``x_dtype``, row stride ldx): the tokens' input rows, which a choice without a row (position
// -1, an identity expert) adds instead of a product's row.
int tl_moe_combine(const float* y, const int* position, const float* weight, float* side, int tokens, int hidden,
                   int top, int weighted, const void* x, int ldx, int x_dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const float* x_f32 = x && x_dtype == TL_DTYPE_F32 ? (const float*)x : nullptr;
  const __nv_bfloat16* x_bf16 = x && x_dtype == TL_DTYPE_BF16 ? (const __nv_bfloat16*)x : nullptr;
  const bool vec = hidden % 4 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(side)) & 15) == 0;
  const int per_block = vec ? 512 : 128;
  const unsigned blocks_y = (unsigned)((hidden + per_block - 1) / per_block);
  if (blocks_y > 65535) return TL_ERR_UNSUPPORTED;
  if (vec)
    tl::launch_kernel(moe_combine_kernel<true>, dim3((unsigned)tokens, blocks_y), 128, 0, stream, y, position, weight, side,
                      hidden, top, weighted, x_f32, x_bf16, ldx);
  else
    tl::launch_kernel(moe_combine_kernel<false>, dim3((unsigned)tokens, blocks_y), 128, 0, stream, y, position, weight, side,
                      hidden, top, weighted, x_f32, x_bf16, ldx);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
