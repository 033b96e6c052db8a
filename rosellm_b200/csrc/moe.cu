// Mixture of experts: routing, and the experts' gated feed-forward as grouped products.
//
// Routing (`moe_select_kernel`, one warp per token, float32): scores s = softmax(z) over all
// experts, or (score_kind 1) s = sigmoid(z) of each expert by itself; the choice is made on s + correction,
// the weights are the chosen experts' s.  With
// groups, the experts form `group_count` equal groups of neighbours, a group's score is the
// largest choice score in it, and only experts of the best `group_keep` groups can be chosen
// (the others count as minus infinity).  Ties go to the lower index.
//
// The chosen (token, expert) pairs are then laid out expert by expert (`moe_plan_kernel`:
// offsets and a list of row tiles from the per-expert counts; `moe_scatter_kernel`: a place for
// every pair), all on the device: the host never learns the counts, so a step's launches depend
// on its token count alone.  `moe_ffn1_kernel` computes a tile of f(h W_gate^T, h W_up^T) with
// the rows of h gathered by token, `moe_ffn2_kernel` the tile's product with W_down, and
// `moe_combine_kernel` sums a token's expert outputs in the order of its choices, times their
// weights (a fixed order: the result does not depend on where the pairs were placed).  Where the
// weight belongs on the expert's INPUT instead (expert(w * h)), `moe_scatter_kernel` leaves each
// place's weight in `place_weight`, the first product scales its two results by it before the
// gate function (W (w h) = w (W h)), and the sum at the end takes no weights.
// Products: float32 as IEEE multiply-adds on 64 x 64 tiles (tile_gemm.cuh); bfloat16 on the tensor
// cores (mma_tile.cuh) with float32 accumulation, or, where an expert has a few rows only (decode
// steps), by `moe_rows_kernel`, which streams the weights once with a warp an output column.
#include <math_constants.h>

#include "gated_act.cuh"
#include "gemm_vec.cuh"
#include "mma_tile.cuh"
#include "tile_gemm.cuh"

namespace rl {

constexpr int MOE_TILE_ROWS = TG_M;
constexpr float MOE_TAKEN = 1e38f;  // marks a group that has been picked

// The lane's candidate (value, index) merged over the warp: the largest value, among equals the
// lowest index.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

__global__ __launch_bounds__(128) void moe_select_kernel(const float* __restrict__ z, long ldz,
                                                         const float* __restrict__ correction, int n_tokens,
                                                         int n_experts, int top, int group_count, int group_keep,
                                                         int score_kind, int* __restrict__ ids, float* __restrict__ weights,
                                                         int* __restrict__ counts) {
  extern __shared__ float smem[];
  pdl_begin();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  const int E = n_experts;
  float* s_w = smem + (size_t)warp * 3 * E;  // scores
  float* c_w = s_w + E;                      // choice scores
  float* g_w = c_w + E;                      // group scores
  const float* zr = z + (size_t)t * ldz;
  float sum = 1.f;
  if (score_kind == 1) {
    for (int e = lane; e < E; e += 32) s_w[e] = 1.0f / (1.0f + expf(-zr[e]));
  } else {
    float mx = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    mx = warp_max(mx);
    sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float ex = expf(zr[e] - mx);
      s_w[e] = ex;
      sum += ex;
    }
    sum = warp_sum(sum);
  }
  for (int e = lane; e < E; e += 32) {
    const float s = score_kind == 1 ? s_w[e] : s_w[e] / sum;
    s_w[e] = s;
    c_w[e] = s + (correction != nullptr ? correction[e] : 0.f);
  }
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    const int per = E / group_count;
    for (int g = lane; g < group_count; g += 32) {
      float best = -CUDART_INF_F;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c_w[e]);
      g_w[g] = best;
    }
    __syncwarp();
    for (int pick = 0; pick < group_keep; ++pick) {
      float v = -CUDART_INF_F;
      int idx = 0x7fffffff;
      for (int g = lane; g < group_count; g += 32) {
        const float gv = g_w[g];
        if (gv < MOE_TAKEN && (gv > v || idx == 0x7fffffff)) {
          v = gv;
          idx = g;
        }
      }
      warp_argmax(v, idx);
      if (lane == 0 && idx != 0x7fffffff) g_w[idx] = MOE_TAKEN;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (g_w[e / per] < MOE_TAKEN) c_w[e] = -CUDART_INF_F;
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    float v = -CUDART_INF_F;
    int idx = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float cv = c_w[e];
      if (cv > v || (idx == 0x7fffffff && cv > -CUDART_INF_F)) {
        v = cv;
        idx = e;
      }
    }
    warp_argmax(v, idx);
    if (idx == 0x7fffffff) idx = 0;  // fewer allowed experts than `top`: refused by the host before
    if (lane == 0) {
      ids[(size_t)t * top + j] = idx;
      weights[(size_t)t * top + j] = s_w[idx];
      atomicAdd(&counts[idx], 1);
      c_w[idx] = -CUDART_INF_F;
    }
    __syncwarp();
  }
}

// Routing without a router: row `token id` of an integer table [vocab, top] names the token's experts (the entries
// of a row differ), each with the same weight.  A thread a (token, choice); ids, weights and counts as
// `moe_select_kernel` leaves them.  An id below zero is row -id - 1 of the engine's token feedback.
__global__ __launch_bounds__(256) void moe_table_select_kernel(const int* __restrict__ token_ids,
                                                               const int* __restrict__ table, int vocab, int n_tokens,
                                                               int n_experts, int top, float weight, int* __restrict__ ids,
                                                               float* __restrict__ weights, int* __restrict__ counts,
                                                               const int* __restrict__ feedback, int n_feedback,
                                                               int* __restrict__ status) {
  pdl_begin();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * top) return;
  const int t = i / top, j = i - t * top;
  int id = token_ids[t];
  if (id < 0 && feedback != nullptr && -id - 1 < n_feedback) id = feedback[-id - 1];
  int e = 0;
  if (id < 0 || id >= vocab) {
    atomicOr(status, RL_STATUS_BAD_TOKEN);
  } else {
    e = table[(size_t)id * top + j];
    if (e < 0 || e >= n_experts) {
      atomicOr(status, RL_STATUS_BAD_TOKEN);
      e = 0;
    }
  }
  ids[i] = e;
  weights[i] = weight;
  atomicAdd(&counts[e], 1);
}

// The same routing with its layout, in one block (fused: choice, counts, offsets, tile list and places, which a
// step of few tokens would otherwise spend three launches on): the counts live in shared memory, the global
// counters are not touched.  At most MOE_ROUTE_MAX_PAIRS pairs.
constexpr int MOE_ROUTE_MAX_PAIRS = 8192, MOE_ROUTE_MAX_EXPERTS = 2048;

__global__ __launch_bounds__(1024) void moe_table_route_kernel(const int* __restrict__ token_ids,
                                                               const int* __restrict__ table, int vocab, int n_tokens,
                                                               int n_experts, int top, float weight, int* __restrict__ ids,
                                                               float* __restrict__ weights, int* __restrict__ offsets,
                                                               int* __restrict__ tiles, int* __restrict__ meta,
                                                               int* __restrict__ row_token, int* __restrict__ place_of,
                                                               const int* __restrict__ feedback, int n_feedback,
                                                               int* __restrict__ status) {
  __shared__ int count_s[MOE_ROUTE_MAX_EXPERTS], off_s[MOE_ROUTE_MAX_EXPERTS + 1], tile_s[MOE_ROUTE_MAX_EXPERTS + 1];
  pdl_begin();
  const int n_pairs = n_tokens * top;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count_s[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int t = i / top, j = i - t * top;
    int id = token_ids[t];
    if (id < 0 && feedback != nullptr && -id - 1 < n_feedback) id = feedback[-id - 1];
    int e = 0;
    if (id < 0 || id >= vocab) {
      atomicOr(status, RL_STATUS_BAD_TOKEN);
    } else {
      e = table[(size_t)id * top + j];
      if (e < 0 || e >= n_experts) {
        atomicOr(status, RL_STATUS_BAD_TOKEN);
        e = 0;
      }
    }
    ids[i] = e;
    weights[i] = weight;
    atomicAdd(&count_s[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tile = 0;
    for (int e = 0; e < n_experts; ++e) {
      off_s[e] = at;
      tile_s[e] = tile;
      at += count_s[e];
      tile += (count_s[e] + MOE_TILE_ROWS - 1) / MOE_TILE_ROWS;
    }
    off_s[n_experts] = at;
    tile_s[n_experts] = tile;
    meta[0] = tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int c = off_s[e + 1] - off_s[e];
    for (int k = 0; k * MOE_TILE_ROWS < c; ++k) {
      int* tl = tiles + 3 * (size_t)(tile_s[e] + k);
      tl[0] = e;
      tl[1] = off_s[e] + k * MOE_TILE_ROWS;
      tl[2] = min(MOE_TILE_ROWS, c - k * MOE_TILE_ROWS);
    }
    offsets[e] = off_s[e];
    count_s[e] = 0;  // from here on: the places handed out
  }
  if (threadIdx.x == 0) offsets[n_experts] = off_s[n_experts];
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];  // this thread's own write
    const int place = off_s[e] + atomicAdd(&count_s[e], 1);
    row_token[place] = i / top;
    place_of[i] = place;
  }
}

// One block.  offsets[e]: first place of expert e; tiles[k] = (expert, first place, rows);
// meta[0]: number of tiles.  Leaves counts and fill zero (the scatter that follows counts the
// places it hands out in fill).
__global__ __launch_bounds__(256) void moe_plan_kernel(int* __restrict__ counts, int* __restrict__ fill,
                                                       int* __restrict__ offsets, int* __restrict__ tiles,
                                                       int* __restrict__ meta, int n_experts) {
  extern __shared__ int plan_s[];  // [E+1] offsets, [E+1] first tile
  pdl_begin();
  int* off_s = plan_s;
  int* tile_s = plan_s + n_experts + 1;
  if (threadIdx.x == 0) {
    int at = 0, tile = 0;
    for (int e = 0; e < n_experts; ++e) {
      off_s[e] = at;
      tile_s[e] = tile;
      const int c = counts[e];
      at += c;
      tile += (c + MOE_TILE_ROWS - 1) / MOE_TILE_ROWS;
    }
    off_s[n_experts] = at;
    tile_s[n_experts] = tile;
    meta[0] = tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int c = off_s[e + 1] - off_s[e];
    for (int k = 0; k * MOE_TILE_ROWS < c; ++k) {
      int* tl = tiles + 3 * (size_t)(tile_s[e] + k);
      tl[0] = e;
      tl[1] = off_s[e] + k * MOE_TILE_ROWS;
      tl[2] = min(MOE_TILE_ROWS, c - k * MOE_TILE_ROWS);
    }
    offsets[e] = off_s[e];
    counts[e] = 0;
    fill[e] = 0;
  }
  if (threadIdx.x == 0) offsets[n_experts] = off_s[n_experts];
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ offsets,
                                   int* __restrict__ fill, int* __restrict__ row_token, int* __restrict__ place_of,
                                   const float* __restrict__ weights, float* __restrict__ place_weight, int n_pairs,
                                   int top) {
  pdl_begin();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = ids[i];
  const int place = offsets[e] + atomicAdd(&fill[e], 1);
  row_token[place] = i / top;
  place_of[i] = place;
  if (place_weight != nullptr) place_weight[place] = weights[i];
}

// act[place, f] = f(h[token] . W_gate[e, f], h[token] . W_up[e, f]).  w_gu: [experts][2][ff][hidden].
template <typename T>
__global__ __launch_bounds__(256) void moe_ffn1_kernel(const T* __restrict__ h, long ldh, const T* __restrict__ w_gu,
                                                       const int* __restrict__ tiles, const int* __restrict__ meta,
                                                       const int* __restrict__ row_token,
                                                       const float* __restrict__ row_scale, T* __restrict__ act,
                                                       long lda, int hidden, int ff, int kind, float alpha,
                                                       float limit) {
  __shared__ TileGemmSmem s;
  __shared__ float up_s[TG_K][TG_N + 1];
  __shared__ int tok[TG_M];
  pdl_begin();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * TG_N;
  if (threadIdx.x < TG_M) tok[threadIdx.x] = threadIdx.x < rows ? row_token[row0 + threadIdx.x] : 0;
  __syncthreads();
  const T* wg = w_gu + (size_t)e * 2 * ff * hidden;
  const T* wu = wg + (size_t)ff * hidden;
  float acc_g[4][4] = {}, acc_u[4][4] = {};
  tile_gemm_pair(
      acc_g, acc_u, hidden,
      [&](int m, int k) { return (m < rows && k < hidden) ? to_f32(h[(size_t)tok[m] * ldh + k]) : 0.f; },
      [&](int k, int n) { return (n0 + n < ff && k < hidden) ? to_f32(wg[(size_t)(n0 + n) * hidden + k]) : 0.f; },
      [&](int k, int n) { return (n0 + n < ff && k < hidden) ? to_f32(wu[(size_t)(n0 + n) * hidden + k]) : 0.f; },
      s, up_s);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
    const float sc = row_scale != nullptr ? row_scale[row0 + m] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < ff)
        act[(size_t)(row0 + m) * lda + n] = from_f32<T>(gated_value(sc * acc_g[i][j], sc * acc_u[i][j], kind, alpha, limit));
    }
  }
}

// eo[place, :] = act[place, :] W_down[e]^T.  w_down: [experts][hidden][ff]; eo float32.
template <typename T>
__global__ __launch_bounds__(256) void moe_ffn2_kernel(const T* __restrict__ act, long lda,
                                                       const T* __restrict__ w_down, const int* __restrict__ tiles,
                                                       const int* __restrict__ meta, float* __restrict__ eo,
                                                       int hidden, int ff) {
  __shared__ TileGemmSmem s;
  pdl_begin();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * TG_N;
  const T* wd = w_down + (size_t)e * hidden * ff;
  float acc[4][4] = {};
  tile_gemm(
      acc, ff, [&](int m, int k) { return (m < rows && k < ff) ? to_f32(act[(size_t)(row0 + m) * lda + k]) : 0.f; },
      [&](int k, int n) { return (n0 + n < hidden && k < ff) ? to_f32(wd[(size_t)(n0 + n) * ff + k]) : 0.f; }, s);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < hidden) eo[(size_t)(row0 + m) * hidden + n] = acc[i][j];
    }
  }
}

// The same two products in bfloat16 on the tensor cores (mma_tile.cuh), float32 accumulation.
template <bool VEC>
__global__ __launch_bounds__(128) void moe_ffn1_mma_kernel(const __nv_bfloat16* __restrict__ h, long ldh,
                                                           const __nv_bfloat16* __restrict__ w_gu,
                                                           const int* __restrict__ tiles, const int* __restrict__ meta,
                                                           const int* __restrict__ row_token,
                                                           const float* __restrict__ row_scale,
                                                           __nv_bfloat16* __restrict__ act, long lda, int hidden, int ff,
                                                           int kind, float alpha, float limit) {
  __shared__ __align__(16) MmaTileSmem s;
  __shared__ __align__(16) __nv_bfloat16 up_s[MT_STAGES][MT_N][MT_LD];
  __shared__ int tok[MT_M];
  pdl_begin();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * MT_N;
  if (threadIdx.x < MT_M) tok[threadIdx.x] = threadIdx.x < rows ? row_token[row0 + threadIdx.x] : 0;
  __syncthreads();
  const __nv_bfloat16* wg = w_gu + (size_t)e * 2 * ff * hidden;
  const __nv_bfloat16* wu = wg + (size_t)ff * hidden;
  float acc_g[2][4][4] = {}, acc_u[2][4][4] = {};
  mma_tile_pair<VEC>(
      acc_g, acc_u, hidden, [&](int m) { return m < rows ? h + (size_t)tok[m] * ldh : nullptr; },
      [&](int n) { return n0 + n < ff ? wg + (size_t)(n0 + n) * hidden : nullptr; },
      [&](int n) { return n0 + n < ff ? wu + (size_t)(n0 + n) * hidden : nullptr; }, s, up_s);
  mma_for_each(acc_g, [&](int m, int n, int mi, int ni, int c) {
    if (m < rows && n0 + n < ff) {
      const float sc = row_scale != nullptr ? row_scale[row0 + m] : 1.f;
      act[(size_t)(row0 + m) * lda + n0 + n] =
          __float2bfloat16_rn(gated_value(sc * acc_g[mi][ni][c], sc * acc_u[mi][ni][c], kind, alpha, limit));
    }
  });
}

template <bool VEC>
__global__ __launch_bounds__(128) void moe_ffn2_mma_kernel(const __nv_bfloat16* __restrict__ act, long lda,
                                                           const __nv_bfloat16* __restrict__ w_down,
                                                           const int* __restrict__ tiles, const int* __restrict__ meta,
                                                           float* __restrict__ eo, int hidden, int ff) {
  __shared__ __align__(16) MmaTileSmem s;
  pdl_begin();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * MT_N;
  const __nv_bfloat16* wd = w_down + (size_t)e * hidden * ff;
  float acc[2][4][4] = {};
  mma_tile<VEC>(
      acc, ff, [&](int m) { return m < rows ? act + (size_t)(row0 + m) * lda : nullptr; },
      [&](int n) { return n0 + n < hidden ? wd + (size_t)(n0 + n) * ff : nullptr; }, s);
  mma_for_each(acc, [&](int m, int n, int mi, int ni, int c) {
    if (m < rows && n0 + n < hidden) eo[(size_t)(row0 + m) * hidden + n0 + n] = acc[mi][ni][c];
  });
}

// Few rows an expert (a decode step): nothing is left of a 64-row tile but its weights, so the
// weights are streamed instead.  A warp owns one output column of its tile's expert: it reads the
// column's weight row (gate and up rows with PAIR) once, 16 bytes a lane a step, against up to
// MOE_ROWS_PASS input rows held in shared memory, and reduces over the lanes; tiles with more
// rows take further passes (their weights then come from L2).  float32 accumulation.
constexpr int MOE_ROWS_PASS = 4;

template <bool PAIR>
__global__ __launch_bounds__(256) void moe_rows_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       const int* __restrict__ tiles, const int* __restrict__ meta,
                                                       const int* __restrict__ row_token,
                                                       const float* __restrict__ row_scale,
                                                       __nv_bfloat16* __restrict__ act, long lda,
                                                       float* __restrict__ eo, int k_total, int n_total, int kind,
                                                       float alpha, float limit) {
  extern __shared__ __align__(16) __nv_bfloat16 rows_s[];  // [MOE_ROWS_PASS][k_total]
  pdl_begin();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.y * 8 + warp;
  // PAIR: w is [experts][2][n_total][k_total] (gate rows, then up rows); else [experts][n_total][k_total]
  const __nv_bfloat16* w0 = w + ((size_t)e * (PAIR ? 2 : 1) * n_total + min(n, n_total - 1)) * k_total;
  const __nv_bfloat16* w1 = w0 + (size_t)n_total * k_total;
  const int k8 = k_total >> 3;
  for (int r0 = 0; r0 < rows; r0 += MOE_ROWS_PASS) {
    const int nr = min(MOE_ROWS_PASS, rows - r0);
    __syncthreads();  // the rows of the pass before have been used
    for (int i = threadIdx.x; i < nr * k8; i += blockDim.x) {
      const int r = i / k8, c = (i - r * k8) * 8;
      const int src = PAIR ? row_token[row0 + r0 + r] : row0 + r0 + r;
      *reinterpret_cast<uint4*>(rows_s + (size_t)r * k_total + c) = *reinterpret_cast<const uint4*>(x + (size_t)src * ldx + c);
    }
    __syncthreads();
    float a0[MOE_ROWS_PASS], a1[MOE_ROWS_PASS];
#pragma unroll
    for (int r = 0; r < MOE_ROWS_PASS; ++r) a0[r] = a1[r] = 0.f;
#pragma unroll 2
    for (int c = lane * 8; c < k_total; c += 256) {
      float wv0[8], wv1[8];
      Vec16<__nv_bfloat16>::load(w0 + c, wv0);
      if (PAIR) Vec16<__nv_bfloat16>::load(w1 + c, wv1);
#pragma unroll
      for (int r = 0; r < MOE_ROWS_PASS; ++r) {
        if (r < nr) {
          float xv[8];
          Vec16<__nv_bfloat16>::load(rows_s + (size_t)r * k_total + c, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            a0[r] = fmaf(wv0[j], xv[j], a0[r]);
            if (PAIR) a1[r] = fmaf(wv1[j], xv[j], a1[r]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < MOE_ROWS_PASS; ++r) {
      if (r >= nr) continue;
      const float s0 = warp_sum(a0[r]);
      const float s1 = PAIR ? warp_sum(a1[r]) : 0.f;
      if (lane == 0 && n < n_total) {
        if (PAIR) {
          const float sc = row_scale != nullptr ? row_scale[row0 + r0 + r] : 1.f;
          act[(size_t)(row0 + r0 + r) * lda + n] = __float2bfloat16_rn(gated_value(sc * s0, sc * s1, kind, alpha, limit));
        } else
          eo[(size_t)(row0 + r0 + r) * n_total + n] = s0;
      }
    }
  }
}

// y[t] (+)= sum_j weights[t, j] * eo[place_of[t, j]], j in order (weights null: plain sum).
__global__ __launch_bounds__(256) void moe_combine_kernel(const float* __restrict__ eo,
                                                          const float* __restrict__ weights,
                                                          const int* __restrict__ place_of, float* __restrict__ y,
                                                          long ldy, int n_tokens, int hidden, int top, int add) {
  pdl_begin();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc = fmaf(weights != nullptr ? weights[(size_t)t * top + j] : 1.f,
                 eo[(size_t)place_of[(size_t)t * top + j] * hidden + d], acc);
    float* o = y + (size_t)t * ldy + d;
    *o = add ? *o + acc : acc;
  }
}

}  // namespace rl

// z: float32 router logits [tokens, experts] (row stride ldz).  ids, weights: [tokens * top].
// counts: [experts], zero on entry; holds the experts' pair counts afterwards.
RL_EXPORT int rl_moe_select(const float* z, long ldz, const float* correction, int n_tokens, int n_experts, int top,
                            int group_count, int group_keep, int score_kind, int* ids, float* weights, int* counts,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_experts <= 0 || n_experts > 2048 || top <= 0 || top > n_experts || score_kind < 0 || score_kind > 1) return -2;
  if (group_count < 1 || n_experts % group_count != 0 || group_keep < 1 || group_keep > group_count ||
      top > group_keep * (n_experts / group_count))
    return -3;
  const size_t smem = (size_t)4 * 3 * n_experts * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(rl::moe_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  rl::launch_pdl(rl::moe_select_kernel, (n_tokens + 3) / 4, 128, smem, stream, z, ldz, correction, n_tokens, n_experts,
                 top, group_count, group_keep, score_kind, ids, weights, counts);
  RL_CHECK_LAUNCH();
  return 0;
}

// table: int32 [vocab, top]; every chosen expert gets `weight`.  ids, weights, counts as rl_moe_select leaves them.
RL_EXPORT int rl_moe_table_select(const int* token_ids, const int* table, int vocab, int n_tokens, int n_experts, int top,
                                  float weight, int* ids, float* weights, int* counts, const int* feedback, int n_feedback,
                                  int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_experts <= 0 || n_experts > 2048 || top <= 0 || top > n_experts || vocab <= 0 || status == nullptr) return -2;
  rl::launch_pdl(rl::moe_table_select_kernel, (n_tokens * top + 255) / 256, 256, 0, stream, token_ids, table, vocab,
                 n_tokens, n_experts, top, weight, ids, weights, counts, feedback, n_feedback, status);
  RL_CHECK_LAUNCH();
  return 0;
}

// Routing by a table and the layout in one launch: what rl_moe_table_select and rl_moe_plan leave, for at most
// 8192 pairs (-3 beyond).  No counters in global memory are used.
RL_EXPORT int rl_moe_table_route(const int* token_ids, const int* table, int vocab, int n_tokens, int n_experts, int top,
                                 float weight, int* ids, float* weights, int* offsets, int* tiles, int* meta,
                                 int* row_token, int* place_of, const int* feedback, int n_feedback, int* status,
                                 cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_experts <= 0 || n_experts > rl::MOE_ROUTE_MAX_EXPERTS || top <= 0 || top > n_experts || vocab <= 0 ||
      status == nullptr)
    return -2;
  if ((long)n_tokens * top > rl::MOE_ROUTE_MAX_PAIRS) return -3;
  const int pairs = n_tokens * top;
  const int threads = pairs >= 1024 ? 1024 : ((pairs + 31) / 32) * 32;
  rl::launch_pdl(rl::moe_table_route_kernel, 1, threads, 0, stream, token_ids, table, vocab, n_tokens, n_experts, top,
                 weight, ids, weights, offsets, tiles, meta, row_token, place_of, feedback, n_feedback, status);
  RL_CHECK_LAUNCH();
  return 0;
}

// The pairs laid out expert by expert: offsets [experts + 1], tiles [max_tiles][3], meta [1],
// row_token and place_of [tokens * top].  counts as rl_moe_select left it, zero afterwards;
// fill is scratch.  max_tiles >= rl_moe_max_tiles(pairs, experts).
// weights, place_weight: both null, or the pairs' weights and a float32 [tokens * top] that receives them by place.
RL_EXPORT int rl_moe_plan(const int* ids, int* counts, int* fill, int* offsets, int* tiles, int* meta, int* row_token,
                          int* place_of, const float* weights, float* place_weight, int n_tokens, int n_experts, int top,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_experts <= 0 || n_experts > 2048) return -2;
  rl::launch_pdl(rl::moe_plan_kernel, 1, 256, (size_t)2 * (n_experts + 1) * sizeof(int), stream, counts, fill, offsets,
                 tiles, meta, n_experts);
  const int pairs = n_tokens * top;
  rl::launch_pdl(rl::moe_scatter_kernel, (pairs + 255) / 256, 256, 0, stream, ids, (const int*)offsets, fill, row_token,
                 place_of, weights, place_weight, pairs, top);
  RL_CHECK_LAUNCH();
  return 0;
}

RL_EXPORT int rl_moe_max_tiles(int n_pairs, int n_experts) {
  return (n_pairs + rl::MOE_TILE_ROWS - 1) / rl::MOE_TILE_ROWS + n_experts;
}

// The experts' feed-forward on the laid-out pairs, and the weighted sum per token.
// h: [tokens, hidden] (row stride ldh); w_gu: [experts][2][ff][hidden]; w_down:
// [experts][hidden][ff]; act: scratch [pairs, ff] (row stride lda); eo: float32 scratch
// [pairs, hidden]; y: float32 [tokens, hidden] (row stride ldy), overwritten or (add) added to.
// place_weight (by place) scales the experts' inputs, weights (by pair) their outputs; either may be null.
RL_EXPORT int rl_moe_experts(int dtype, const void* h, long ldh, const void* w_gu, const void* w_down, const int* tiles,
                             const int* meta, const int* row_token, const int* place_of, const float* weights,
                             const float* place_weight, void* act, long lda, float* eo, float* y, long ldy, int n_tokens, int hidden, int ff,
                             int n_experts, int top, int kind, float alpha, float limit, int add,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hidden <= 0 || ff <= 0 || kind < 0 || kind > 3) return -2;
  const int max_tiles = rl_moe_max_tiles(n_tokens * top, n_experts);
  const dim3 g1(max_tiles, (ff + rl::TG_N - 1) / rl::TG_N), g2(max_tiles, (hidden + rl::TG_N - 1) / rl::TG_N);
  if (g1.y > 65535 || g2.y > 65535) return -2;
  if (dtype == RL_F32) {
    rl::launch_pdl(rl::moe_ffn1_kernel<float>, g1, 256, 0, stream, (const float*)h, ldh, (const float*)w_gu, tiles,
                   meta, row_token, place_weight, (float*)act, lda, hidden, ff, kind, alpha, limit);
    rl::launch_pdl(rl::moe_ffn2_kernel<float>, g2, 256, 0, stream, (const float*)act, lda, (const float*)w_down, tiles,
                   meta, eo, hidden, ff);
  } else {
    const bool vec1 = hidden % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)h % 16) == 0 && ((uintptr_t)w_gu % 16) == 0;
    const bool vec2 = ff % 8 == 0 && lda % 8 == 0 && ((uintptr_t)act % 16) == 0 && ((uintptr_t)w_down % 16) == 0;
    // few pairs an expert (decode steps; on average one pass of rows each): stream the weights, a warp an
    // output column.  Measured at 32 experts, top 4: 8 requests 0.997 -> 0.843 ms a step, but 64 requests (8
    // rows an expert, two passes and more) 1.57 -> 2.16 ms, hence the bound
    const bool few = (long)n_tokens * top <= (long)rl::MOE_ROWS_PASS * n_experts && vec1 && vec2 && (size_t)hidden * 8 <= 48 * 1024 &&
                     (size_t)ff * 8 <= 48 * 1024;
    if (few) {
      rl::launch_pdl(rl::moe_rows_kernel<true>, dim3(max_tiles, (ff + 7) / 8), 256,
                     (size_t)rl::MOE_ROWS_PASS * hidden * 2, stream, (const __nv_bfloat16*)h, ldh,
                     (const __nv_bfloat16*)w_gu, tiles, meta, row_token, place_weight, (__nv_bfloat16*)act, lda, (float*)nullptr,
                     hidden, ff, kind, alpha, limit);
      rl::launch_pdl(rl::moe_rows_kernel<false>, dim3(max_tiles, (hidden + 7) / 8), 256,
                     (size_t)rl::MOE_ROWS_PASS * ff * 2, stream, (const __nv_bfloat16*)act, lda,
                     (const __nv_bfloat16*)w_down, tiles, meta, row_token, (const float*)nullptr, (__nv_bfloat16*)nullptr, 0L, eo, ff, hidden,
                     kind, alpha, limit);
    } else {
    auto k1 = vec1 ? rl::moe_ffn1_mma_kernel<true> : rl::moe_ffn1_mma_kernel<false>;
    auto k2 = vec2 ? rl::moe_ffn2_mma_kernel<true> : rl::moe_ffn2_mma_kernel<false>;
    // three stages of three operands are 46 KB a block: with the common half-and-half split of an
    // SM's memory two blocks fit, with all of it as shared memory four (the registers' limit)
    static bool carved[4] = {false, false, false, false};
    if (!carved[vec1]) {
      cudaFuncSetAttribute(k1, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
      carved[vec1] = true;
    }
    if (!carved[2 + vec2]) {
      cudaFuncSetAttribute(k2, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
      carved[2 + vec2] = true;
    }
    rl::launch_pdl_split(false, k1, g1, 128, 0, stream, (const __nv_bfloat16*)h, ldh, (const __nv_bfloat16*)w_gu, tiles,
                         meta, row_token, place_weight, (__nv_bfloat16*)act, lda, hidden, ff, kind, alpha, limit);
    rl::launch_pdl_split(false, k2, g2, 128, 0, stream, (const __nv_bfloat16*)act, lda, (const __nv_bfloat16*)w_down,
                         tiles, meta, eo, hidden, ff);
    }
  }
  rl::launch_pdl(rl::moe_combine_kernel, n_tokens, 256, 0, stream, (const float*)eo, weights, place_of, y, ldy,
                 n_tokens, hidden, top, add);
  RL_CHECK_LAUNCH();
  return 0;
}
