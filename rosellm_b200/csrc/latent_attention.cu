// Attention over a cache of latents: one row per token, shared by all heads, that serves as
// key and as value.
//
// A mixer of this kind projects a token to a short latent c (normalised) and a rotated key
// part k_r that all heads share, and caches only the row [c, k_r].  Per head the key would be
// [W_uk c, k_r] and the value W_uv c; because both are linear in c, the query takes W_uk over
// to its side (q_c = W_uk^T q_plain, computed by the per-head product in head_linear.cu) and
// the value's W_uv is applied after the weighted sum.  What is left is attention of H query
// rows [q_c, q_r] per token against the same cached rows, with the first `rank` entries of a
// row as its value:
//   s_j = scale * (q_c . c_j + q_r . k_r,j),  p = softmax over j <= position (with a sink),
//   o = sum_j p_j c_j.
// The sink is one more term exp(sink_h) in the denominator with no key and no value: the online
// softmax starts from m = sink_h, l = 1, o = 0 instead of m = -inf, l = 0.  Scores, softmax and
// sums are float32 in both precisions.
//
// Pool layout of one layer: [pages][page size][row width], row width = rank + rotated
// entries, filled with zeros up to a multiple of 8 elements (rows start on 16-byte boundaries).
//
// Kernels (the last three are the float32 path, and the bfloat16 path of sizes the tensor-core
// kernel `latent_attn_mma_kernel` does not take): `latent_kv_write_kernel` (RMS norm of c, rotation of k_r, write into the page);
// `latent_q_rope_kernel` (rotation of the queries' rotated part into the query rows);
// `latent_attn_tile_kernel` (16 queries of one request and head against tiles of 32 keys in
// shared memory: prompt portions, and decoded tokens in the 32-bit mode);
// `latent_attn_decode_kernel` (a decoded token: one block takes all heads of a request and a
// share of its keys, so that a cached row is read once for all heads) with
// `latent_attn_merge_kernel`.
#include <math_constants.h>

#include "common.cuh"
#include "gemm_vec.cuh"

namespace rl {

// (u, v) at angle a -> (u cos a - v sin a, v cos a + u sin a); element j of the pair (2i, 2i+1).
__device__ __forceinline__ float rotate_element(float u, float v, float angle, int odd) {
  float s, c;
  sincosf(angle, &s, &c);
  return odd ? fmaf(v, c, u * s) : fmaf(u, c, -(v * s));
}

template <typename T>
__global__ __launch_bounds__(128) void latent_kv_write_kernel(
    const float* __restrict__ dkv, long ld, const float* __restrict__ gamma, float eps,
    const float* __restrict__ inv_freq, int rot_dims, T* __restrict__ pool, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ positions, const int* __restrict__ req_of_token,
    const int* __restrict__ slots, int n_tokens, int rank, int rot_dim, int row_width, int page_size, int max_pos,
    float rot_mult, int* __restrict__ status) {
  __shared__ float scratch[33];
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  const int pos = positions[n];
  const int slot = slots[req_of_token[n]];
  if (slot < 0) return;  // padding of a fixed-size batch
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_POSITION);
    return;
  }
  const int page = block_table[(size_t)slot * bt_stride + pos / page_size];
  if (page < 0) {
    if (threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_PAGE);
    return;
  }
  const float* src = dkv + (size_t)n * ld;
  float s = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) s = fmaf(src[d], src[d], s);
  const float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)rank + eps);
  T* dst = pool + ((size_t)page * page_size + pos % page_size) * row_width;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_f32<T>(src[d] * r * gamma[d]);
  const float* kr = src + rank;
  for (int j = threadIdx.x; j < row_width - rank; j += blockDim.x) {
    float v = 0.f;
    if (j < rot_dims) {
      const int i = j >> 1;
      v = rotate_element(kr[2 * i], kr[2 * i + 1], (float)pos * inv_freq[i], j & 1) * rot_mult;
    } else if (j < rot_dim) {
      v = kr[j];
    }
    dst[rank + j] = from_f32<T>(v);
  }
}

// The rotated part of every head's query, turned by the token's position, into the query rows
// (entries [rank, row_width) of head h's row; beyond the rotated entries: zeros).
template <typename T>
__global__ __launch_bounds__(128) void latent_q_rope_kernel(
    const T* __restrict__ q, long q_stride, int head_in, int plain, T* __restrict__ rows, long rows_stride,
    int row_width, int rank, int rot_dim, int rot_dims, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, int n_tokens, int n_heads, float rot_mult) {
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  const float pos = (float)positions[n];
  const int tail = row_width - rank;
  for (int i = threadIdx.x; i < n_heads * tail; i += blockDim.x) {
    const int h = i / tail, j = i - h * tail;
    const T* qr = q + (size_t)n * q_stride + (size_t)h * head_in + plain;
    float v = 0.f;
    if (j < rot_dims) {
      const int pair = j >> 1;
      v = rotate_element(to_f32(qr[2 * pair]), to_f32(qr[2 * pair + 1]), pos * inv_freq[pair], j & 1) * rot_mult;
    } else if (j < rot_dim) {
      v = to_f32(qr[j]);
    }
    rows[(size_t)n * rows_stride + (size_t)h * row_width + rank + j] = from_f32<T>(v);
  }
}

struct LatentParams {
  const void* q;      // query row of token n, head h: q + n*q_stride + h*row_width
  long q_stride;      // in elements
  const void* pool;
  const int* block_table;
  int bt_stride;
  const int* q_start;  // [requests+1]
  const int* kv_len;   // [requests] rows the request has after this step's write
  const int* slots;    // [requests]
  void* out;           // out + n*out_stride + h*rank
  long out_stride;
  const float* sink;   // [heads], or null
  int n_heads, rank, row_width, page_size;
  float scale;
  int* status;
};

constexpr int LT_Q = 16;     // queries per block
constexpr int LT_KV = 32;    // keys per tile: one per lane
constexpr int LT_ROWS = 4;   // queries per warp

// Blocks [0, n_tiles): (request, first query) from `tiles`; blocks beyond: decoded requests.
template <typename T, int NCHUNK>
__global__ __launch_bounds__(128) void latent_attn_tile_kernel(LatentParams p, const int* __restrict__ tiles,
                                                               int n_tiles, const int* __restrict__ decode_reqs) {
  extern __shared__ __align__(16) float smem[];
  pdl_begin();
  const int W = p.row_width;
  float* q_s = smem;               // [LT_Q][W], scaled
  float* k_s = q_s + LT_Q * W;     // [LT_KV][W+1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int req, t0;
  if ((int)blockIdx.x < n_tiles) {
    req = tiles[2 * blockIdx.x];
    t0 = tiles[2 * blockIdx.x + 1];
  } else {
    req = decode_reqs[blockIdx.x - n_tiles];
    t0 = 0;
  }
  const int h = blockIdx.y;
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int rows = min(LT_Q, q_len - t0);
  T* out = (T*)p.out;
  const int slot = p.slots[req];
  if (slot < 0) {  // padding of a fixed-size batch: no cache behind it
    for (int i = tid; i < rows * p.rank; i += blockDim.x)
      out[(size_t)(qs + t0 + i / p.rank) * p.out_stride + (size_t)h * p.rank + i % p.rank] = from_f32<T>(0.f);
    return;
  }
  const int kv_len = p.kv_len[req];
  const int pos0 = kv_len - q_len;
  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  const T* q = (const T*)p.q;
  for (int i = tid; i < LT_Q * W; i += blockDim.x) {
    const int r = i / W, d = i - r * W;
    q_s[i] = r < rows ? to_f32(q[(size_t)(qs + t0 + r) * p.q_stride + (size_t)h * W + d]) * p.scale : 0.f;
  }
  const int first_pos = pos0 + t0;
  const int kv_hi = first_pos + rows;
  const float sink = p.sink != nullptr ? p.sink[h] : -CUDART_INF_F;
  float m[LT_ROWS], l[LT_ROWS], o[LT_ROWS][NCHUNK];
#pragma unroll
  for (int r = 0; r < LT_ROWS; ++r) {
    m[r] = sink;
    l[r] = p.sink != nullptr ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) o[r][c] = 0.f;
  }
  const int W4 = W >> 2;
  for (int kt = 0; kt < kv_hi; kt += LT_KV) {
    __syncthreads();
    for (int i = tid; i < LT_KV * W4; i += blockDim.x) {
      const int j = i / W4, d = (i - j * W4) * 4;
      const int key = kt + j;
      float kk[4] = {0.f, 0.f, 0.f, 0.f};
      if (key < kv_hi) {
        const int page = bt[key / p.page_size];
        if (page < 0)
          atomicOr(p.status, RL_STATUS_BAD_PAGE);
        else
          load4((const T*)p.pool + ((size_t)page * p.page_size + key % p.page_size) * W + d, kk);
      }
      float* kd = k_s + j * (W + 1) + d;
      kd[0] = kk[0]; kd[1] = kk[1]; kd[2] = kk[2]; kd[3] = kk[3];
    }
    __syncthreads();
    float s[LT_ROWS];
#pragma unroll
    for (int r = 0; r < LT_ROWS; ++r) s[r] = 0.f;
    const float* kr = k_s + lane * (W + 1);
    const float* qr = q_s + warp * LT_ROWS * W;
    for (int d = 0; d < W; ++d) {
      const float kd = kr[d];
#pragma unroll
      for (int r = 0; r < LT_ROWS; ++r) s[r] = fmaf(qr[r * W + d], kd, s[r]);
    }
    const int key = kt + lane;
    float pr[LT_ROWS];
#pragma unroll
    for (int r = 0; r < LT_ROWS; ++r) {
      const int row = warp * LT_ROWS + r;
      const bool valid = row < rows && key <= first_pos + row;
      const float sv = valid ? s[r] : -CUDART_INF_F;
      const float m_new = fmaxf(m[r], warp_max(sv));
      const float alpha = m_new == -CUDART_INF_F ? 1.f : expf(m[r] - m_new);
      pr[r] = valid ? expf(sv - m_new) : 0.f;
      l[r] = l[r] * alpha + warp_sum(pr[r]);
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) o[r][c] *= alpha;
      m[r] = m_new;
    }
    const int cnt = min(LT_KV, kv_hi - kt);
    for (int j = 0; j < cnt; ++j) {
      float pj[LT_ROWS];
#pragma unroll
      for (int r = 0; r < LT_ROWS; ++r) pj[r] = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int d = lane + 32 * c;
        const float vv = d < p.rank ? k_s[j * (W + 1) + d] : 0.f;
#pragma unroll
        for (int r = 0; r < LT_ROWS; ++r) o[r][c] = fmaf(pj[r], vv, o[r][c]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < LT_ROWS; ++r) {
    const int row = warp * LT_ROWS + r;
    if (row >= rows) continue;
    const float inv = 1.0f / l[r];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int d = lane + 32 * c;
      if (d < p.rank) out[(size_t)(qs + t0 + row) * p.out_stride + (size_t)h * p.rank + d] = from_f32<T>(o[r][c] * inv);
    }
  }
}

// A decoded token: block (request, split) takes the keys [beg, end) of the request for ALL
// heads.  A tile of LD_KV cached rows is staged in shared memory once; warp w then serves heads
// w, w + warps, ...: lane = key for the scores, lane = value entry for the weighted sum.
// The queries of all heads lie in shared memory (float32, scaled).  Partial results
// (m, l, o[rank]) per (request, head, split) are merged by latent_attn_merge_kernel; with one
// split the result goes straight to `out`.  The sink belongs to split 0.
constexpr int LD_KV = 32;
constexpr int LD_WARPS = 8;

template <typename T, int NCHUNK>
__global__ __launch_bounds__(32 * LD_WARPS) void latent_attn_decode_kernel(
    LatentParams p, const int* __restrict__ decode_reqs, int n_splits, float* __restrict__ part_o,
    float* __restrict__ part_ml) {
  extern __shared__ __align__(16) float smem[];
  pdl_begin();
  const int W = p.row_width, H = p.n_heads;
  float* k_s = smem;                      // [LD_KV][W+1]
  float* q_s = k_s + LD_KV * (W + 1);     // [H][W]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int req = decode_reqs[blockIdx.x], sp = blockIdx.y;
  const int n = p.q_start[req];
  const int slot = p.slots[req];
  T* out = (T*)p.out;
  if (slot < 0) {
    if (sp == 0)
      for (int i = tid; i < H * p.rank; i += blockDim.x) out[(size_t)n * p.out_stride + i] = from_f32<T>(0.f);
    return;
  }
  const int kv_len = p.kv_len[req];
  const int chunk = ((kv_len + n_splits - 1) / n_splits + LD_KV - 1) / LD_KV * LD_KV;
  const int beg = sp * chunk, end = min(kv_len, beg + chunk);
  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  const T* q = (const T*)p.q + (size_t)n * p.q_stride;
  for (int i = tid; i < H * W; i += blockDim.x) q_s[i] = to_f32(q[i]) * p.scale;
  const int W4 = W >> 2;
  // this warp's heads: at most HPW of them are kept in registers at once
  constexpr int HPW = 4;
  for (int base = 0; base < H; base += LD_WARPS * HPW) {  // the same count for every warp: barriers inside
    const int h0 = base + warp;
    float m[HPW], l[HPW], o[HPW][NCHUNK];
#pragma unroll
    for (int r = 0; r < HPW; ++r) {
      const int h = h0 + r * LD_WARPS;
      const bool sinked = p.sink != nullptr && sp == 0 && h < H;
      m[r] = sinked ? p.sink[h] : -CUDART_INF_F;
      l[r] = sinked ? 1.f : 0.f;
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) o[r][c] = 0.f;
    }
    for (int kt = beg; kt < end; kt += LD_KV) {
      __syncthreads();
      for (int i = tid; i < LD_KV * W4; i += blockDim.x) {
        const int j = i / W4, d = (i - j * W4) * 4;
        const int key = kt + j;
        float kk[4] = {0.f, 0.f, 0.f, 0.f};
        if (key < end) {
          const int page = bt[key / p.page_size];
          if (page < 0)
            atomicOr(p.status, RL_STATUS_BAD_PAGE);
          else
            load4((const T*)p.pool + ((size_t)page * p.page_size + key % p.page_size) * W + d, kk);
        }
        float* kd = k_s + j * (W + 1) + d;
        kd[0] = kk[0]; kd[1] = kk[1]; kd[2] = kk[2]; kd[3] = kk[3];
      }
      __syncthreads();
      const float* kr = k_s + lane * (W + 1);
      const bool valid = kt + lane < end;
      const int cnt = min(LD_KV, end - kt);
      float pr[HPW];
#pragma unroll
      for (int r = 0; r < HPW; ++r) {
        const int h = h0 + r * LD_WARPS;
        pr[r] = 0.f;
        if (h >= H) continue;  // the same for the whole warp
        const float* qr = q_s + (size_t)h * W;
        float s = 0.f;
        for (int d = 0; d < W; ++d) s = fmaf(qr[d], kr[d], s);
        const float sv = valid ? s : -CUDART_INF_F;
        const float m_new = fmaxf(m[r], warp_max(sv));
        const float alpha = m_new == -CUDART_INF_F ? 1.f : expf(m[r] - m_new);
        pr[r] = valid ? expf(sv - m_new) : 0.f;
        l[r] = l[r] * alpha + warp_sum(pr[r]);
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) o[r][c] *= alpha;
        m[r] = m_new;
      }
      for (int j = 0; j < cnt; ++j) {
        float pj[HPW];
#pragma unroll
        for (int r = 0; r < HPW; ++r) pj[r] = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
          const int d = lane + 32 * c;
          const float vv = d < p.rank ? k_s[j * (W + 1) + d] : 0.f;
#pragma unroll
          for (int r = 0; r < HPW; ++r) o[r][c] = fmaf(pj[r], vv, o[r][c]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < HPW; ++r) {
      const int h = h0 + r * LD_WARPS;
      if (h >= H) continue;
      if (n_splits == 1) {
        const float inv = 1.0f / l[r];
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
          const int d = lane + 32 * c;
          if (d < p.rank) out[(size_t)n * p.out_stride + (size_t)h * p.rank + d] = from_f32<T>(o[r][c] * inv);
        }
      } else {
        const size_t row = ((size_t)blockIdx.x * H + h) * n_splits + sp;
        if (lane == 0) {
          part_ml[2 * row] = m[r];
          part_ml[2 * row + 1] = l[r];
        }
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
          const int d = lane + 32 * c;
          if (d < p.rank) part_o[row * p.rank + d] = o[r][c];
        }
      }
    }
  }
}

// out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s over the parts, in their order.  The parts'
// weights e^{m_s - M} / sum are worked out once a block (at most 64 parts), then every thread sums
// its columns.
template <typename T>
__global__ __launch_bounds__(128) void latent_attn_merge_kernel(const float* __restrict__ part_o,
                                                                const float* __restrict__ part_ml, int n_splits,
                                                                const int* __restrict__ decode_reqs,
                                                                const int* __restrict__ q_start,
                                                                const int* __restrict__ slots, T* __restrict__ out,
                                                                long out_stride, int n_heads, int rank) {
  __shared__ float w_s[64];
  pdl_begin();
  const int di = blockIdx.x, h = blockIdx.y;
  const int req = decode_reqs[di];
  if (slots[req] < 0) return;  // written by the attention kernel
  const size_t row0 = ((size_t)di * n_heads + h) * n_splits;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    if (lane < n_splits) {
      m0 = part_ml[2 * (row0 + lane)];
      l0 = part_ml[2 * (row0 + lane) + 1];
    }
    if (lane + 32 < n_splits) {
      m1 = part_ml[2 * (row0 + lane + 32)];
      l1 = part_ml[2 * (row0 + lane + 32) + 1];
    }
    const float top = warp_max(fmaxf(m0, m1));
    const float e0 = m0 == -CUDART_INF_F ? 0.f : expf(m0 - top), e1 = m1 == -CUDART_INF_F ? 0.f : expf(m1 - top);
    // the denominator in the parts' order: lane by lane
    float den = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float term = s < 32 ? __shfl_sync(0xffffffffu, e0 * l0, s) : __shfl_sync(0xffffffffu, e1 * l1, s - 32);
      den += term;
    }
    const float inv = 1.0f / den;
    w_s[lane] = e0 * inv;
    w_s[lane + 32] = e1 * inv;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) acc = fmaf(w_s[s], part_o[(row0 + s) * rank + d], acc);
    out[(size_t)q_start[req] * out_stride + (size_t)h * rank + d] = from_f32<T>(acc);
  }
}

// ---- bfloat16 on the tensor cores ---------------------------------------------------------------
//
// All heads of a token meet the same cached rows, so the (token, head) pairs of a request are
// simply rows of one matrix Q': a block takes RB consecutive pairs (of up to 16 tokens of a
// prompt portion, or the heads of one decoded token and one part of its keys) and walks the
// keys in tiles of 32 staged in shared memory.  Per tile a warp computes S = Q' K^T for its 16
// rows with mma.sync m16n8k16 (operands read straight from shared memory, whose row stride is
// 4 words mod 8: no bank conflicts), masks by each row's own position, keeps the online softmax
// of its rows in float32 (base 2; the sink is the starting value), repacks P from the
// accumulator layout into A fragments and adds P V, V being the first `rank` columns of the
// same tile, fetched transposed with ldmatrix.  A warp holds NVW value tiles of 8 columns;
// latents beyond 256 entries are split over two warps that share their rows (DVS = 2).
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ void mma_16x8x16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int NVW, int DVS, int NKT>
__global__ __launch_bounds__(128) void latent_attn_mma_kernel(LatentParams p, const int* __restrict__ tiles,
                                                              const int* __restrict__ decode_reqs, int decode,
                                                              int n_splits, float* __restrict__ part_o,
                                                              float* __restrict__ part_ml) {
  using bf16 = __nv_bfloat16;
  constexpr int RB = 16 * (4 / DVS), LM_KT = 8 * NKT;
  extern __shared__ __align__(16) unsigned char latent_smem[];
  pdl_begin();
  const int W = p.row_width, H = p.n_heads;
  const int Wk = (W + 15) & ~15, LD = Wk + 8, W8 = Wk >> 3;
  bf16* q_s = reinterpret_cast<bf16*>(latent_smem);  // [RB][LD]
  bf16* k_s = q_s + RB * LD;                         // [2 stages][LM_KT][LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  int req, t0 = 0, sp = 0;
  if (!decode) {
    // the list runs from a request's first tile to its last, which walks the most keys: blocks take
    // it from the back, so that the long ones start first and the short ones fill the SMs' last round
    const int tile = gridDim.y - 1 - blockIdx.y;  // prompt portions: grid (chunks of rows, tiles)
    req = tiles[2 * tile];
    t0 = tiles[2 * tile + 1];
  } else {
    req = decode_reqs[blockIdx.x];
    sp = blockIdx.z;
  }
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int rows_total = (decode ? 1 : min(LT_Q, q_len - t0)) * H;
  const int row0 = (decode ? blockIdx.y : blockIdx.x) * RB;
  if (row0 >= rows_total) return;
  bf16* out = (bf16*)p.out;
  const int slot = p.slots[req];
  if (slot < 0) {  // padding of a fixed-size batch
    if (sp == 0)
      for (int i = tid; i < min(RB, rows_total - row0) * p.rank; i += blockDim.x) {
        const int gr = row0 + i / p.rank;
        out[(size_t)(qs + t0 + gr / H) * p.out_stride + (size_t)(gr % H) * p.rank + i % p.rank] = __float2bfloat16_rn(0.f);
      }
    return;
  }
  const int kv_len = p.kv_len[req];
  const int pos0 = kv_len - q_len;
  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  int beg = 0, end = pos0 + t0 + (min(rows_total, row0 + RB) - 1) / H + 1;
  if (decode) {
    const int chunk = ((kv_len + n_splits - 1) / n_splits + LM_KT - 1) / LM_KT * LM_KT;
    beg = sp * chunk;
    end = min(kv_len, beg + chunk);
  }
  const bf16* q = (const bf16*)p.q;
  for (int i = tid; i < RB * W8; i += 128) {
    const int r = i / W8, c = (i - r * W8) * 8;
    const int gr = row0 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (gr < rows_total && c < W)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(qs + t0 + gr / H) * p.q_stride + (size_t)(gr % H) * W + c);
    *reinterpret_cast<uint4*>(q_s + r * LD + c) = v;
  }
  const int rg = warp / DVS, vh = warp % DVS;
  const int row_a = row0 + rg * 16 + g, row_b = row_a + 8;
  const int qpos_a = row_a < rows_total ? pos0 + t0 + row_a / H : -1;
  const int qpos_b = row_b < rows_total ? pos0 + t0 + row_b / H : -1;
  const float scale2 = p.scale * LOG2E;
  const bool sinked = p.sink != nullptr && sp == 0;
  float m_a = sinked && row_a < rows_total ? p.sink[row_a % H] * LOG2E : -CUDART_INF_F;
  float m_b = sinked && row_b < rows_total ? p.sink[row_b % H] * LOG2E : -CUDART_INF_F;
  float l_a = m_a == -CUDART_INF_F ? 0.f : 1.f, l_b = m_b == -CUDART_INF_F ? 0.f : 1.f;
  float o[NVW][4];
#pragma unroll
  for (int i = 0; i < NVW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t q_s_addr = (uint32_t)__cvta_generic_to_shared(q_s);
  const uint32_t k_s_addr = (uint32_t)__cvta_generic_to_shared(k_s);

  // a tile of keys into stage `st`: valid 16-byte pieces by cp.async, the rest zeros
  auto stage_keys = [&](int kt, int st) {
    bf16* dst = k_s + st * LM_KT * LD;
    for (int i = tid; i < LM_KT * W8; i += 128) {
      const int j = i / W8, c = (i - j * W8) * 8;
      const int key = kt + j;
      int page = -1;
      if (key < end && c < W) {
        page = bt[key / p.page_size];
        if (page < 0) atomicOr(p.status, RL_STATUS_BAD_PAGE);
      }
      if (page >= 0) {
        const bf16* src = (const bf16*)p.pool + ((size_t)page * p.page_size + key % p.page_size) * W + c;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + j * LD + c)),
                     "l"(src)
                     : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst + j * LD + c) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (beg < end) stage_keys(beg, 0);
  int st = 0;
  for (int kt = beg; kt < end; kt += LM_KT, st ^= 1) {
    if (kt + LM_KT < end) {
      stage_keys(kt + LM_KT, st ^ 1);  // the stage was last read two tiles ago, before that tile's closing barrier
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();  // this tile has landed for every thread (first pass: q_s is written too)
    const uint32_t k_t_addr = k_s_addr + (uint32_t)(st * LM_KT * LD * 2);
    float s[NKT][4];
#pragma unroll
    for (int ni = 0; ni < NKT; ++ni) s[ni][0] = s[ni][1] = s[ni][2] = s[ni][3] = 0.f;
    // fragments by ldmatrix, four 8 x 8 pieces an instruction: of Q (rows, k), (rows + 8, k),
    // (rows, k + 8), (rows + 8, k + 8); of the keys (keys, k), (keys, k + 8), (keys + 8, k), (keys + 8, k + 8)
    const uint32_t qa_addr = q_s_addr + (uint32_t)(((rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8) * 2);
    const uint32_t kb_addr = k_t_addr + (uint32_t)((((lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8) * 2);
    // two sets of accumulators take the K steps in turn: every step adds into the accumulators of
    // the step before last, so twice as many independent mma chains are in flight (the kernel's
    // first stall reason was the fixed latency between dependent mma instructions)
    float s2[NKT][4];
#pragma unroll
    for (int ni = 0; ni < NKT; ++ni) s2[ni][0] = s2[ni][1] = s2[ni][2] = s2[ni][3] = 0.f;
    auto score_step = [&](int ks, float (&acc)[NKT][4]) {
      uint32_t a[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                   : "r"(qa_addr + (uint32_t)(ks * 2)));
#pragma unroll
      for (int ni = 0; ni < NKT; ni += 2) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(kb_addr + (uint32_t)((ni * 8 * LD + ks) * 2)));
        mma_16x8x16(acc[ni], a, b0, b1);
        mma_16x8x16(acc[ni + 1], a, b2, b3);
      }
    };
    int ks = 0;
    for (; ks + 32 <= Wk; ks += 32) {
      score_step(ks, s);
      score_step(ks + 16, s2);
    }
    if (ks < Wk) score_step(ks, s);
#pragma unroll
    for (int ni = 0; ni < NKT; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[ni][c] += s2[ni][c];
    // mask by each row's own position, online softmax in base 2
    float top_a = -CUDART_INF_F, top_b = -CUDART_INF_F;
#pragma unroll
    for (int ni = 0; ni < NKT; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = kt + ni * 8 + 2 * t + (c & 1);
        const bool ok = key < end && key <= (c < 2 ? qpos_a : qpos_b);
        s[ni][c] = ok ? s[ni][c] * scale2 : -CUDART_INF_F;
        if (c < 2) top_a = fmaxf(top_a, s[ni][c]); else top_b = fmaxf(top_b, s[ni][c]);
      }
    const float new_a = fmaxf(m_a, quad_max(top_a)), new_b = fmaxf(m_b, quad_max(top_b));
    const float alpha_a = new_a == -CUDART_INF_F ? 1.f : exp2f(m_a - new_a);
    const float alpha_b = new_b == -CUDART_INF_F ? 1.f : exp2f(m_b - new_b);
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int ni = 0; ni < NKT; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float top = c < 2 ? new_a : new_b;
        const float pv = s[ni][c] == -CUDART_INF_F ? 0.f : exp2f(s[ni][c] - top);
        s[ni][c] = pv;
        if (c < 2) sum_a += pv; else sum_b += pv;
      }
    l_a = l_a * alpha_a + quad_sum(sum_a);
    l_b = l_b * alpha_b + quad_sum(sum_b);
    m_a = new_a;
    m_b = new_b;
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      o[i][0] *= alpha_a; o[i][1] *= alpha_a; o[i][2] *= alpha_b; o[i][3] *= alpha_b;
    }
    // P as A fragments of two steps of 16 keys, then O += P V with V read transposed
#pragma unroll
    for (int j = 0; j < NKT / 2; ++j) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
      pa[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
      pa[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
      pa[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
      for (int nv = 0; nv < NVW; nv += 2) {
        const int col = min((vh * NVW + nv + (lane >> 4)) * 8, Wk - 8);
        const uint32_t addr = k_t_addr + (uint32_t)(((j * 16 + (lane & 15)) * LD + col) * 2);
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(addr));
        mma_16x8x16(o[nv], pa, b0, b1);
        mma_16x8x16(o[nv + 1], pa, b2, b3);
      }
    }
    __syncthreads();  // the stage may be written again
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int gr = half ? row_b : row_a;
    if (gr >= rows_total) continue;
    const float l = half ? l_b : l_a, m = half ? m_b : m_a;
    const int tok = qs + t0 + gr / H, hd = gr % H;
    if (!decode || n_splits == 1) {
      const float inv = 1.0f / l;
#pragma unroll
      for (int nv = 0; nv < NVW; ++nv) {
        const int d = (vh * NVW + nv) * 8 + 2 * t;
        if (d < p.rank) out[(size_t)tok * p.out_stride + (size_t)hd * p.rank + d] = __float2bfloat16_rn(o[nv][2 * half] * inv);
        if (d + 1 < p.rank)
          out[(size_t)tok * p.out_stride + (size_t)hd * p.rank + d + 1] = __float2bfloat16_rn(o[nv][2 * half + 1] * inv);
      }
    } else {
      const size_t prow = ((size_t)blockIdx.x * H + hd) * n_splits + sp;
      if (t == 0 && vh == 0) {
        part_ml[2 * prow] = m == -CUDART_INF_F ? m : m * LN2;  // the merge works in natural units
        part_ml[2 * prow + 1] = l;
      }
#pragma unroll
      for (int nv = 0; nv < NVW; ++nv) {
        const int d = (vh * NVW + nv) * 8 + 2 * t;
        if (d < p.rank) part_o[prow * p.rank + d] = o[nv][2 * half];
        if (d + 1 < p.rank) part_o[prow * p.rank + d + 1] = o[nv][2 * half + 1];
      }
    }
  }
}

// DVS_DEC, NVW_DEC: the form of the kernel that decoded tokens take (few heads: the value columns
// spread over all four warps, so that none of them idles on rows that do not exist).
template <int NVW, int DVS, int NKT, int NVW_DEC, int DVS_DEC>
static inline void launch_latent_mma(const LatentParams& p, const int* tiles, int n_tiles, const int* decode_reqs,
                                     int n_decode, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
  constexpr int RB = 16 * (4 / DVS), RB_DEC = 16 * (4 / DVS_DEC), LM_KT = 8 * NKT, KT_DEC = 32;
  const int Wk = (p.row_width + 15) & ~15;
  const size_t smem = (size_t)(RB + 2 * LM_KT) * (Wk + 8) * 2;
  static size_t granted = 0;
  if (smem > 48 * 1024 && smem > granted) {
    cudaFuncSetAttribute(latent_attn_mma_kernel<NVW, DVS, NKT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    granted = smem;
  }
  // Prompt portions run for hundreds of microseconds and want every block the registers allow:
  // with the common half-and-half split of an SM's memory only one block of 76 KB fits (measured:
  // 4 warps an SM, 0.22 instructions issued a cycle and scheduler), so this form asks for all of
  // it as shared memory.
  static bool carved = false;
  if (!carved) {
    cudaFuncSetAttribute(latent_attn_mma_kernel<NVW, DVS, NKT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    carved = true;
  }
  if (n_tiles > 0)
    launch_pdl_split(false, latent_attn_mma_kernel<NVW, DVS, NKT>, dim3((LT_Q * p.n_heads + RB - 1) / RB, n_tiles), 128, smem, stream, p,
               tiles, decode_reqs, 0, 1, part_o, part_ml);
  if (n_decode > 0) {
    const size_t smem_dec = (size_t)(RB_DEC + 2 * KT_DEC) * (Wk + 8) * 2;
    static size_t granted_dec = 0;
    if (smem_dec > 48 * 1024 && smem_dec > granted_dec) {
      cudaFuncSetAttribute(latent_attn_mma_kernel<NVW_DEC, DVS_DEC, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem_dec);
      granted_dec = smem_dec;
    }
    launch_pdl(latent_attn_mma_kernel<NVW_DEC, DVS_DEC, 4>, dim3(n_decode, (p.n_heads + RB_DEC - 1) / RB_DEC, n_splits),
               128, smem_dec, stream, p, tiles, decode_reqs, 1, n_splits, part_o, part_ml);
    if (n_splits > 1)
      launch_pdl(latent_attn_merge_kernel<__nv_bfloat16>, dim3(n_decode, p.n_heads), 128, 0, stream,
                 (const float*)part_o, (const float*)part_ml, n_splits, decode_reqs, p.q_start, p.slots,
                 (__nv_bfloat16*)p.out, p.out_stride, p.n_heads, p.rank);
  }
}

static int latent_prefill_form = 0;

// The tensor-core kernel for these sizes, or false when it does not take them.
static inline bool dispatch_latent_mma(const LatentParams& p, const int* tiles, int n_tiles, const int* decode_reqs,
                                       int n_decode, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
  const int Wk = (p.row_width + 15) & ~15;
  if (n_tiles > 65535) return false;
  const int n8 = (p.rank + 7) / 8;
  // shared memory of the form the rule below picks: its rows of queries and two stages of keys
  const int rows = n8 > 32 ? 32 : 64, keys = n8 <= 16 ? 64 : 32;
  if ((size_t)(rows + 2 * keys) * (Wk + 8) * 2 > 200 * 1024) return false;
  // decoded tokens: up to 16 heads are one warp's rows, up to 32 two warps'
  const bool few = p.n_heads <= 16, some = p.n_heads <= 32;
#define RL_LATENT_MMA(NVW, DVS, NKT, NVW4, NVW2)                                                                         \
  do {                                                                                                                   \
    if (few) launch_latent_mma<NVW, DVS, NKT, NVW4, 4>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, part_o, part_ml, stream); \
    else if (some) launch_latent_mma<NVW, DVS, NKT, NVW2, 2>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, part_o, part_ml, stream); \
    else launch_latent_mma<NVW, DVS, NKT, NVW, DVS>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, part_o, part_ml, stream); \
  } while (0)
  // latent_prefill_form (for measurements): 0 the rule below; 1: latents of 129 to 256 with their
  // value columns over two warps; 2: the same with key tiles of 64
  if (n8 <= 2) RL_LATENT_MMA(2, 1, 8, 2, 2);
  else if (n8 <= 4) RL_LATENT_MMA(4, 1, 8, 2, 2);
  else if (n8 <= 8) RL_LATENT_MMA(8, 1, 8, 2, 4);
  else if (n8 <= 16) RL_LATENT_MMA(16, 1, 8, 4, 8);
  else if (n8 <= 32 && latent_prefill_form == 1) RL_LATENT_MMA(16, 2, 4, 8, 16);
  else if (n8 <= 32 && latent_prefill_form == 2 && (size_t)(32 + 128) * (Wk + 8) * 2 <= 200 * 1024)
    RL_LATENT_MMA(16, 2, 8, 8, 16);
  else if (n8 <= 32) RL_LATENT_MMA(32, 1, 4, 8, 16);
  else if (n8 <= 64) RL_LATENT_MMA(32, 2, 4, 16, 32);
  else return false;
#undef RL_LATENT_MMA
  return true;
}

template <typename T, int NCHUNK>
static inline void launch_latent(const LatentParams& p, const int* tiles, int n_tiles, const int* decode_reqs,
                                 int n_decode, int n_splits, bool decode_by_request, float* part_o, float* part_ml,
                                 cudaStream_t stream) {
  const int W = p.row_width;
  const int tile_blocks = n_tiles + (decode_by_request ? 0 : n_decode);
  if (tile_blocks > 0) {
    const size_t smem = (size_t)(LT_Q * W + LT_KV * (W + 1)) * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attn_tile_kernel<T, NCHUNK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(latent_attn_tile_kernel<T, NCHUNK>, dim3(tile_blocks, p.n_heads), 128, smem, stream, p, tiles, n_tiles,
               decode_reqs);
  }
  if (decode_by_request && n_decode > 0) {
    const size_t smem = (size_t)(LD_KV * (W + 1) + p.n_heads * W) * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attn_decode_kernel<T, NCHUNK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(latent_attn_decode_kernel<T, NCHUNK>, dim3(n_decode, n_splits), 32 * LD_WARPS, smem, stream, p,
               decode_reqs, n_splits, part_o, part_ml);
    if (n_splits > 1)
      launch_pdl(latent_attn_merge_kernel<T>, dim3(n_decode, p.n_heads), 128, 0, stream, (const float*)part_o,
                 (const float*)part_ml, n_splits, decode_reqs, p.q_start, p.slots, (T*)p.out, p.out_stride, p.n_heads,
                 p.rank);
  }
}

template <typename T>
static inline int dispatch_latent(const LatentParams& p, const int* tiles, int n_tiles, const int* decode_reqs,
                                  int n_decode, int n_splits, bool by_request, float* part_o, float* part_ml,
                                  cudaStream_t stream) {
  const int chunks = (p.rank + 31) / 32;
  if (chunks <= 1) launch_latent<T, 1>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, by_request, part_o, part_ml, stream);
  else if (chunks <= 2) launch_latent<T, 2>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, by_request, part_o, part_ml, stream);
  else if (chunks <= 4) launch_latent<T, 4>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, by_request, part_o, part_ml, stream);
  else if (chunks <= 8) launch_latent<T, 8>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, by_request, part_o, part_ml, stream);
  else if (chunks <= 16) launch_latent<T, 16>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, by_request, part_o, part_ml, stream);
  else return -2;
  return 0;
}

}  // namespace rl

// How many bytes of shared memory the kernels above may ask for.
static constexpr size_t LATENT_SMEM_LIMIT = 200 * 1024;

// Which form of the tensor-core kernel prompt portions take (measurements; 0: the default rule).
RL_EXPORT void rl_latent_prefill_form(int form) { rl::latent_prefill_form = form; }

// 1 if the sizes fit the kernels (value width up to 512, shared memory), else 0.
RL_EXPORT int rl_latent_attention_fits(int n_heads, int rank, int row_width) {
  if (rank <= 0 || rank > 512 || row_width < rank || row_width % 8 != 0 || n_heads <= 0) return 0;
  const size_t tile = (size_t)(rl::LT_Q * row_width + rl::LT_KV * (row_width + 1)) * sizeof(float);
  return tile <= LATENT_SMEM_LIMIT ? 1 : 0;
}

// 1 if the all-heads decode kernel fits these sizes (its queries lie in shared memory).
RL_EXPORT int rl_latent_decode_fits(int n_heads, int rank, int row_width) {
  if (!rl_latent_attention_fits(n_heads, rank, row_width)) return 0;
  const size_t smem = (size_t)(rl::LD_KV * (row_width + 1) + (size_t)n_heads * row_width) * sizeof(float);
  return smem <= LATENT_SMEM_LIMIT ? 1 : 0;
}

// dkv: float32 [tokens, >= rank + rot_dim] with row stride ld: the first `rank` entries are
// normalised (gamma, eps), the next `rot_dim` rotated in their first `rot_dims` entries; rot_mult: a factor
// of the cosines and sines (of the turned entries), 1 for a plain rotation.
RL_EXPORT int rl_latent_kv_write(int dtype, const float* dkv, long ld, const float* gamma, float eps,
                                 const float* inv_freq, int rot_dims, void* pool, const int* block_table,
                                 int bt_stride, const int* positions, const int* req_of_token, const int* slots,
                                 int n_tokens, int rank, int rot_dim, int row_width, int page_size, int max_pos,
                                 float rot_mult, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || row_width < rank + rot_dim ||
      status == nullptr)
    return -2;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::latent_kv_write_kernel<float>, n_tokens, 128, 0, stream, dkv, ld, gamma, eps, inv_freq, rot_dims,
                   (float*)pool, block_table, bt_stride, positions, req_of_token, slots, n_tokens, rank, rot_dim,
                   row_width, page_size, max_pos, rot_mult, status);
  else
    rl::launch_pdl(rl::latent_kv_write_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, dkv, ld, gamma, eps, inv_freq,
                   rot_dims, (__nv_bfloat16*)pool, block_table, bt_stride, positions, req_of_token, slots, n_tokens,
                   rank, rot_dim, row_width, page_size, max_pos, rot_mult, status);
  RL_CHECK_LAUNCH();
  return 0;
}

// q: [tokens, heads * head_in] (row stride q_stride), head h's rotated part at h*head_in + plain;
// rows: [tokens, heads * row_width] (row stride rows_stride), written at [rank, row_width).
RL_EXPORT int rl_latent_q_rope(int dtype, const void* q, long q_stride, int head_in, int plain, void* rows,
                               long rows_stride, int row_width, int rank, int rot_dim, int rot_dims,
                               const float* inv_freq, const int* positions, int n_tokens, int n_heads,
                               float rot_mult, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rot_dims > rot_dim || (rot_dims & 1) || row_width < rank + rot_dim || plain + rot_dim > head_in) return -2;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::latent_q_rope_kernel<float>, n_tokens, 128, 0, stream, (const float*)q, q_stride, head_in, plain,
                   (float*)rows, rows_stride, row_width, rank, rot_dim, rot_dims, inv_freq, positions, n_tokens, n_heads,
                   rot_mult);
  else
    rl::launch_pdl(rl::latent_q_rope_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, (const __nv_bfloat16*)q, q_stride,
                   head_in, plain, (__nv_bfloat16*)rows, rows_stride, row_width, rank, rot_dim, rot_dims, inv_freq,
                   positions, n_tokens, n_heads, rot_mult);
  RL_CHECK_LAUNCH();
  return 0;
}

// tiles: [n_tiles][2] = (request, first query) of 16-query tiles of prompt portions;
// decode_reqs: requests with one query.  decode_by_request: decoded requests go to the kernel
// that takes all heads of a request in one block, their keys cut into n_splits parts
// (part_o: n_decode*heads*n_splits*rank floats, part_ml: n_decode*heads*n_splits*2); otherwise
// they are tiles of one query.  bfloat16 runs on the tensor-core kernel (decoded requests then
// always by request) unless simt_only is set (for comparisons) or its sizes do not fit.
RL_EXPORT int rl_latent_attention(int dtype, const void* q, long q_stride, const void* pool, const int* block_table,
                                  int bt_stride, const int* q_start, const int* kv_len, const int* slots, void* out,
                                  long out_stride, const float* sink, int n_heads, int rank, int row_width,
                                  int page_size, float scale, const int* tiles, int n_tiles, const int* decode_reqs,
                                  int n_decode, int decode_by_request, int n_splits, float* part_o, float* part_ml,
                                  int simt_only, int* status, cudaStream_t stream) {
  if (!rl_latent_attention_fits(n_heads, rank, row_width) || status == nullptr) return -2;
  if (decode_by_request && !rl_latent_decode_fits(n_heads, rank, row_width)) return -3;
  if (n_splits < 1 || n_splits > 64 || (decode_by_request && n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
    return -4;  // the merge takes up to 64 parts
  rl::LatentParams p{q, q_stride, pool, block_table, bt_stride, q_start, kv_len, slots, out, out_stride, sink,
                     n_heads, rank, row_width, page_size, scale, status};
  int rc = 0;
  if (dtype == RL_F32)
    rc = rl::dispatch_latent<float>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, decode_by_request != 0, part_o,
                                    part_ml, stream);
  else if (!(simt_only == 0 && (n_decode == 0 || decode_by_request) &&
             rl::dispatch_latent_mma(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, part_o, part_ml, stream)))
    rc = rl::dispatch_latent<__nv_bfloat16>(p, tiles, n_tiles, decode_reqs, n_decode, n_splits, decode_by_request != 0,
                                            part_o, part_ml, stream);
  if (rc != 0) return rc;
  RL_CHECK_LAUNCH();
  return 0;
}
