// Causal attention with a distance bias, a query temperature, key and value sizes of their own, grouped
// key/value heads and an output gate, over a paged cache that keeps one row a token and key/value head:
// [key (dk entries) | value (dv entries)], the value at entry `v_at`.
//
//   score(i, j) = (q_i . k_j) * scale * temp(i) - slope_h * (i - j),  j <= i
//   temp(i)     = 1 + temp_coef * ln(floor((i + 1) / temp_every) + 1)          (temp_every = 0: 1)
//   slope_h     : a table the caller gives, one entry a head                    (absent: no bias)
//   head_scale  : a further factor of the score per head, from a table            (absent: 1)
//   window      : a query at i sees the keys j with 0 <= i - j < window            (0: all keys j <= i);
//                 pages that lie wholly before a block's window are never looked up (the cache gives them back)
//   sink        : one more term exp(sink_h) in the softmax's denominator, a table with one entry a head; it
//                 has no key and no value and is not scaled                       (absent: a plain softmax)
//   out         = softmax(score) V * sigmoid(gate)                             (gate absent: no gate); the gate's
//                 logits are one a value column, or (gate_per_head) one a head
//
// Scores, softmax and the weighted sums are float32 whatever the cache holds.  Queries and gate logits are
// float32 columns of the layer's packed projections.
//
// `bias_kv_store_kernel` writes a step's keys and values into their pages and mixes the values on the way:
// v <- (1 - lambda) v + lambda v_src with v_src the values that an earlier layer computed for the same tokens
// (that layer leaves them in a float32 buffer: mode "source"); the pages receive the value after mixing.
//
// `bias_attn_kernel`: rows of a block are (token, head) pairs that share a key/value head, so a key tile
// fetched once serves all of a group's heads; 32 rows x 32 keys a round, online softmax, float32 on the CUDA
// cores.  A decoded token is a tile of one token; where a step has few of them, the keys of each are cut into
// parts, a block a part, and `bias_attn_merge_kernel` puts the parts together in their order.
#include <math_constants.h>

#include "common.cuh"

namespace rl {

constexpr int BA_ROWS = 32, BA_KEYS = 32, BA_THREADS = 128;  // BA_ROWS: the rows of a prompt tile's block

struct BiasAttnParams {
  const float* q;  // [tokens, ldq]; head h at columns [h * dk, (h + 1) * dk)
  long ldq;
  const float* gate;  // [tokens, ldg] logits, head h at [h * dv, ...); or null
  long ldg;
  const void* pool;  // [pages, 1, n_kv, page_size, row]
  const int* block_table;
  long ldt;
  const int *q_start, *kv_len, *slots, *tiles, *decode_reqs;
  void* out;  // [tokens, ldo], head h at [h * dv, ...)
  long ldo;
  int n_heads, n_kv, dk, dv, v_at, row, page_size, max_pages;
  int n_tiles, tile_tokens, tokens_per_block, heads_per_block, n_decode;
  float scale, temp_coef;
  int temp_every;
  const float* slopes;  // [n_heads] or null
  int* status;
  int window;               // 0: none
  const float* head_scale;  // [n_heads] or null
  // decoded tokens whose keys are cut into parts: a block takes one part and leaves its unnormalised sums
  // in part_o [(decoded request, head, part), dv] and (maximum, sum of weights) in part_ml
  int n_splits;
  float* part_o;
  float* part_ml;
  const float* sink;  // [n_heads] or null
  int gate_per_head;  // the gate holds one logit a (token, head): [tokens, ldg], head h at column h
};

// The gate's logits of a (token, head): a pointer to the head's dv logits (stride 1), or to its one logit (stride 0).
__device__ __forceinline__ const float* bias_gate_row(const BiasAttnParams& p, int tok, int head, int& stride) {
  stride = p.gate_per_head ? 0 : 1;
  if (p.gate == nullptr) return nullptr;
  return p.gate + (size_t)tok * p.ldg + (p.gate_per_head ? (size_t)head : (size_t)head * p.dv);
}

}  // namespace rl

#include "bias_attention_mma.cuh"

namespace rl {

// LPR lanes share a row (their keys tx + LPR b, their value columns tx + LPR c), RPT rows a thread: a block has
// (BA_THREADS / LPR) * RPT rows.  Prompt tiles run 8 lanes x 2 rows (32 rows); a decoded token has only its
// group's heads as rows, so its blocks run 16 or 32 lanes a row (8 or 4 rows) and every thread has work.
template <typename T, int LPR, int RPT, int DVC, typename TOut>
__global__ __launch_bounds__(BA_THREADS) void bias_attn_kernel(const BiasAttnParams p) {
  constexpr int ROWS = BA_THREADS / LPR * RPT, KPT = BA_KEYS / LPR;
  extern __shared__ __align__(16) float ba_s[];
  pdl_begin();
  const int subs = p.tile_tokens / p.tokens_per_block;
  int req, first;  // the request and the first of its new tokens that this block takes
  int split = 0, dec = -1;  // for a decoded token: which part of its keys, and its place among the decoded requests
  if ((int)blockIdx.x < p.n_tiles * subs) {
    const int tile = blockIdx.x / subs, sub = blockIdx.x - tile * subs;
    req = p.tiles[2 * tile];
    first = p.tiles[2 * tile + 1] + sub * p.tokens_per_block;
  } else {
    dec = (blockIdx.x - p.n_tiles * subs) / p.n_splits;
    split = (blockIdx.x - p.n_tiles * subs) - dec * p.n_splits;
    req = p.decode_reqs[dec];
    first = 0;
  }
  const bool parted = dec >= 0 && p.n_splits > 1;
  const int slot = p.slots[req];
  const int t_begin = p.q_start[req], n_new = p.q_start[req + 1] - t_begin;
  if (slot < 0 || first >= n_new) return;
  const int n_tok = min(p.tokens_per_block, n_new - first);
  const int pos0 = p.kv_len[req] - n_new + first;  // position of the block's first token
  const int g = blockIdx.y, hg = p.n_heads / p.n_kv;
  const int hb0 = blockIdx.z * p.heads_per_block;
  const int HB = p.heads_per_block;
  const int dk = p.dk, dv = p.dv;
  const int ldq_s = dk | 1, ldk_s = dk | 1, ldv_s = LPR * DVC;
  float* Qs = ba_s;                        // [ROWS][ldq_s]
  float* Ks = Qs + ROWS * ldq_s;           // [BA_KEYS][ldk_s]
  float* Vs = Ks + BA_KEYS * ldk_s;        // [BA_KEYS][ldv_s]
  float* Ps = Vs + BA_KEYS * ldv_s;        // [ROWS][BA_KEYS + 1]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ty = tid / LPR, tx = tid % LPR;
  // queries
  for (int r = warp; r < ROWS; r += BA_THREADS / 32) {
    const int tl = r / HB, hl = r - tl * HB;
    const bool ok = tl < n_tok && hb0 + hl < hg;
    const float* src = p.q + (size_t)(t_begin + first + tl) * p.ldq + (size_t)(g * hg + hb0 + hl) * dk;
    for (int d = lane; d < dk; d += 32) Qs[r * ldq_s + d] = ok ? src[d] : 0.f;
  }
  int row_pos[RPT], row_head[RPT];
  float row_mul[RPT], row_slope[RPT], m[RPT], l[RPT];
  bool row_ok[RPT];
  float acc[RPT][DVC];
#pragma unroll
  for (int a = 0; a < RPT; ++a) {
    const int r = ty * RPT + a, tl = r / HB, hl = r - tl * HB;
    row_ok[a] = tl < n_tok && hb0 + hl < hg;
    row_pos[a] = pos0 + tl;
    row_head[a] = g * hg + hb0 + hl;
    float temp = 1.0f;
    if (p.temp_every > 0) temp = 1.0f + p.temp_coef * logf((float)((row_pos[a] + 1) / p.temp_every + 1));
    row_mul[a] = p.scale * temp;
    if (p.head_scale != nullptr && row_ok[a]) row_mul[a] *= p.head_scale[row_head[a]];
    row_slope[a] = (p.slopes != nullptr && row_ok[a]) ? p.slopes[row_head[a]] : 0.f;
    m[a] = -CUDART_INF_F;
    l[a] = 0.f;
#pragma unroll
    for (int c = 0; c < DVC; ++c) acc[a][c] = 0.f;
  }
  const int last_pos = pos0 + n_tok - 1;
  const int first_seen = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;  // the earliest key any row of the block sees
  const T* pool = reinterpret_cast<const T*>(p.pool);
  const int* table = p.block_table + (size_t)slot * p.ldt;
  // Where each key of a tile lies (null: beyond the block's last position, or no page): looked up by one
  // thread a key for the tile AFTER the one being copied, so that the copies themselves, 16 bytes a thread
  // and several in flight, depend on nothing but shared memory.
  __shared__ const T* key_src[2][BA_KEYS];
  auto locate = [&](int j0, int buf) {
    if (tid < BA_KEYS) {
      const int j = j0 + tid;
      const T* src = nullptr;
      if (j <= last_pos && j >= first_seen) {
        const int lp = j / p.page_size;
        const int page = lp < p.max_pages ? table[lp] : -1;
        if (page < 0)
          atomicOr(p.status, RL_STATUS_BAD_PAGE);
        else
          src = pool + (((size_t)page * p.n_kv + g) * p.page_size + (j - lp * p.page_size)) * p.row;
      }
      key_src[buf][tid] = src;
    }
  };
  constexpr int EV = 16 / (int)sizeof(T);  // elements of a 16-byte piece
  const bool vec = dk % EV == 0 && dv % EV == 0 && p.row % EV == 0 && p.v_at % EV == 0 &&
                   (reinterpret_cast<uintptr_t>(p.pool) & 15) == 0;
  for (int i = tid; i < BA_KEYS * ldv_s; i += BA_THREADS) Vs[i] = 0.f;  // the fill beyond dv stays zero
  int j_begin = first_seen / BA_KEYS * BA_KEYS, j_end = last_pos + 1;  // the keys this block walks
  if (parted) {
    const int tiles_all = (last_pos + BA_KEYS) / BA_KEYS - j_begin / BA_KEYS;
    const int per = (tiles_all + p.n_splits - 1) / p.n_splits;
    j_end = min(j_end, j_begin + (split + 1) * per * BA_KEYS);
    j_begin += split * per * BA_KEYS;
  }
  locate(j_begin, 0);
  int buf = 0;
  for (int j0 = j_begin; j0 < j_end; j0 += BA_KEYS, buf ^= 1) {
    __syncthreads();  // the tile before has been used; this tile's places (and, the first time, the queries) are known
    if (vec) {
      const int kp = dk / EV, vp = dv / EV, per_key = kp + vp;
#pragma unroll 4
      for (int i = tid; i < BA_KEYS * per_key; i += BA_THREADS) {
        const int jj = i / per_key, piece = i - jj * per_key;
        const T* src = key_src[buf][jj];
        const bool is_v = piece >= kp;
        const int at = is_v ? (piece - kp) * EV : piece * EV;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (src != nullptr) raw = *reinterpret_cast<const uint4*>(src + (is_v ? p.v_at : 0) + at);
        const T* e = reinterpret_cast<const T*>(&raw);
        float* dst = is_v ? Vs + jj * ldv_s + at : Ks + jj * ldk_s + at;
#pragma unroll
        for (int x = 0; x < EV; ++x) dst[x] = to_f32(e[x]);
      }
    } else {
      const int per_key = dk + dv;
#pragma unroll 4
      for (int i = tid; i < BA_KEYS * per_key; i += BA_THREADS) {
        const int jj = i / per_key, c = i - jj * per_key;
        const T* src = key_src[buf][jj];
        const bool is_v = c >= dk;
        const float val = src != nullptr ? to_f32(src[is_v ? p.v_at + c - dk : c]) : 0.f;
        if (is_v) Vs[jj * ldv_s + c - dk] = val;
        else Ks[jj * ldk_s + c] = val;
      }
    }
    locate(j0 + BA_KEYS, buf ^ 1);
    __syncthreads();
    float s[RPT][KPT] = {};
    const float* q0 = Qs + (ty * RPT) * ldq_s;
    const float* kb = Ks + tx * ldk_s;
#pragma unroll 4
    for (int d = 0; d < dk; ++d) {
      float qa[RPT];
#pragma unroll
      for (int a = 0; a < RPT; ++a) qa[a] = q0[a * ldq_s + d];
#pragma unroll
      for (int b = 0; b < KPT; ++b) {
        const float kv = kb[b * LPR * ldk_s + d];
#pragma unroll
        for (int a = 0; a < RPT; ++a) s[a][b] = fmaf(qa[a], kv, s[a][b]);
      }
    }
#pragma unroll
    for (int a = 0; a < RPT; ++a) {
      float tile_max = -CUDART_INF_F;
#pragma unroll
      for (int b = 0; b < KPT; ++b) {
        const int j = j0 + tx + LPR * b;
        const bool see = row_ok[a] && j <= row_pos[a] && (p.window <= 0 || row_pos[a] - j < p.window);
        s[a][b] = see ? s[a][b] * row_mul[a] - row_slope[a] * (float)(row_pos[a] - j) : -CUDART_INF_F;
        tile_max = fmaxf(tile_max, s[a][b]);
      }
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
      const float m_new = fmaxf(m[a], tile_max);
      const float corr = m[a] == -CUDART_INF_F ? 0.f : expf(m[a] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int b = 0; b < KPT; ++b) {
        const float pr = s[a][b] == -CUDART_INF_F ? 0.f : expf(s[a][b] - m_new);
        Ps[(ty * RPT + a) * (BA_KEYS + 1) + tx + LPR * b] = pr;
        sum += pr;
      }
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l[a] = l[a] * corr + sum;
      m[a] = m_new;
#pragma unroll
      for (int c = 0; c < DVC; ++c) acc[a][c] *= corr;
    }
    __syncwarp();  // a row's probabilities are written and read by the lanes of one warp
    const float* p0 = Ps + (ty * RPT) * (BA_KEYS + 1);
#pragma unroll 4
    for (int jj = 0; jj < BA_KEYS; ++jj) {
      float w[RPT];
#pragma unroll
      for (int a = 0; a < RPT; ++a) w[a] = p0[a * (BA_KEYS + 1) + jj];
      const float* vr = Vs + jj * ldv_s + tx;
#pragma unroll
      for (int c = 0; c < DVC; ++c) {
        const float v = vr[LPR * c];
#pragma unroll
        for (int a = 0; a < RPT; ++a) acc[a][c] = fmaf(w[a], v, acc[a][c]);
      }
    }
  }
  if (parted) {
#pragma unroll
    for (int a = 0; a < RPT; ++a) {
      if (!row_ok[a]) continue;
      const size_t at = ((size_t)dec * p.n_heads + row_head[a]) * p.n_splits + split;
#pragma unroll
      for (int c = 0; c < DVC; ++c)
        if (tx + LPR * c < dv) p.part_o[at * dv + tx + LPR * c] = acc[a][c];
      if (tx == 0) {
        p.part_ml[2 * at] = m[a];
        p.part_ml[2 * at + 1] = l[a];
      }
    }
    return;
  }
#pragma unroll
  for (int a = 0; a < RPT; ++a) {
    if (!row_ok[a]) continue;
    const int tok = t_begin + first + (ty * RPT + a) / HB;
    const float inv = 1.0f / (l[a] + (p.sink != nullptr ? expf(p.sink[row_head[a]] - m[a]) : 0.f));
    TOut* o = reinterpret_cast<TOut*>(p.out) + (size_t)tok * p.ldo + (size_t)row_head[a] * dv;
    int gs;
    const float* gr = bias_gate_row(p, tok, row_head[a], gs);
#pragma unroll
    for (int c = 0; c < DVC; ++c) {
      const int col = tx + LPR * c;
      if (col < dv) {
        float v = acc[a][c] * inv;
        if (gr != nullptr) v *= 1.0f / (1.0f + expf(-gr[col * gs]));
        o[col] = from_f32<TOut>(v);
      }
    }
  }
}

// The parts of a decoded token's keys put together, in their order: out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M),
// times the gate.  A warp a (decoded request, head); lane s works out part s's weight once (at most 32 parts).
template <typename TOut>
__global__ __launch_bounds__(128) void bias_attn_merge_kernel(const BiasAttnParams p) {
  pdl_begin();
  const int dec = blockIdx.x, req = p.decode_reqs[dec];
  if (p.slots[req] < 0) return;
  const int tok = p.q_start[req], dv = p.dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y * 4 + warp;
  if (head >= p.n_heads) return;
  const size_t at = ((size_t)dec * p.n_heads + head) * p.n_splits;
  const float ms = lane < p.n_splits ? p.part_ml[2 * (at + lane)] : -CUDART_INF_F;
  const float ls = lane < p.n_splits ? p.part_ml[2 * (at + lane) + 1] : 0.f;
  const float M = warp_max(ms);
  const float w = ms == -CUDART_INF_F ? 0.f : expf(ms - M);
  float L = 0.f;  // summed in the parts' order, by every lane alike
  for (int s = 0; s < p.n_splits; ++s) L = fmaf(__shfl_sync(0xffffffffu, ls, s), __shfl_sync(0xffffffffu, w, s), L);
  if (p.sink != nullptr) L += expf(p.sink[head] - M);  // the sink counts once, after the parts
  TOut* o = reinterpret_cast<TOut*>(p.out) + (size_t)tok * p.ldo + (size_t)head * dv;
  int gs;
  const float* gr = bias_gate_row(p, tok, head, gs);
  for (int c0 = 0; c0 < dv; c0 += 32) {
    const int c = c0 + lane;
    float acc = 0.f;
    for (int s = 0; s < p.n_splits; ++s) {
      const float ws = __shfl_sync(0xffffffffu, w, s);
      if (c < dv && ws != 0.f) acc = fmaf(p.part_o[(at + s) * dv + c], ws, acc);
    }
    if (c < dv) {
      float v = acc / L;
      if (gr != nullptr) v *= 1.0f / (1.0f + expf(-gr[c * gs]));
      o[c] = from_f32<TOut>(v);
    }
  }
}

// mix: 0 values as they are; 1 also left in v_src (this layer is the source); 2 mixed with v_src by *lambda.
template <typename T>
__global__ void bias_kv_store_kernel(const float* __restrict__ k, long ldk, const float* __restrict__ v, long ldv,
                                     float* __restrict__ v_src, const float* __restrict__ lambda, int mix,
                                     T* __restrict__ pool, const int* __restrict__ block_table, long ldt,
                                     const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                     const int* __restrict__ slots, int n_tokens, int n_kv, int dk, int dv, int v_at,
                                     int row, int page_size, int max_pages, int* __restrict__ status) {
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  const int slot = slots[req_of_token[n]];
  if (slot < 0) return;
  const int pos = positions[n], lp = pos / page_size;
  const int page = (pos >= 0 && lp < max_pages) ? block_table[(size_t)slot * ldt + lp] : -1;
  const float lam = mix == 2 ? *lambda : 0.f;
  for (int i = threadIdx.x; i < n_kv * dv; i += blockDim.x) {  // the source is left even where the page is missing
    float val = v[(size_t)n * ldv + i];
    if (mix == 1) v_src[(size_t)n * n_kv * dv + i] = val;
    if (mix == 2) val = (1.0f - lam) * val + lam * v_src[(size_t)n * n_kv * dv + i];
    if (page >= 0) {
      const int g = i / dv, c = i - g * dv;
      pool[(((size_t)page * n_kv + g) * page_size + (pos - lp * page_size)) * row + v_at + c] = from_f32<T>(val);
    }
  }
  if (page < 0) {
    if (threadIdx.x == 0) atomicOr(status, pos < 0 || lp >= max_pages ? RL_STATUS_BAD_POSITION : RL_STATUS_BAD_PAGE);
    return;
  }
  for (int i = threadIdx.x; i < n_kv * dk; i += blockDim.x) {
    const int g = i / dk, c = i - g * dk;
    pool[(((size_t)page * n_kv + g) * page_size + (pos - lp * page_size)) * row + c] = from_f32<T>(k[(size_t)n * ldk + i]);
  }
}

template <typename T, int LPR, int RPT, int DVC, typename TOut>
static void launch_bias_attn(const BiasAttnParams& p, dim3 grid, cudaStream_t stream) {
  constexpr int ROWS = BA_THREADS / LPR * RPT;
  const size_t smem = ((size_t)ROWS * (p.dk | 1) + (size_t)BA_KEYS * (p.dk | 1) + (size_t)BA_KEYS * LPR * DVC +
                       (size_t)ROWS * (BA_KEYS + 1)) * sizeof(float);
  auto kernel = bias_attn_kernel<T, LPR, RPT, DVC, TOut>;
  if (smem > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      note_launch(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      raised = true;
    }
  }
  launch_pdl(kernel, grid, BA_THREADS, smem, stream, p);
}

// rows: 32 (prompt tiles, and decoded tokens of large groups), 8 or 4 (decoded tokens)
template <typename T, typename TOut>
static void dispatch_bias_attn(const BiasAttnParams& p, int rows, dim3 grid, cudaStream_t stream) {
  if (rows == 4) {
    if (p.dv <= 64) launch_bias_attn<T, 32, 1, 2, TOut>(p, grid, stream);
    else launch_bias_attn<T, 32, 1, 8, TOut>(p, grid, stream);
  } else if (rows == 8) {
    if (p.dv <= 64) launch_bias_attn<T, 16, 1, 4, TOut>(p, grid, stream);
    else launch_bias_attn<T, 16, 1, 16, TOut>(p, grid, stream);
  } else {
    if (p.dv <= 32) launch_bias_attn<T, 8, 2, 4, TOut>(p, grid, stream);
    else if (p.dv <= 64) launch_bias_attn<T, 8, 2, 8, TOut>(p, grid, stream);
    else if (p.dv <= 128) launch_bias_attn<T, 8, 2, 16, TOut>(p, grid, stream);
    else launch_bias_attn<T, 8, 2, 32, TOut>(p, grid, stream);
  }
}

static void dispatch_bias_attn_types(int cache_dtype, int out_dtype, const BiasAttnParams& p, int rows, dim3 grid,
                                     cudaStream_t stream) {
  if (cache_dtype == RL_F32) {
    if (out_dtype == RL_F32) dispatch_bias_attn<float, float>(p, rows, grid, stream);
    else dispatch_bias_attn<float, __nv_bfloat16>(p, rows, grid, stream);
  } else {
    if (out_dtype == RL_F32) dispatch_bias_attn<__nv_bfloat16, float>(p, rows, grid, stream);
    else dispatch_bias_attn<__nv_bfloat16, __nv_bfloat16>(p, rows, grid, stream);
  }
}

}  // namespace rl

// For comparisons: whether prompt tiles on the tensor cores may take the form whose key tiles travel by cp.async
// (on by default; sizes that cannot be copied in 16-byte pieces never take it).
RL_EXPORT void rl_bias_attention_async(int on) { rl::BIAS_ATTENTION_ASYNC = on != 0; }

// How the `rows` rows of a prompt tile's block (32: the CUDA-core kernel; 64: the tensor-core kernel) are cut
// into tokens and heads for `heads_per_group` query heads a key/value head: heads a block (at most `rows`) and
// tokens a block (a power of two, at most `rows`).
RL_EXPORT int rl_bias_attention_shape(int heads_per_group, int rows, int* heads_per_block, int* tokens_per_block) {
  if (heads_per_group <= 0 || (rows != rl::BA_ROWS && rows != rl::BM_ROWS)) return -2;
  const int hb = heads_per_group < rows ? heads_per_group : rows;
  int tt = 1;
  while (tt * 2 * hb <= rows) tt *= 2;
  *heads_per_block = hb;
  *tokens_per_block = tt;
  return 0;
}

// n_splits > 1: every decoded request's keys are cut into so many parts, a block each, merged by a second
// kernel; part_o float32 [n_decode * heads * n_splits, dv], part_ml float32 [n_decode * heads * n_splits, 2].
// tensor_cores: prompt tiles go to `bias_attn_mma_kernel` where the types and sizes allow (64 rows a block: the
// tiles must then be cut as rl_bias_attention_shape(.., 64, ..) says).
// sink: float32 [heads] or null; gate_per_head: the gate's rows hold one logit a head, not one a value column.
// tiles: (request, first new token) of portions cut every `tile_tokens` tokens (a multiple of the tokens a
// block takes); decode_reqs: the requests that bring one token.  cache_dtype: the pool's element type;
// out_dtype: that of out.
RL_EXPORT int rl_bias_attention(int cache_dtype, int out_dtype, const float* q, long ldq, const float* gate, long ldg,
                                const void* pool, const int* block_table, long ldt, const int* q_start,
                                const int* kv_len, const int* slots, const int* tiles, int n_tiles, int tile_tokens,
                                const int* decode_reqs, int n_decode, void* out, long ldo, int n_heads, int n_kv, int dk,
                                int dv, int v_at, int row, int page_size, int max_pages, float scale, float temp_coef,
                                int temp_every, const float* slopes, int* status, int n_splits, float* part_o,
                                float* part_ml, int tensor_cores, int window, const float* head_scale,
                                const float* sink, int gate_per_head, cudaStream_t stream) {
  if (n_tiles <= 0 && n_decode <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dk <= 0 || dk > 256 || dv <= 0 || dv > 256 || v_at < dk ||
      v_at + dv > row || n_kv > 65535 || window < 0)
    return -2;
  // prompt tiles on the tensor cores: bfloat16 cache and output, per-head sizes up to 128
  const bool mma = tensor_cores && cache_dtype == RL_BF16 && out_dtype == RL_BF16 && dk <= 128 && dv <= 128;
  int hb, tt;
  rl_bias_attention_shape(n_heads / n_kv, mma ? rl::BM_ROWS : rl::BA_ROWS, &hb, &tt);
  if (n_tiles > 0 && (tile_tokens < tt || tile_tokens % tt)) return -3;
  if (n_tiles <= 0) tile_tokens = tt;
  if (n_splits < 1 || n_splits > 32 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr))) return -4;
  if (n_decode <= 0) n_splits = 1;
  const int hg = n_heads / n_kv;
  rl::BiasAttnParams p{q, ldq, gate, ldg, pool, block_table, ldt, q_start, kv_len, slots, tiles, decode_reqs, out, ldo,
                       n_heads, n_kv, dk, dv, v_at, row, page_size, max_pages, n_tiles > 0 ? n_tiles : 0, tile_tokens,
                       tt, hb, 0, scale, temp_coef, temp_every, slopes, status, window, head_scale, 1, part_o, part_ml,
                       sink, gate_per_head != 0};
  if (p.n_tiles > 0) {  // the prompt portions: 32 or 64 rows a block, cut into tokens and heads as rl_bias_attention_shape says
    const dim3 grid(p.n_tiles * (tile_tokens / tt), n_kv, (hg + hb - 1) / hb);
    if (mma) rl::dispatch_bias_attn_mma(p, grid, stream);
    else rl::dispatch_bias_attn_types(cache_dtype, out_dtype, p, 32, grid, stream);
  }
  if (n_decode > 0) {  // the decoded tokens: a block's rows are heads of one group, 4, 8 or 32 of them
    const int rows = hg <= 4 ? 4 : (hg <= 8 ? 8 : 32);
    p.n_tiles = 0;
    p.n_decode = n_decode;
    p.n_splits = n_splits;
    p.tokens_per_block = p.tile_tokens = 1;
    p.heads_per_block = hg < rows ? hg : rows;
    rl::dispatch_bias_attn_types(cache_dtype, out_dtype, p, rows,
                                 dim3(n_decode * n_splits, n_kv, (hg + p.heads_per_block - 1) / p.heads_per_block), stream);
  }
  if (n_splits > 1) {
    const dim3 mg(p.n_decode, (n_heads + 3) / 4);
    if (out_dtype == RL_F32) rl::launch_pdl(rl::bias_attn_merge_kernel<float>, mg, 128, 0, stream, p);
    else rl::launch_pdl(rl::bias_attn_merge_kernel<__nv_bfloat16>, mg, 128, 0, stream, p);
  }
  RL_CHECK_LAUNCH();
  return 0;
}

// The step's keys and values (float32 columns of the packed projections) into their pages; see the kernel.
RL_EXPORT int rl_bias_kv_store(int cache_dtype, const float* k, long ldk, const float* v, long ldv, float* v_src,
                               const float* lambda, int mix, void* pool, const int* block_table, long ldt,
                               const int* positions, const int* req_of_token, const int* slots, int n_tokens, int n_kv,
                               int dk, int dv, int v_at, int row, int page_size, int max_pages, int* status,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (mix < 0 || mix > 2 || (mix != 0 && v_src == nullptr) || (mix == 2 && lambda == nullptr) || v_at < dk ||
      v_at + dv > row)
    return -2;
  if (cache_dtype == RL_F32)
    rl::launch_pdl(rl::bias_kv_store_kernel<float>, n_tokens, 128, 0, stream, k, ldk, v, ldv, v_src, lambda, mix,
                   (float*)pool, block_table, ldt, positions, req_of_token, slots, n_tokens, n_kv, dk, dv, v_at, row,
                   page_size, max_pages, status);
  else
    rl::launch_pdl(rl::bias_kv_store_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, k, ldk, v, ldv, v_src, lambda,
                   mix, (__nv_bfloat16*)pool, block_table, ldt, positions, req_of_token, slots, n_tokens, n_kv, dk, dv,
                   v_at, row, page_size, max_pages, status);
  RL_CHECK_LAUNCH();
  return 0;
}

namespace rl {

// What a layer does to its queries, keys and values between the projections and the cache, in place on the
// float32 columns of the packed projections, a warp a (token, head); a token's heads are spread over the blocks
// of grid row y, so that a step of few tokens is as many short chains side by side, not one long one:
//   queries and keys: each head's entries divided by their root mean square (eps inside the root) and
//     multiplied by a weight the heads share (q_norm / k_norm; absent: left as they are, or with `unit_qk`
//     divided by the root mean square and no weight), then the first
//     `rot_dims` entries turned, entry 2i with entry 2i + 1, by the angle position * freq[i];
//   values: each head's entries divided by their root mean square, no weight (unit_values; else untouched).
// Angles are formed and evaluated in float32.  With a cache target the keys and values go into their pages on the
// way (as `bias_kv_store_kernel` would put them) and are not written back.
// Where the keys and values of a step go when this kernel also writes the cache (fused: the store kernel's work
// rides on the pass that normalises and rotates; keys and values are then NOT written back in place).
struct QkvCacheTarget {
  void* pool;  // [pages, 1, n_kv, page_size, row], or null: no store
  const int* block_table;
  long ldt;
  const int *req_of_token, *slots;
  int v_at, row, page_size, max_pages;
  int* status;
};

template <typename T>
__global__ __launch_bounds__(128) void qkv_norm_rotate_kernel(float* __restrict__ q, long ldq, float* __restrict__ k,
                                                              long ldk, float* __restrict__ v, long ldv,
                                                              const float* __restrict__ q_norm,
                                                              const float* __restrict__ k_norm,
                                                              const float* __restrict__ freq,
                                                              const int* __restrict__ positions, int n_tokens,
                                                              int n_heads, int n_kv, int dk, int dv, int rot_dims,
                                                              int unit_values, int unit_qk, float eps,
                                                              const QkvCacheTarget c) {
  pdl_begin();
  const int tok = blockIdx.x;
  if (tok >= n_tokens) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int ipos = positions[tok];
  const float pos = (float)ipos;
  const bool store = c.pool != nullptr;
  const int units = n_heads + n_kv + ((unit_values || store) ? n_kv : 0);
  // the token's place in the cache: a row of its page a key/value head (null: a padding row, or no page)
  T* cache_row = nullptr;
  long head_step = 0;
  if (store) {
    const int slot = c.slots[c.req_of_token[tok]];
    if (slot >= 0) {
      const int lp = ipos / c.page_size;
      const int page = (ipos >= 0 && lp < c.max_pages) ? c.block_table[(size_t)slot * c.ldt + lp] : -1;
      if (page < 0) {
        if (threadIdx.x == 0 && blockIdx.y == 0)
          atomicOr(c.status, ipos < 0 || lp >= c.max_pages ? RL_STATUS_BAD_POSITION : RL_STATUS_BAD_PAGE);
      } else {
        head_step = (long)c.page_size * c.row;
        cache_row = reinterpret_cast<T*>(c.pool) + ((size_t)page * n_kv * c.page_size + (ipos - lp * c.page_size)) * c.row;
      }
    }
  }
  // the token's angles are the same for all its heads: their sines and cosines once a block
  __shared__ float2 turn[128];
  for (int i = threadIdx.x; 2 * i < rot_dims; i += blockDim.x) sincosf(pos * freq[i], &turn[i].y, &turn[i].x);
  __syncthreads();
  for (int u = blockIdx.y * n_warps + warp; u < units; u += n_warps * gridDim.y) {
    if (u < n_heads + n_kv) {
      const bool is_q = u < n_heads;
      float* e = is_q ? q + (size_t)tok * ldq + (size_t)u * dk : k + (size_t)tok * ldk + (size_t)(u - n_heads) * dk;
      const float* w = is_q ? q_norm : k_norm;
      T* to_cache = (!is_q && cache_row != nullptr) ? cache_row + (size_t)(u - n_heads) * head_step : nullptr;
      const bool in_place = is_q || !store;
      float r = 1.0f;
      if (w != nullptr || unit_qk) {
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(e[d], e[d], ss);
        r = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
      }
      for (int i = lane; 2 * i < dk; i += 32) {  // a lane takes whole pairs; an odd last entry has no partner
        const int d0 = 2 * i, d1 = 2 * i + 1;
        float a = e[d0] * r, b = d1 < dk ? e[d1] * r : 0.f;
        if (w != nullptr) {
          a *= w[d0];
          if (d1 < dk) b *= w[d1];
        }
        if (d1 < rot_dims) {
          const float cs = turn[i].x, sn = turn[i].y;
          const float ra = a * cs - b * sn, rb = b * cs + a * sn;
          a = ra;
          b = rb;
        }
        if (in_place) {
          e[d0] = a;
          if (d1 < dk) e[d1] = b;
        }
        if (to_cache != nullptr) {
          to_cache[d0] = from_f32<T>(a);
          if (d1 < dk) to_cache[d1] = from_f32<T>(b);
        }
      }
    } else {
      const int g = u - n_heads - n_kv;
      float* e = v + (size_t)tok * ldv + (size_t)g * dv;
      float r = 1.0f;
      if (unit_values) {
        float ss = 0.f;
        for (int d = lane; d < dv; d += 32) ss = fmaf(e[d], e[d], ss);
        r = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
      }
      if (!store) {
        for (int d = lane; d < dv; d += 32) e[d] *= r;
      } else if (cache_row != nullptr) {
        T* to_cache = cache_row + (size_t)g * head_step + c.v_at;
        for (int d = lane; d < dv; d += 32) to_cache[d] = from_f32<T>(e[d] * r);
      }
    }
  }
}

}  // namespace rl

// Queries [tokens, heads * dk], keys [tokens, kv heads * dk] and values [tokens, kv heads * dv] (float32, row
// strides given) normalised and rotated in place; see the kernel.  q_norm / k_norm: float32 [dk] or null (both
// or neither; unit_qk: without weights, queries and keys are still divided by their root mean square);
// freq: float32 [rot_dims / 2] (rot_dims even, at most dk; 0: no rotation).
// pool (or null): the cache [pages, 1, n_kv, page_size, row] of element type cache_dtype: keys and values go to
// their pages (the value at entry v_at of a row) instead of back in place, as rl_bias_kv_store would put them.
RL_EXPORT int rl_qkv_norm_rotate(float* q, long ldq, float* k, long ldk, float* v, long ldv, const float* q_norm,
                                 const float* k_norm, const float* freq, const int* positions, int n_tokens, int n_heads,
                                 int n_kv, int dk, int dv, int rot_dims, int unit_values, int unit_qk, float eps,
                                 int cache_dtype, void* pool, const int* block_table, long ldt, const int* req_of_token,
                                 const int* slots, int v_at, int row, int page_size, int max_pages, int* status,
                                 cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || dk <= 0 || dv <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > dk ||
      rot_dims > 256 || (rot_dims > 0 && freq == nullptr) || (q_norm == nullptr) != (k_norm == nullptr))
    return -2;
  if (pool != nullptr && (block_table == nullptr || req_of_token == nullptr || slots == nullptr || status == nullptr ||
                          v_at < dk || v_at + dv > row || page_size <= 0))
    return -2;
  const int units = n_heads + n_kv + ((unit_values || pool != nullptr) ? n_kv : 0);
  // a warp a (token, head) in a step of few tokens; with many tokens a block takes more of a token's heads
  const int want = (148 * 40 + n_tokens - 1) / n_tokens, most = units < 4 * 1024 ? (units + 3) / 4 : 1024;
  const int rows = want < most ? want : most;
  const rl::QkvCacheTarget c{pool, block_table, ldt, req_of_token, slots, v_at, row, page_size, max_pages, status};
  if (pool != nullptr && cache_dtype == RL_F32)
    rl::launch_pdl(rl::qkv_norm_rotate_kernel<float>, dim3(n_tokens, rows), 128, 0, stream, q, ldq, k, ldk, v, ldv, q_norm,
                   k_norm, freq, positions, n_tokens, n_heads, n_kv, dk, dv, rot_dims, unit_values, unit_qk, eps, c);
  else
    rl::launch_pdl(rl::qkv_norm_rotate_kernel<__nv_bfloat16>, dim3(n_tokens, rows), 128, 0, stream, q, ldq, k, ldk, v, ldv,
                   q_norm, k_norm, freq, positions, n_tokens, n_heads, n_kv, dk, dv, rot_dims, unit_values, unit_qk, eps, c);
  RL_CHECK_LAUNCH();
  return 0;
}
