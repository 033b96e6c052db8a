// Prompt portions of the distance-biased attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands,
// float32 accumulation), for the 16-bit mode: the same rows ((token, head) pairs of one key/value head), the
// same scores, bias, temperature, softmax and gate as `bias_attn_kernel`, which remains the kernel of the
// 32-bit mode, of decoded tokens and of per-head sizes above 128.
//
// A block of four warps takes 64 rows, a warp 16 of them, and walks the keys 64 at a time.  Queries (rounded
// to bfloat16) and the key tile lie in shared memory row by row, so that both operand fragments of S = Q K^T
// are 32-bit loads; the value tile is stored transposed (column by column) for the same reason in P V.  The
// scores stay in the accumulator registers through bias, mask and online softmax (float32) and become the
// A fragments of the second product without leaving the thread.
#pragma once
#include <math_constants.h>

#include "common.cuh"

namespace rl {

constexpr int BM_ROWS = 64, BM_KEYS = 64, BM_THREADS = 128, BM_PAD = 8;
// Switch (for comparisons): off, every size takes the form that copies key tiles through registers.
static bool BIAS_ATTENTION_ASYNC = true;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// DKT: 16-entry steps of the key size (dk <= 16 DKT); DVT: 8-column tiles of the value size (dv <= 8 DVT).
template <int DKT, int DVT>
__global__ __launch_bounds__(BM_THREADS) void bias_attn_mma_kernel(const BiasAttnParams p) {
  extern __shared__ __align__(16) unsigned char bm_s[];
  pdl_begin();
  constexpr int DKP = 16 * DKT, DVP = 8 * DVT;
  constexpr int LDQ = DKP + BM_PAD, LDV = BM_KEYS + BM_PAD;  // row strides in elements (multiples of 8: 16-byte rows)
  const int subs = p.tile_tokens / p.tokens_per_block;
  const int tile = blockIdx.x / subs, sub = blockIdx.x - tile * subs;
  const int req = p.tiles[2 * tile];
  const int first = p.tiles[2 * tile + 1] + sub * p.tokens_per_block;
  const int slot = p.slots[req];
  const int t_begin = p.q_start[req], n_new = p.q_start[req + 1] - t_begin;
  if (slot < 0 || first >= n_new) return;
  const int n_tok = min(p.tokens_per_block, n_new - first);
  const int pos0 = p.kv_len[req] - n_new + first;
  const int g = blockIdx.y, hg = p.n_heads / p.n_kv;
  const int HB = p.heads_per_block, hb0 = blockIdx.z * HB;
  const int dk = p.dk, dv = p.dv;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(bm_s);  // [BM_ROWS][LDQ]
  __nv_bfloat16* Ks = Qs + BM_ROWS * LDQ;                       // [BM_KEYS][LDQ]
  __nv_bfloat16* Vt = Ks + BM_KEYS * LDQ;                       // [DVP][LDV]: column by column
  __shared__ const __nv_bfloat16* key_src[2][BM_KEYS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = lane >> 2, in_quad = lane & 3;
  // queries, rounded to bfloat16; rows beyond the block's tokens and entries beyond dk are zero
  for (int i = tid; i < BM_ROWS * DKP; i += BM_THREADS) {
    const int r = i / DKP, d = i - r * DKP;
    const int tl = r / HB, hl = r - tl * HB;
    float v = 0.f;
    if (tl < n_tok && hb0 + hl < hg && d < dk)
      v = p.q[(size_t)(t_begin + first + tl) * p.ldq + (size_t)(g * hg + hb0 + hl) * dk + d];
    Qs[r * LDQ + d] = __float2bfloat16_rn(v);
  }
  for (int i = tid; i < BM_KEYS * LDQ; i += BM_THREADS) Ks[i] = __float2bfloat16_rn(0.f);
  for (int i = tid; i < DVP * LDV; i += BM_THREADS) Vt[i] = __float2bfloat16_rn(0.f);
  int row_pos[2], row_head[2];
  float row_mul[2], row_slope[2], m[2], l[2];
  bool row_ok[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = warp * 16 + quad + 8 * a, tl = r / HB, hl = r - tl * HB;
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
  }
  float o[DVT][4];
#pragma unroll
  for (int nt = 0; nt < DVT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  const int last_pos = pos0 + n_tok - 1;
  const int first_seen = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;  // the earliest key any row of the block sees
  const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(p.pool);
  const int* table = p.block_table + (size_t)slot * p.ldt;
  auto locate = [&](int j0, int buf) {
    if (tid < BM_KEYS) {
      const int j = j0 + tid;
      const __nv_bfloat16* src = nullptr;
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
  const bool vec = dk % 8 == 0 && dv % 8 == 0 && (reinterpret_cast<uintptr_t>(p.pool) & 15) == 0;
  const int j_begin = first_seen / BM_KEYS * BM_KEYS;
  locate(j_begin, 0);
  int buf = 0;
  const uint32_t* Qw = reinterpret_cast<const uint32_t*>(Qs);
  const uint32_t* Kw = reinterpret_cast<const uint32_t*>(Ks);
  const uint32_t* Vw = reinterpret_cast<const uint32_t*>(Vt);
  for (int j0 = j_begin; j0 <= last_pos; j0 += BM_KEYS, buf ^= 1) {
    __syncthreads();  // the tile before has been used; this tile's places (and, the first time, the queries) are known
    if (vec) {
      const int kp = dk / 8, vp = dv / 8, per_key = kp + vp;
#pragma unroll 4
      for (int i = tid; i < BM_KEYS * per_key; i += BM_THREADS) {
        const int jj = i / per_key, piece = i - jj * per_key;
        const __nv_bfloat16* src = key_src[buf][jj];
        const bool is_v = piece >= kp;
        const int at = is_v ? (piece - kp) * 8 : piece * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (src != nullptr) raw = *reinterpret_cast<const uint4*>(src + (is_v ? p.v_at : 0) + at);
        if (!is_v) {
          *reinterpret_cast<uint4*>(Ks + jj * LDQ + at) = raw;
        } else {
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
          for (int x = 0; x < 8; ++x) Vt[(at + x) * LDV + jj] = e[x];
        }
      }
    } else {
      const int per_key = dk + dv;
#pragma unroll 4
      for (int i = tid; i < BM_KEYS * per_key; i += BM_THREADS) {
        const int jj = i / per_key, c = i - jj * per_key;
        const __nv_bfloat16* src = key_src[buf][jj];
        const bool is_v = c >= dk;
        const __nv_bfloat16 val = src != nullptr ? src[is_v ? p.v_at + c - dk : c] : __float2bfloat16_rn(0.f);
        if (is_v) Vt[(c - dk) * LDV + jj] = val;
        else Ks[jj * LDQ + c] = val;
      }
    }
    locate(j0 + BM_KEYS, buf ^ 1);
    __syncthreads();
    // S = Q K^T: 16 rows x 64 keys a warp
    float s[BM_KEYS / 8][4];
#pragma unroll
    for (int nt = 0; nt < BM_KEYS / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int kc = 0; kc < DKT; ++kc) {
      uint32_t a[4];
      const int qrow = warp * 16 + quad, qw = kc * 8 + in_quad;  // in 32-bit words
      a[0] = Qw[qrow * (LDQ / 2) + qw];
      a[1] = Qw[(qrow + 8) * (LDQ / 2) + qw];
      a[2] = Qw[qrow * (LDQ / 2) + qw + 4];
      a[3] = Qw[(qrow + 8) * (LDQ / 2) + qw + 4];
#pragma unroll
      for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
        const int key = nt * 8 + quad;
        mma_bf16_16816(s[nt], a, Kw[key * (LDQ / 2) + qw], Kw[key * (LDQ / 2) + qw + 4]);
      }
    }
    // bias, mask and online softmax in float32 on the accumulators: a thread holds, of rows quad and quad + 8,
    // the keys 8 nt + 2 in_quad + {0, 1}
    uint32_t pa[BM_KEYS / 16][4];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      float tile_max = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j0 + nt * 8 + 2 * in_quad + e;
          float& v = s[nt][2 * a + e];
          const bool see = row_ok[a] && j <= row_pos[a] && (p.window <= 0 || row_pos[a] - j < p.window);
          v = see ? v * row_mul[a] - row_slope[a] * (float)(row_pos[a] - j) : -CUDART_INF_F;
          tile_max = fmaxf(tile_max, v);
        }
      }
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float m_new = fmaxf(m[a], tile_max);
      const float corr = m[a] == -CUDART_INF_F ? 0.f : expf(m[a] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float& v = s[nt][2 * a + e];
          v = v == -CUDART_INF_F ? 0.f : expf(v - m_new);
          sum += v;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[a] = l[a] * corr + sum;
      m[a] = m_new;
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        o[nt][2 * a] *= corr;
        o[nt][2 * a + 1] *= corr;
      }
    }
    // the probabilities as A fragments: keys 16 kc .. 16 kc + 15 are the score tiles 2 kc and 2 kc + 1
#pragma unroll
    for (int kc = 0; kc < BM_KEYS / 16; ++kc) {
      pa[kc][0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
      pa[kc][1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
      pa[kc][2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
      pa[kc][3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
    }
#pragma unroll
    for (int kc = 0; kc < BM_KEYS / 16; ++kc) {
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        const int colw = (nt * 8 + quad) * (LDV / 2) + kc * 8 + in_quad;
        mma_bf16_16816(o[nt], pa[kc], Vw[colw], Vw[colw + 4]);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (!row_ok[a]) continue;
    const int r = warp * 16 + quad + 8 * a;
    const int tok = t_begin + first + r / HB;
    const float inv = 1.0f / (l[a] + (p.sink != nullptr ? expf(p.sink[row_head[a]] - m[a]) : 0.f));
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + (size_t)row_head[a] * dv;
    int gs;
    const float* gr = bias_gate_row(p, tok, row_head[a], gs);
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = nt * 8 + 2 * in_quad + e;
        if (col < dv) {
          float v = o[nt][2 * a + e] * inv;
          if (gr != nullptr) v *= 1.0f / (1.0f + expf(-gr[col * gs]));
          out[col] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

// The same kernel for sizes whose cache rows can be copied in 16-byte pieces (dk, dv, the value's place and the
// row multiples of 8, the pool on a 16-byte boundary): the key and value tiles travel by cp.async into a ring of two
// stages, the next tile's copies in flight under this tile's two products; values lie row by row as in the cache
// and their fragments are fetched transposed (ldmatrix.trans); only the lookups of page addresses, two tiles ahead,
// are ordinary loads.
__device__ __forceinline__ void bm_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
constexpr float BM_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float bm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void bm_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void bm_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <int DKT, int DVT>
__global__ __launch_bounds__(BM_THREADS, (DVT <= 8 ? 4 : 3)) void bias_attn_mma_async_kernel(const BiasAttnParams p) {
  extern __shared__ __align__(16) unsigned char bm_s[];
  pdl_begin();
  constexpr int DKP = 16 * DKT, DVP = 8 * DVT;
  constexpr int LDQ = DKP + BM_PAD, LDW = DVP + BM_PAD;  // row strides in elements (multiples of 8: 16-byte rows)
  const int subs = p.tile_tokens / p.tokens_per_block;
  // a portion's last tiles walk the most keys: taken first, they do not run alone at the end
  const int bx = gridDim.x - 1 - blockIdx.x;
  const int tile = bx / subs, sub = bx - tile * subs;
  const int req = p.tiles[2 * tile];
  const int first = p.tiles[2 * tile + 1] + sub * p.tokens_per_block;
  const int slot = p.slots[req];
  const int t_begin = p.q_start[req], n_new = p.q_start[req + 1] - t_begin;
  if (slot < 0 || first >= n_new) return;
  const int n_tok = min(p.tokens_per_block, n_new - first);
  const int pos0 = p.kv_len[req] - n_new + first;
  const int g = blockIdx.y, hg = p.n_heads / p.n_kv;
  const int HB = p.heads_per_block, hb0 = blockIdx.z * HB;
  const int dk = p.dk, dv = p.dv;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(bm_s);  // [BM_ROWS][LDQ]
  __nv_bfloat16* Kr = Qs + BM_ROWS * LDQ;                       // [2][BM_KEYS][LDQ]
  __nv_bfloat16* Vr = Kr + 2 * BM_KEYS * LDQ;                   // [2][BM_KEYS][LDW]: row by row
  __shared__ const __nv_bfloat16* key_src[2][BM_KEYS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = lane >> 2, in_quad = lane & 3;
  for (int i = tid; i < BM_ROWS * DKP; i += BM_THREADS) {
    const int r = i / DKP, d = i - r * DKP;
    const int tl = r / HB, hl = r - tl * HB;
    float v = 0.f;
    if (tl < n_tok && hb0 + hl < hg && d < dk)
      v = p.q[(size_t)(t_begin + first + tl) * p.ldq + (size_t)(g * hg + hb0 + hl) * dk + d];
    Qs[r * LDQ + d] = __float2bfloat16_rn(v);
  }
  // entries beyond dk and dv are never copied: they stay zero
  for (int i = tid; i < 2 * BM_KEYS * LDQ; i += BM_THREADS) Kr[i] = __float2bfloat16_rn(0.f);
  for (int i = tid; i < 2 * BM_KEYS * LDW; i += BM_THREADS) Vr[i] = __float2bfloat16_rn(0.f);
  int row_pos[2], row_head[2];
  float row_mul[2], row_slope[2], m[2], l[2];
  bool row_ok[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = warp * 16 + quad + 8 * a, tl = r / HB, hl = r - tl * HB;
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
  }
  float o[DVT][4];
#pragma unroll
  for (int nt = 0; nt < DVT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  const int last_pos = pos0 + n_tok - 1;
  const int first_seen = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(p.pool);
  const int* table = p.block_table + (size_t)slot * p.ldt;
  auto locate = [&](int j0, int buf) {
    if (tid < BM_KEYS) {
      const int j = j0 + tid;
      const __nv_bfloat16* src = nullptr;
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
  const int kp = dk / 8, vp = dv / 8, per_key = kp + vp;
  // the copies of one tile into stage `st`, from the places in key_src[st]; keys nobody sees get zeros
  auto fetch = [&](int st) {
    __nv_bfloat16* kd = Kr + st * BM_KEYS * LDQ;
    __nv_bfloat16* vd = Vr + st * BM_KEYS * LDW;
    for (int i = tid; i < BM_KEYS * per_key; i += BM_THREADS) {
      const int jj = i / per_key, piece = i - jj * per_key;
      const __nv_bfloat16* src = key_src[st][jj];
      const bool is_v = piece >= kp;
      const int at = is_v ? (piece - kp) * 8 : piece * 8;
      __nv_bfloat16* dst = is_v ? vd + jj * LDW + at : kd + jj * LDQ + at;
      if (src != nullptr) bm_cp_async16((uint32_t)__cvta_generic_to_shared(dst), src + (is_v ? p.v_at : 0) + at);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int j_begin = first_seen / BM_KEYS * BM_KEYS;
  // tile t uses stage t & 1 and the places in key_src[t & 1]; the places are looked up two tiles ahead
  locate(j_begin, 0);
  __syncthreads();  // the zero fill is done, the first tile's places are known
  fetch(0);
  locate(j_begin + BM_KEYS, 1);
  __syncthreads();  // every thread has read the first tile's places
  locate(j_begin + 2 * BM_KEYS, 0);
  // the queries' fragments do not change from tile to tile: in registers once, where the key size leaves room
  constexpr bool Q_IN_REGS = DKT <= 4;
  const uint32_t* Qw = reinterpret_cast<const uint32_t*>(Qs);
  uint32_t qa[Q_IN_REGS ? DKT : 1][4];
  if (Q_IN_REGS) {
#pragma unroll
    for (int kc = 0; kc < DKT; ++kc) {
      const int qrow = warp * 16 + quad, qw = kc * 8 + in_quad;  // in 32-bit words
      qa[kc][0] = Qw[qrow * (LDQ / 2) + qw];
      qa[kc][1] = Qw[(qrow + 8) * (LDQ / 2) + qw];
      qa[kc][2] = Qw[qrow * (LDQ / 2) + qw + 4];
      qa[kc][3] = Qw[(qrow + 8) * (LDQ / 2) + qw + 4];
    }
  }
  int st = 0;
  for (int j0 = j_begin; j0 <= last_pos; j0 += BM_KEYS, st ^= 1) {
    __syncthreads();  // the tile before has been used: its stage is free; the next tile's places are known
    const bool more = j0 + BM_KEYS <= last_pos;
    if (more) {
      fetch(st ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();  // this tile has arrived for every thread; the next tile's places have been read
    if (more) locate(j0 + 3 * BM_KEYS, st ^ 1);
    const __nv_bfloat16* Ks = Kr + st * BM_KEYS * LDQ;
    const __nv_bfloat16* Vs = Vr + st * BM_KEYS * LDW;
    float s[BM_KEYS / 8][4];
#pragma unroll
    for (int nt = 0; nt < BM_KEYS / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    // S = Q K^T: the key fragments of keys 8 nt .. + 15 and entries 16 kc .. + 15 in one load: lanes 0-7 name the
    // rows of keys 8 nt .. + 7 (entries 0-7), lanes 8-15 the same keys (entries 8-15), lanes 16-31 the next 8 keys
#pragma unroll
    for (int kc = 0; kc < DKT; ++kc) {
      uint32_t a[4];
      if (Q_IN_REGS) {
        a[0] = qa[kc][0], a[1] = qa[kc][1], a[2] = qa[kc][2], a[3] = qa[kc][3];
      } else {
        const int qrow = warp * 16 + quad, qw = kc * 8 + in_quad;  // in 32-bit words
        a[0] = Qw[qrow * (LDQ / 2) + qw];
        a[1] = Qw[(qrow + 8) * (LDQ / 2) + qw];
        a[2] = Qw[qrow * (LDQ / 2) + qw + 4];
        a[3] = Qw[(qrow + 8) * (LDQ / 2) + qw + 4];
      }
#pragma unroll
      for (int nt = 0; nt < BM_KEYS / 8; nt += 2) {
        uint32_t kf[4];
        const int key = (nt + (lane >> 4)) * 8 + (lane & 7);
        bm_ldmatrix_x4(kf, (uint32_t)__cvta_generic_to_shared(Ks + key * LDQ + kc * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16_16816(s[nt], a, kf[0], kf[1]);
        mma_bf16_16816(s[nt + 1], a, kf[2], kf[3]);
      }
    }
    uint32_t pa[BM_KEYS / 16][4];
    // a tile that every row of the block sees whole (all of it at or before the block's first position and
    // inside the last row's window) needs no mask
    const bool whole = j0 + BM_KEYS - 1 <= pos0 && (p.window <= 0 || last_pos - j0 < p.window);
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      float tile_max = -CUDART_INF_F;
      if (whole && p.slopes == nullptr) {
#pragma unroll
        for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float& v = s[nt][2 * a + e];
            v *= row_mul[a];
            tile_max = fmaxf(tile_max, v);
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = j0 + nt * 8 + 2 * in_quad + e;
            float& v = s[nt][2 * a + e];
            const bool see = row_ok[a] && j <= row_pos[a] && (p.window <= 0 || row_pos[a] - j < p.window);
            v = see ? v * row_mul[a] - row_slope[a] * (float)(row_pos[a] - j) : -CUDART_INF_F;
            tile_max = fmaxf(tile_max, v);
          }
        }
      }
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float m_new = fmaxf(m[a], tile_max);
      const float corr = m[a] == -CUDART_INF_F ? 0.f : expf(m[a] - m_new);
      // e^(v - m) as 2^(v log2 e - m log2 e): one multiply-add and the hardware's 2^x (two units in the last place
      // of a float32, far below what the rounding of the probabilities to bfloat16 leaves; 2^-inf is 0)
      const float mb = m_new == -CUDART_INF_F ? 0.f : m_new * BM_LOG2E;
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < BM_KEYS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float& v = s[nt][2 * a + e];
          v = bm_ex2(fmaf(v, BM_LOG2E, -mb));
          sum += v;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[a] = l[a] * corr + sum;
      m[a] = m_new;
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        o[nt][2 * a] *= corr;
        o[nt][2 * a + 1] *= corr;
      }
    }
#pragma unroll
    for (int kc = 0; kc < BM_KEYS / 16; ++kc) {
      pa[kc][0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
      pa[kc][1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
      pa[kc][2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
      pa[kc][3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
    }
    // P V: the value fragments of keys 16 kc .. + 15 and columns 16 n2 .. + 15 in one transposed load: lanes 0-7
    // name the rows of keys 0-7, lanes 8-15 of keys 8-15 (both of the first eight columns), lanes 16-31 the same
    // keys of the next eight columns
#pragma unroll
    for (int kc = 0; kc < BM_KEYS / 16; ++kc) {
      const int key = kc * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int n2 = 0; n2 < DVT / 2; ++n2) {
        uint32_t vf[4];
        bm_ldmatrix_x4_trans(vf, (uint32_t)__cvta_generic_to_shared(Vs + key * LDW + n2 * 16 + (lane >> 4) * 8));
        mma_bf16_16816(o[2 * n2], pa[kc], vf[0], vf[1]);
        mma_bf16_16816(o[2 * n2 + 1], pa[kc], vf[2], vf[3]);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (!row_ok[a]) continue;
    const int r = warp * 16 + quad + 8 * a;
    const int tok = t_begin + first + r / HB;
    const float inv = 1.0f / (l[a] + (p.sink != nullptr ? expf(p.sink[row_head[a]] - m[a]) : 0.f));
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tok * p.ldo + (size_t)row_head[a] * dv;
    int gs;
    const float* gr = bias_gate_row(p, tok, row_head[a], gs);
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = nt * 8 + 2 * in_quad + e;
        if (col < dv) {
          float v = o[nt][2 * a + e] * inv;
          if (gr != nullptr) v *= 1.0f / (1.0f + expf(-gr[col * gs]));
          out[col] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

template <int DKT, int DVT>
static void launch_bias_attn_mma(const BiasAttnParams& p, dim3 grid, cudaStream_t stream) {
  // cache rows in 16-byte pieces: the form whose tiles travel by cp.async (all of an SM's memory as shared memory,
  // so that as many of its larger blocks fit as registers allow)
  if (BIAS_ATTENTION_ASYNC && p.dk % 8 == 0 && p.dv % 8 == 0 && p.v_at % 8 == 0 && p.row % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(p.pool) & 15) == 0) {
    constexpr int LDQA = 16 * DKT + BM_PAD, LDWA = 8 * DVT + BM_PAD;
    const size_t smem_a = ((size_t)BM_ROWS * LDQA + (size_t)2 * BM_KEYS * LDQA + (size_t)2 * BM_KEYS * LDWA) * sizeof(__nv_bfloat16);
    auto kernel_a = bias_attn_mma_async_kernel<DKT, DVT>;
    static bool raised_a = false;
    if (!raised_a) {
      note_launch(cudaFuncSetAttribute(kernel_a, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      note_launch(cudaFuncSetAttribute(kernel_a, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       (int)cudaSharedmemCarveoutMaxShared));
      raised_a = true;
    }
    launch_pdl_split(false, kernel_a, grid, BM_THREADS, smem_a, stream, p);
    return;
  }
  constexpr int LDQ = 16 * DKT + BM_PAD, LDV = BM_KEYS + BM_PAD;
  const size_t smem = ((size_t)BM_ROWS * LDQ + (size_t)BM_KEYS * LDQ + (size_t)8 * DVT * LDV) * sizeof(__nv_bfloat16);
  auto kernel = bias_attn_mma_kernel<DKT, DVT>;
  if (smem > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      note_launch(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
      raised = true;
    }
  }
  launch_pdl(kernel, grid, BM_THREADS, smem, stream, p);
}

// dk, dv <= 128
static void dispatch_bias_attn_mma(const BiasAttnParams& p, dim3 grid, cudaStream_t stream) {
  const int kt = p.dk <= 32 ? 0 : (p.dk <= 64 ? 1 : 2), vt = p.dv <= 32 ? 0 : (p.dv <= 64 ? 1 : 2);
  switch (kt * 3 + vt) {
    case 0: launch_bias_attn_mma<2, 4>(p, grid, stream); break;
    case 1: launch_bias_attn_mma<2, 8>(p, grid, stream); break;
    case 2: launch_bias_attn_mma<2, 16>(p, grid, stream); break;
    case 3: launch_bias_attn_mma<4, 4>(p, grid, stream); break;
    case 4: launch_bias_attn_mma<4, 8>(p, grid, stream); break;
    case 5: launch_bias_attn_mma<4, 16>(p, grid, stream); break;
    case 6: launch_bias_attn_mma<8, 4>(p, grid, stream); break;
    case 7: launch_bias_attn_mma<8, 8>(p, grid, stream); break;
    default: launch_bias_attn_mma<8, 16>(p, grid, stream); break;
  }
}

}  // namespace rl
