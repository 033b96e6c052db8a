// Mixers with a matrix-valued state per request and head: S_t = diag(w_t) S_(t-1) [- (a_t * u_t)(u_t^T S_(t-1))]
// + k_t v_t^T, o_t = S_t^T r_t, the state [dk, dv] in float32, carried from step to step in a state slot.
//
// Two forms share the kernels (MODE):
//   0, the generalized delta rule: per key channel a decay w = exp(-decay_scale * sigmoid(w0 + W2 tanh(p)))
//     (p: a low-rank projection of the layer's input), a removal rate a = sigmoid(a' + a_bias), the unit key
//     u = k / sqrt(sum k^2 + unit_eps); decay and removal both act on S_(t-1).  Output: each
//     head's o divided by its root mean square, times a weight per (head, column), times sigmoid(g).
//   1, a gated linear recurrence with one gate for forgetting and writing: f = l + (1 - l) *
//     sigmoid(f' + f_bias), w = f, k = 1 - f, r = silu(q'), no removal.  Output: each head's o RMS-normed with
//     a weight per column that the heads share.
//   2, linear attention with a decay per key channel: w = sigmoid(z)^(1/tau) with z = w0 + W2 p (p: a low-rank
//     projection of the layer's input, no function in between), evaluated as exp(logsigmoid(z) / tau); k as it
//     comes, r = q' * qscale, no removal.  Output: each head's o RMS-normed with a weight per column that the
//     heads share, times silu(g).
//   3, a matrix memory with exponential gates and a running maximum m per head (kept beside the state, zero
//     at the start): i = cap * tanh((i' + i_bias) / cap), f = logsigmoid(cap * tanh((f' + f_bias) / cap)),
//     m_t = max(f + m_(t-1), i), w = exp(f + m_(t-1) - m_t) for every channel, k = exp(i - m_t) k', r = q' * qscale.
//     The normaliser n_t = w n_(t-1) + k is one more column of the state, whose value is 1 for every token, so
//     the state has dv = (value size + 1) columns and n . r arrives as the output's last column.  Output:
//     o / (max(|n . r|, exp(-m_t)) + floor_eps), each head's divided by its root mean square, times a weight
//     per (head, column), times sigmoid(g).  `recurrence_gate_scan_kernel` walks a request's tokens in their order for
//     m_t, a warp a (request, head), and leaves (w, exp(i - m_t), exp(-m_t)) per (token, head).
//
// The inputs are columns of one float32 matrix (the packed projections of the layer's input).  Three kernels:
//   `recurrence_prep_kernel`, a block a token: everything that does not depend on the state (sigmoids,
//     exponentials, the low-rank product, the unit key), in float32, into one record per (head, token):
//     [w | k | r (| u | a*u)] of DKP entries each, then the token's values (DVP entries);
//   `recurrence_seq_kernel`, a block a (request, head, group of state columns): the only sequential part.  Eight
//     neighbouring lanes share a column of the state, each holding an eighth of its rows in registers; a token costs
//     them two reductions over the eight lanes (u^T S and S^T r).  The records of a chunk of tokens are one contiguous
//     piece of memory, copied into shared memory with cp.async while the chunk before is worked on;
//   `recurrence_out_kernel`, a warp a (token, head): the head's norm, weight and gate, in the activation type.
#include "common.cuh"

namespace rl {

struct RecurParams {
  const float* proj;  // [tokens, ldp]
  long ldp;
  int off_r, off_k, off_v, off_a, off_g, off_w;  // first column of each projection (-1: the form has none)
  const float* a_bias;      // [heads * dk]: the removal rate's bias (0), the forget gate's bias (1)
  const float* w0;          // [heads * dk]: the decay's bias (0), the forget gate's lower bound (1)
  const float* w2t;         // [rank, heads * dk] (0): the low-rank product's second matrix, transposed
  int rank;
  const float* out_weight;  // [heads * dv] (0), [dv] (1)
  float* state;             // [slots, heads, dk, dv]
  void* out;                // [tokens, ldo]
  long ldo;
  const int* q_start;
  const int* slots;
  float* prep;  // [heads, tokens, rec]
  float* oraw;  // [tokens, heads * dv]
  int n_tokens, n_heads, dk, dv, dkp, dvp, rec;
  float eps, decay_scale, unit_eps;
  long state_stride;  // floats a slot
  int m_off;          // (3) where a slot's running maxima [heads] begin
  int dv_in;          // value columns a head in proj (dv, or dv - 1 for the form whose last column is the normaliser)
  float tau_inv, cap, floor_eps, qscale;
  float* gates;       // (3) [tokens, heads, 4]: w, exp(i - m_t), exp(-m_t)
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The running maximum of the matrix memory and what follows from it.  The maximum is walked token by token in
// order (so that the numbers do not depend on how a prompt was cut), a warp a (request, head); what does not lie
// on that chain is spread over the block's threads: a block takes a request and SCAN_HEADS heads and works through
// the request's tokens in rounds of SCAN_TOKENS: (a) the capped gates of all the round's (token, head) pairs
// into shared memory, (b) each warp walks its head's tokens, a token costing the chain one sum and one maximum,
// and parks the maximum before and after every token, (c) the exponentials of all pairs.
// 16 warps a block: the gates' functions are a few hundred dependent instructions a (token, head), which four warps
// alone on an SM would run at one instruction every few cycles
constexpr int SCAN_TOKENS = 512, SCAN_THREADS = 512, SCAN_HEADS = 1, SCAN_ROW = SCAN_TOKENS + 8;  // rows apart by 8 banks

__global__ __launch_bounds__(SCAN_THREADS) void recurrence_gate_scan_kernel(const RecurParams p) {
  __shared__ float s_i[SCAN_HEADS * SCAN_ROW], s_f[SCAN_HEADS * SCAN_ROW], s_before[SCAN_HEADS * SCAN_ROW], s_after[SCAN_HEADS * SCAN_ROW];
  pdl_begin();
  const int req = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h0 = blockIdx.y * SCAN_HEADS, nh = min(SCAN_HEADS, p.n_heads - h0);
  if (nh <= 0) return;
  const int slot = p.slots[req];
  if (slot < 0) return;
  const int t0 = p.q_start[req], t1 = p.q_start[req + 1];
  float* mp = p.state + (size_t)slot * p.state_stride + p.m_off + h0 + warp;
  float m = warp < nh ? *mp : 0.f;
  for (int base = t0; base < t1; base += SCAN_TOKENS) {
    const int n = min(SCAN_TOKENS, t1 - base);
    // (a) all of a thread's logits are on their way before the first is used
    float zi[SCAN_TOKENS * SCAN_HEADS / SCAN_THREADS], zf[SCAN_TOKENS * SCAN_HEADS / SCAN_THREADS];
#pragma unroll
    for (int k = 0; k < SCAN_TOKENS * SCAN_HEADS / SCAN_THREADS; ++k) {
      const int idx = threadIdx.x + k * SCAN_THREADS, tt = idx / nh, hh = idx - tt * nh;
      if (idx < n * nh) {
        const float* row = p.proj + (size_t)(base + tt) * p.ldp;
        zi[k] = row[p.off_a + h0 + hh] + p.a_bias[h0 + hh];
        zf[k] = row[p.off_w + h0 + hh] + p.w0[h0 + hh];
      }
    }
#pragma unroll
    for (int k = 0; k < SCAN_TOKENS * SCAN_HEADS / SCAN_THREADS; ++k) {
      const int idx = threadIdx.x + k * SCAN_THREADS, tt = idx / nh, hh = idx - tt * nh;
      if (idx < n * nh) {
        s_i[hh * SCAN_ROW + tt] = p.cap * tanhf(zi[k] / p.cap);
        s_f[hh * SCAN_ROW + tt] = logsigmoidf_(p.cap * tanhf(zf[k] / p.cap));
      }
    }
    __syncthreads();
    // (b) every lane of the head's warp walks the same chain, eight tokens at a time: their gates are taken from
    // shared memory into registers first (loads that do not wait for m; past the round's last token gates that
    // leave m as it is), and the maxima are parked by lane 0 after the eight steps, so nothing but one sum and
    // one maximum a token lies between a token's m and the next
    if (warp < nh) {
      const float* gi = s_i + warp * SCAN_ROW;
      const float* gf = s_f + warp * SCAN_ROW;
      for (int t8 = 0; t8 < n; t8 += 8) {
        float f8[8], i8[8], m8[9];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          f8[k] = t8 + k < n ? gf[t8 + k] : 0.f;
          i8[k] = t8 + k < n ? gi[t8 + k] : -INFINITY;
        }
        m8[0] = m;
#pragma unroll
        for (int k = 0; k < 8; ++k) m8[k + 1] = fmaxf(f8[k] + m8[k], i8[k]);
        m = m8[8];
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (t8 + k < n) {
              s_before[warp * SCAN_ROW + t8 + k] = m8[k];
              s_after[warp * SCAN_ROW + t8 + k] = m8[k + 1];
            }
        }
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * nh; idx += blockDim.x) {
      const int tt = idx / nh, hh = idx - tt * nh, at = hh * SCAN_ROW + tt;
      const float m_after = s_after[at];
      float* g = p.gates + ((size_t)(base + tt) * p.n_heads + h0 + hh) * 4;
      g[0] = expf(s_f[at] + s_before[at] - m_after);
      g[1] = expf(s_i[at] - m_after);
      g[2] = expf(-m_after);
    }
    __syncthreads();  // the next round overwrites what this one read
  }
  if (warp < nh && lane == 0) *mp = m;
}

// A block takes one token and `heads_per_block` heads.  Dynamic shared memory (MODE 0): tanh of the low-rank
// input [rank], then k and a of the block's channels [heads_per_block * dk] each.
template <int MODE>
__global__ __launch_bounds__(256) void recurrence_prep_kernel(const RecurParams p, int heads_per_block) {
  extern __shared__ float prep_s[];
  pdl_begin();
  const int tok = blockIdx.x;
  const int h0 = blockIdx.y * heads_per_block, h1 = min(p.n_heads, h0 + heads_per_block);  // this block's heads
  const int C = p.n_heads * p.dk, dk = p.dk, dkp = p.dkp;
  const float* row = p.proj + (size_t)tok * p.ldp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  auto record = [&](int head) { return p.prep + ((size_t)head * p.n_tokens + tok) * p.rec; };
  if (MODE == 0) {
    float* Ls = prep_s;
    float* Ks = Ls + p.rank - h0 * dk;            // indexed by channel; the block's own channels are kept
    float* As = Ks + heads_per_block * dk;
    for (int r = threadIdx.x; r < p.rank; r += blockDim.x) Ls[r] = tanhf(row[p.off_w + r]);
    __syncthreads();
    for (int c = h0 * dk + threadIdx.x; c < h1 * dk; c += blockDim.x) {
      float wl = p.w0[c];
#pragma unroll 8
      for (int q = 0; q < p.rank; ++q) wl = fmaf(p.w2t[(size_t)q * C + c], Ls[q], wl);
      const int head = c / dk, i = c - head * dk;
      float* rec = record(head);
      const float k = row[p.off_k + c];
      rec[i] = expf(-p.decay_scale * sigmoidf_(wl));
      rec[dkp + i] = k;
      rec[2 * dkp + i] = row[p.off_r + c];
      Ks[c] = k;
      As[c] = sigmoidf_(row[p.off_a + c] + p.a_bias[c]);
    }
    __syncthreads();
    for (int head = h0 + warp; head < h1; head += n_warps) {
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss = fmaf(Ks[head * dk + i], Ks[head * dk + i], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + p.unit_eps);
      float* rec = record(head);
      for (int i = lane; i < dkp; i += 32) {
        const float u = i < dk ? Ks[head * dk + i] * inv : 0.f;
        rec[3 * dkp + i] = u;
        rec[4 * dkp + i] = i < dk ? As[head * dk + i] * u : 0.f;
        if (i >= dk) rec[i] = rec[dkp + i] = rec[2 * dkp + i] = 0.f;
      }
    }
  } else {
    if (MODE == 2) {  // the low-rank input of the decay, as it comes
      for (int r = threadIdx.x; r < p.rank; r += blockDim.x) prep_s[r] = row[p.off_w + r];
      __syncthreads();
    }
    for (int c = h0 * dkp + threadIdx.x; c < h1 * dkp; c += blockDim.x) {
      const int head = c / dkp, i = c - head * dkp;
      float w = 0.f, k = 0.f, r = 0.f;
      if (i < dk) {
        const int ch = head * dk + i;
        if (MODE == 1) {
          const float l = p.w0[ch];
          const float f = l + (1.0f - l) * sigmoidf_(row[p.off_a + ch] + p.a_bias[ch]);
          const float q = row[p.off_r + ch];
          w = f;
          k = 1.0f - f;
          r = q * sigmoidf_(q);
        } else if (MODE == 2) {
          float z = p.w0[ch];
#pragma unroll 8
          for (int q = 0; q < p.rank; ++q) z = fmaf(p.w2t[(size_t)q * C + ch], prep_s[q], z);
          w = expf(logsigmoidf_(z) * p.tau_inv);
          k = row[p.off_k + ch];
          r = row[p.off_r + ch] * p.qscale;
        } else {
          const float* g = p.gates + ((size_t)tok * p.n_heads + head) * 4;
          w = g[0];
          k = g[1] * row[p.off_k + ch];
          r = row[p.off_r + ch] * p.qscale;
        }
      }
      float* rec = record(head);
      rec[i] = w;
      rec[dkp + i] = k;
      rec[2 * dkp + i] = r;
    }
  }
  constexpr int NV = MODE == 0 ? 5 : 3;
  for (int c = h0 * p.dvp + threadIdx.x; c < h1 * p.dvp; c += blockDim.x) {
    const int head = c / p.dvp, j = c - head * p.dvp;
    float v = 0.f;
    if (j < p.dv_in) v = row[p.off_v + head * p.dv_in + j];
    else if (j < p.dv) v = 1.0f;  // the normaliser's column
    record(head)[NV * dkp + j] = v;
  }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// TPC lanes share a column of the state; DKQ = DKP / TPC rows a thread.  Thread (column = tid / TPC, part =
// tid % TPC) holds the rows 4 TPC m + 4 part + e (m < DKQ / 4, e < 4) of its column: the parts read
// neighbouring 16-byte pieces of a record's vectors.  chunk: tokens a buffer of shared memory; cols: columns a
// block.  A token is a chain of dependent steps (u^T S, its reduction over the parts, the update, S^T r, its
// reduction), and a warp has nothing else to do meanwhile: so the vectors of the NEXT token are taken from
// shared memory into registers before the current token's reductions, and the chain itself is kept short.
constexpr int REC_THREADS = 256;  // most threads a block

template <int MODE, int NV, int DKQ>
struct TokenVectors {
  float4 v[NV][DKQ / 4];
  float value;
};

template <int MODE, int TPC, int DKQ>
__global__ __launch_bounds__(REC_THREADS) void recurrence_seq_kernel(const RecurParams p, int chunk, int cols) {
  extern __shared__ __align__(16) float seq_s[];
  pdl_begin();
  const int req = blockIdx.x, head = blockIdx.y;
  const int slot = p.slots[req];
  if (slot < 0) return;  // a padding row of a captured step
  constexpr int NV = MODE == 0 ? 5 : 3;
  constexpr int DKP = TPC * DKQ;
  const int t0 = p.q_start[req], t1 = p.q_start[req + 1];
  const int dk = p.dk, dv = p.dv, rec = p.rec;
  const int col = blockIdx.z * cols + threadIdx.x / TPC, part = threadIdx.x % TPC;
  float S[DKQ];
  float* st = p.state + (size_t)slot * p.state_stride + ((size_t)head * dk) * dv;
#pragma unroll
  for (int k = 0; k < DKQ; ++k) {
    const int r = (k >> 2) * 4 * TPC + 4 * part + (k & 3);
    S[k] = (r < dk && col < dv) ? st[(size_t)r * dv + col] : 0.f;
  }
  const float* src = p.prep + ((size_t)head * p.n_tokens + t0) * rec;
  const int n_tok = t1 - t0;
  const int n_chunks = (n_tok + chunk - 1) / chunk;
  auto fetch = [&](int c) {
    const int nt = min(chunk, n_tok - c * chunk);
    float* dst = seq_s + (size_t)(c & 1) * chunk * rec;
    const float* from = src + (size_t)c * chunk * rec;
    for (int i = threadIdx.x; i < nt * rec / 4; i += blockDim.x) cp_async16(dst + 4 * i, from + 4 * i);
    cp_async_commit();
  };
  auto take = [&](const float* r_, auto& tv) {
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const float4* V4 = reinterpret_cast<const float4*>(r_ + n * DKP);
#pragma unroll
      for (int m = 0; m < DKQ / 4; ++m) tv.v[n][m] = V4[TPC * m + part];
    }
    tv.value = col < p.dvp ? r_[NV * DKP + col] : 0.f;
  };
  fetch(0);
  constexpr bool AHEAD = NV * DKQ <= 80;  // two sets of a token's vectors fit the registers
  float* Po = seq_s + (size_t)2 * chunk * rec;  // [chunk][threads]: every thread's share of S^T r, summed after the chunk
  // One token: the state's update, and this thread's share of the output, parked in shared memory (its sum
  // over the lanes of a column is not on the way to the next token, so it waits for the end of the chunk).
  auto step = [&](const auto& tv, int t) {
    const float vj = tv.value;
    float pj = 0.f;
    if (MODE == 0) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int m = 0; m < DKQ / 4; ++m) {
        const float4 u = tv.v[3][m];
        a0 = fmaf(u.x, S[4 * m], fmaf(u.y, S[4 * m + 1], a0));
        a1 = fmaf(u.z, S[4 * m + 2], fmaf(u.w, S[4 * m + 3], a1));
      }
      pj = a0 + a1;
#pragma unroll
      for (int o = 1; o < TPC; o <<= 1) pj += __shfl_xor_sync(0xffffffffu, pj, o);
    }
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int m = 0; m < DKQ / 4; ++m) {
      const float4 w = tv.v[0][m], k = tv.v[1][m], r = tv.v[2][m];
      float4 au = make_float4(0.f, 0.f, 0.f, 0.f);
      if (MODE == 0) au = tv.v[NV - 1][m];
      const float s0 = fmaf(w.x, S[4 * m], fmaf(-au.x, pj, k.x * vj));
      const float s1 = fmaf(w.y, S[4 * m + 1], fmaf(-au.y, pj, k.y * vj));
      const float s2 = fmaf(w.z, S[4 * m + 2], fmaf(-au.z, pj, k.z * vj));
      const float s3 = fmaf(w.w, S[4 * m + 3], fmaf(-au.w, pj, k.w * vj));
      S[4 * m] = s0;
      S[4 * m + 1] = s1;
      S[4 * m + 2] = s2;
      S[4 * m + 3] = s3;
      o0 = fmaf(s0, r.x, fmaf(s1, r.y, o0));
      o1 = fmaf(s2, r.z, fmaf(s3, r.w, o1));
    }
    Po[t * blockDim.x + threadIdx.x] = o0 + o1;
  };
  TokenVectors<MODE, NV, DKQ> va;
  TokenVectors<MODE, NV, AHEAD ? DKQ : 4> vb;
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) {
      fetch(c + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int nt = min(chunk, n_tok - c * chunk);
    const float* buf = seq_s + (size_t)(c & 1) * chunk * rec;
    if constexpr (AHEAD) {  // two sets of registers in turn: a token's vectors are on their way while the one before is worked on
      take(buf, va);
      for (int t = 0; t < nt; t += 2) {
        if (t + 1 < nt) take(buf + (size_t)(t + 1) * rec, vb);
        step(va, t);
        if (t + 1 < nt) {
          if (t + 2 < nt) take(buf + (size_t)(t + 2) * rec, va);
          step(vb, t + 1);
        }
      }
    } else {
      for (int t = 0; t < nt; ++t) {
        take(buf + (size_t)t * rec, va);
        step(va, t);
      }
    }
    __syncthreads();  // the shares of a column are summed by whichever thread the (token, column) pair falls to
    // the chunk's outputs: (token, column) pairs over the block's threads, the column's parts summed in order
    const int cols_here = blockDim.x / TPC;
    for (int i = threadIdx.x; i < nt * cols_here; i += blockDim.x) {
      const int t = i / cols_here, cl = i - t * cols_here;
      const float* pp = Po + t * blockDim.x + cl * TPC;
      float o = 0.f;
#pragma unroll
      for (int x = 0; x < TPC; ++x) o += pp[x];
      const int cg = blockIdx.z * cols + cl;
      if (cg < dv) p.oraw[(size_t)(t0 + c * chunk + t) * p.n_heads * dv + (size_t)head * dv + cg] = o;
    }
    __syncthreads();  // the buffer is free for the chunk after the next, the parked shares have been read
  }
#pragma unroll
  for (int k = 0; k < DKQ; ++k) {
    const int r = (k >> 2) * 4 * TPC + 4 * part + (k & 3);
    if (r < dk && col < dv) st[(size_t)r * dv + col] = S[k];
  }
}

template <int MODE, typename TOut>
__global__ __launch_bounds__(256) void recurrence_out_kernel(const RecurParams p) {
  pdl_begin();
  const int tok = blockIdx.x, dvs = p.dv, dv = p.dv_in;  // columns of the state, and those that are values
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const float* row = p.proj + (size_t)tok * p.ldp;
  for (int head = warp; head < p.n_heads; head += n_warps) {
    const float* o = p.oraw + (size_t)tok * p.n_heads * dvs + (size_t)head * dvs;
    float div = 1.0f;
    if (MODE == 3) {
      const float em = p.gates[((size_t)tok * p.n_heads + head) * 4 + 2];
      div = 1.0f / (fmaxf(fabsf(o[dv]), em) + p.floor_eps);
    }
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
      const float v = o[c] * div;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)dv + p.eps);
    TOut* orow = reinterpret_cast<TOut*>(p.out) + (size_t)tok * p.ldo + (size_t)head * dv;
    for (int c = lane; c < dv; c += 32) {
      float v = o[c] * div * rn;
      if (MODE == 0 || MODE == 3) {
        v = v * p.out_weight[head * dv + c] * sigmoidf_(row[p.off_g + head * dv + c]);
      } else {
        v = v * p.out_weight[c];
        if (MODE == 2) {
          const float g = row[p.off_g + head * dv + c];
          v *= g * sigmoidf_(g);
        }
      }
      orow[c] = from_f32<TOut>(v);
    }
  }
}

template <int MODE, int TPC, int DKQ>
static void launch_seq(const RecurParams& p, int n_reqs, cudaStream_t stream) {
  // Columns a block: a token's work is a chain of dependent steps that every warp walks for itself, so few
  // columns a block and many blocks are what is fast, as long as there are SMs for them: halved from the
  // most a block takes until the grid fills the device (down to one warp).
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  constexpr int per_warp = 32 / TPC;
  int cols = (p.dv + per_warp - 1) / per_warp * per_warp;
  cols = cols > REC_THREADS / TPC ? REC_THREADS / TPC : cols;
  while (cols > per_warp && (long)n_reqs * p.n_heads * ((p.dv + cols - 1) / cols) < sms) cols /= 2;
  cols = (cols + per_warp - 1) / per_warp * per_warp;
  const int col_blocks = (p.dv + cols - 1) / cols;
  // Tokens a buffer: a block's shared memory (two buffers of records and the parked output shares) is kept
  // near 36 KB, so that three blocks fit an SM under the library's common split and a grid of up to three
  // blocks an SM runs in one round (with 80 KB a block, the 256 blocks of a prompt step of two requests took
  // two rounds: 515 us against 315);
  // at most 16, at least 2.
  const size_t per_token = ((size_t)2 * p.rec + (size_t)TPC * cols) * sizeof(float);
  int chunk = (int)(36 * 1024 / per_token);
  chunk = chunk < 2 ? 2 : (chunk > 16 ? 16 : chunk);
  const size_t smem = (size_t)chunk * per_token;
  auto kernel = recurrence_seq_kernel<MODE, TPC, DKQ>;
  if (smem > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      note_launch(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      raised = true;
    }
  }
  launch_pdl(kernel, dim3(n_reqs, p.n_heads, col_blocks), TPC * cols, smem, stream, p, chunk, cols);
}

// Eight lanes a column wherever a thread still holds whole 16-byte pieces (DKP >= 32); four for DKP = 16.
template <int MODE>
static void dispatch_seq(const RecurParams& p, int n_reqs, cudaStream_t stream) {
  switch (p.dkp) {
    case 16: launch_seq<MODE, 4, 4>(p, n_reqs, stream); break;
    case 32: launch_seq<MODE, 8, 4>(p, n_reqs, stream); break;
    case 64: launch_seq<MODE, 8, 8>(p, n_reqs, stream); break;
    case 128: launch_seq<MODE, 8, 16>(p, n_reqs, stream); break;
    default: launch_seq<MODE, 8, 32>(p, n_reqs, stream); break;
  }
}

}  // namespace rl

// The padded key size of a record's vectors (16, 32, 64, 128 or 256), the padded value size, and the floats a
// record takes: what the caller sizes `prep` by (heads * tokens * record floats).
RL_EXPORT int rl_recurrence_record(int mode, int dk, int dv, int* dkp, int* dvp, int* rec) {
  if (mode < 0 || mode > 3 || dk <= 0 || dk > 256 || dv <= 0 || dv > 257 || (dv > 256 && mode != 3)) return -2;
  int k = 16;
  while (k < dk) k *= 2;
  *dkp = k;
  *dvp = (dv + 3) & ~3;
  *rec = (mode == 0 ? 5 : 3) * k + *dvp;
  return 0;
}

// mode 0: generalized delta rule; 1: gated recurrence; 2: linear attention with decaying key channels; 3: matrix
// memory (see the top of this file).  proj: float32 [tokens, ldp] holding the projections at the given column
// offsets (3: off_a the input gate's and off_w the forget gate's logits, one column a head; a_bias and w0 their
// biases [heads]); state: float32, `state_stride` floats a slot, of which the first heads * dk * dv are the
// matrices (3: dv is the value size + 1, and the heads' running maxima lie at `m_off`), read and written for the
// step's requests (slot < 0: skipped); out: [tokens, heads * value size] of out_dtype, row stride ldo.
// prep: float32 scratch [heads * tokens * record]; oraw: float32 scratch [tokens, heads * dv]; gates (3): float32
// scratch [tokens * heads * 4].
RL_EXPORT int rl_recurrence(int mode, int out_dtype, const float* proj, long ldp, int off_r, int off_k, int off_v,
                            int off_a, int off_g, int off_w, const float* a_bias, const float* w0, const float* w2t,
                            int rank, const float* out_weight, float* state, void* out, long ldo, const int* q_start,
                            const int* slots, float* prep, float* oraw, int n_tokens, int n_reqs, int n_heads, int dk,
                            int dv, float eps, float decay_scale, float unit_eps, long state_stride, int m_off,
                            float tau, float cap, float floor_eps, float qscale, float* gates, cudaStream_t stream) {
  if (n_reqs <= 0 || n_tokens <= 0) return 0;
  int dkp, dvp, rec;
  if (rl_recurrence_record(mode, dk, dv, &dkp, &dvp, &rec) != 0 || n_heads <= 0 || n_heads > 65535 || rank < 0) return -2;
  if (state_stride < (long)n_heads * dk * dv) return -2;
  if (mode == 2 && (tau <= 0.f || w2t == nullptr || rank <= 0)) return -2;
  if (mode == 3 && (cap <= 0.f || gates == nullptr || dv < 2 || m_off < n_heads * dk * dv || m_off + n_heads > state_stride))
    return -2;
  rl::RecurParams p{proj, ldp, off_r, off_k, off_v, off_a, off_g, off_w, a_bias, w0, w2t, rank, out_weight, state, out,
                    ldo, q_start, slots, prep, oraw, n_tokens, n_heads, dk, dv, dkp, dvp, rec, eps, decay_scale, unit_eps,
                    state_stride, m_off, mode == 3 ? dv - 1 : dv, mode == 2 ? 1.0f / tau : 0.f, cap, floor_eps, qscale, gates};
  // heads a block of the preparation: about 256 channels (a thread a channel), fewer with many tokens' worth of blocks anyway
  int hpb = 256 / dk;
  hpb = hpb < 1 ? 1 : (hpb > n_heads ? n_heads : hpb);
  const dim3 prep_grid(n_tokens, (n_heads + hpb - 1) / hpb);
  const size_t prep_smem = mode == 0 ? ((size_t)rank + 2 * (size_t)hpb * dk) * sizeof(float)
                                     : (mode == 2 ? (size_t)rank * sizeof(float) : 0);
  if (prep_smem > 48 * 1024) return -2;
  if (mode == 0) {
    rl::launch_pdl(rl::recurrence_prep_kernel<0>, prep_grid, 256, prep_smem, stream, p, hpb);
    rl::dispatch_seq<0>(p, n_reqs, stream);
    if (out_dtype == RL_F32) rl::launch_pdl(rl::recurrence_out_kernel<0, float>, n_tokens, 256, 0, stream, p);
    else rl::launch_pdl(rl::recurrence_out_kernel<0, __nv_bfloat16>, n_tokens, 256, 0, stream, p);
  } else if (mode == 1) {
    rl::launch_pdl(rl::recurrence_prep_kernel<1>, prep_grid, 256, 0, stream, p, hpb);
    rl::dispatch_seq<1>(p, n_reqs, stream);
    if (out_dtype == RL_F32) rl::launch_pdl(rl::recurrence_out_kernel<1, float>, n_tokens, 256, 0, stream, p);
    else rl::launch_pdl(rl::recurrence_out_kernel<1, __nv_bfloat16>, n_tokens, 256, 0, stream, p);
  } else if (mode == 2) {  // the sequential kernel is the one of the form without removal
    rl::launch_pdl(rl::recurrence_prep_kernel<2>, prep_grid, 256, prep_smem, stream, p, hpb);
    rl::dispatch_seq<1>(p, n_reqs, stream);
    if (out_dtype == RL_F32) rl::launch_pdl(rl::recurrence_out_kernel<2, float>, n_tokens, 256, 0, stream, p);
    else rl::launch_pdl(rl::recurrence_out_kernel<2, __nv_bfloat16>, n_tokens, 256, 0, stream, p);
  } else {
    rl::launch_pdl(rl::recurrence_gate_scan_kernel, dim3(n_reqs, (n_heads + rl::SCAN_HEADS - 1) / rl::SCAN_HEADS), rl::SCAN_THREADS, 0, stream, p);
    rl::launch_pdl(rl::recurrence_prep_kernel<3>, prep_grid, 256, 0, stream, p, hpb);
    rl::dispatch_seq<1>(p, n_reqs, stream);
    if (out_dtype == RL_F32) rl::launch_pdl(rl::recurrence_out_kernel<3, float>, n_tokens, 256, 0, stream, p);
    else rl::launch_pdl(rl::recurrence_out_kernel<3, __nv_bfloat16>, n_tokens, 256, 0, stream, p);
  }
  RL_CHECK_LAUNCH();
  return 0;
}
