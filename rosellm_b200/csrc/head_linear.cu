// One small product per head: out[t, h, :] = in[t, h, :] W_h, for every token t and head h.
//
// Mixers that cache a latent instead of keys and values move the keys' and values'
// per-head up-projections to the query and to the output (see latent_attention.cu): the query
// of head h becomes q_plain W_uk,h (a [dim] row times a [dim, rank] matrix) and the head's
// output (sum of probabilities x latents) W_uv,h^T (a [rank] row times [rank, vdim]).  Both
// are this kernel; the weight of head h is reached by three strides (head, inner index, output
// index), so either storage order can be read.  float32: IEEE multiply-adds on 64 x 64 tiles
// (tile_gemm.cuh).  bfloat16 with the weight's inner index contiguous: the tensor cores
// (mma_tile.cuh), float32 accumulation; any other bfloat16 layout takes the float32 tiles.
// An output gate may ride on the epilogue (fused): out[t, h, n] *= sigmoid(gate[t, h, n]) with float32 logits
// reached by strides of their own, so a mixer that gates its merged heads needs no kernel for it.
#include "mma_tile.cuh"
#include "tile_gemm.cuh"

namespace rl {

template <typename T>
__global__ __launch_bounds__(256) void head_linear_kernel(const T* __restrict__ in, long in_tok, long in_head,
                                                          const T* __restrict__ w, long w_head, long w_k, long w_n,
                                                          T* __restrict__ out, long out_tok, long out_head,
                                                          int n_tokens, int k_total, int n_total,
                                                          const float* __restrict__ gate, long gate_tok, long gate_head) {
  __shared__ TileGemmSmem s;
  pdl_begin();
  const int h = blockIdx.z;
  const int m0 = blockIdx.x * TG_M, n0 = blockIdx.y * TG_N;
  const T* in_h = in + (size_t)h * in_head;
  const T* w_h = w + (size_t)h * w_head;
  float acc[4][4] = {};
  tile_gemm(
      acc, k_total,
      [&](int m, int k) {
        return (m0 + m < n_tokens && k < k_total) ? to_f32(in_h[(size_t)(m0 + m) * in_tok + k]) : 0.f;
      },
      [&](int k, int n) {
        return (n0 + n < n_total && k < k_total) ? to_f32(w_h[(size_t)k * w_k + (size_t)(n0 + n) * w_n]) : 0.f;
      },
      s);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < n_total) {
        float v = acc[i][j];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)m * gate_tok + (size_t)h * gate_head + n]));
        out[(size_t)m * out_tok + (size_t)h * out_head + n] = from_f32<T>(v);
      }
    }
  }
}

// bfloat16 on the tensor cores; the weight's inner index is contiguous (w_k == 1).
template <bool VEC>
__global__ __launch_bounds__(128) void head_linear_mma_kernel(const __nv_bfloat16* __restrict__ in, long in_tok,
                                                              long in_head, const __nv_bfloat16* __restrict__ w,
                                                              long w_head, long w_n, __nv_bfloat16* __restrict__ out,
                                                              long out_tok, long out_head, int n_tokens, int k_total,
                                                              int n_total, const float* __restrict__ gate,
                                                              long gate_tok, long gate_head) {
  __shared__ __align__(16) MmaTileSmem s;
  pdl_begin();
  const int h = blockIdx.z;
  const int m0 = blockIdx.x * MT_M, n0 = blockIdx.y * MT_N;
  const __nv_bfloat16* in_h = in + (size_t)h * in_head;
  const __nv_bfloat16* w_h = w + (size_t)h * w_head;
  float acc[2][4][4] = {};
  mma_tile<VEC>(
      acc, k_total, [&](int m) { return m0 + m < n_tokens ? in_h + (size_t)(m0 + m) * in_tok : nullptr; },
      [&](int n) { return n0 + n < n_total ? w_h + (size_t)(n0 + n) * w_n : nullptr; }, s);
  mma_for_each(acc, [&](int m, int n, int mi, int ni, int c) {
    if (m0 + m < n_tokens && n0 + n < n_total) {
      float v = acc[mi][ni][c];
      if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)(m0 + m) * gate_tok + (size_t)h * gate_head + n0 + n]));
      out[(size_t)(m0 + m) * out_tok + (size_t)h * out_head + n0 + n] = __float2bfloat16_rn(v);
    }
  });
}

}  // namespace rl

// in: element (t, h, k) at in + t*in_tok + h*in_head + k; w: element (h, k, n) at
// w + h*w_head + k*w_k + n*w_n; out: element (t, h, n) at out + t*out_tok + h*out_head + n.
// gate: null, or float32 logits, element (t, h, n) at gate + t*gate_tok + h*gate_head + n: out *= sigmoid(gate).
RL_EXPORT int rl_head_linear(int dtype, const void* in, long in_tok, long in_head, const void* w, long w_head, long w_k,
                             long w_n, void* out, long out_tok, long out_head, int n_tokens, int n_heads, int k_total,
                             int n_total, const float* gate, long gate_tok, long gate_head, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_heads <= 0 || n_heads > 65535 || k_total <= 0 || n_total <= 0) return -2;
  const dim3 grid((n_tokens + rl::TG_M - 1) / rl::TG_M, (n_total + rl::TG_N - 1) / rl::TG_N, n_heads);
  if (grid.y > 65535) return -2;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::head_linear_kernel<float>, grid, 256, 0, stream, (const float*)in, in_tok, in_head,
                   (const float*)w, w_head, w_k, w_n, (float*)out, out_tok, out_head, n_tokens, k_total, n_total, gate,
                   gate_tok, gate_head);
  else if (w_k == 1) {
    const bool vec = k_total % 8 == 0 && in_tok % 8 == 0 && in_head % 8 == 0 && w_head % 8 == 0 && w_n % 8 == 0 &&
                     ((uintptr_t)in % 16) == 0 && ((uintptr_t)w % 16) == 0;
    auto kernel = vec ? rl::head_linear_mma_kernel<true> : rl::head_linear_mma_kernel<false>;
    rl::launch_pdl(kernel, grid, 128, 0, stream, (const __nv_bfloat16*)in, in_tok, in_head, (const __nv_bfloat16*)w,
                   w_head, w_n, (__nv_bfloat16*)out, out_tok, out_head, n_tokens, k_total, n_total, gate, gate_tok, gate_head);
  } else
    rl::launch_pdl(rl::head_linear_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)in, in_tok,
                   in_head, (const __nv_bfloat16*)w, w_head, w_k, w_n, (__nv_bfloat16*)out, out_tok, out_head, n_tokens,
                   k_total, n_total, gate, gate_tok, gate_head);
  RL_CHECK_LAUNCH();
  return 0;
}
