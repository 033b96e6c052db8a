// RMS norm: y = x / sqrt(mean(x^2) + eps) * w, statistics and arithmetic in float32.
//
// Two uses.  `rmsnorm_store_kernel` writes normalised rows (optionally gathered by index) in
// float32 or bfloat16: a final norm ahead of a head, or a norm ahead of a sublayer.
// `rmsnorm_add_kernel` serves blocks that normalise a sublayer's OUTPUT: the float32 residual
// stream gets `stream += mult * rmsnorm(y) * w`, and the same kernel may leave a bfloat16 copy
// of the stream's new rows for the products of the next sublayer to read, so that no kernel of
// its own has to round the stream.  `cast_rows_kernel` makes that copy where nothing precedes.
#include "common.cuh"

namespace rl {

// One block per row; the row is read twice (the second time from L1/L2).
template <typename TOut>
__global__ __launch_bounds__(256) void rmsnorm_store_kernel(const float* __restrict__ x, long ldx,
                                                            const int* __restrict__ rows,
                                                            const float* __restrict__ gamma, TOut* __restrict__ out,
                                                            long ldo, int n_out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_begin();
  const int i = blockIdx.x;
  if (i >= n_out) return;
  const int src = rows != nullptr ? rows[i] : i;
  const float* xr = x + (size_t)src * ldx;
  float s = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = xr[d];
    s = fmaf(v, v, s);
  }
  const float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)width + eps);
  TOut* o = out + (size_t)i * ldo;
  for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = from_f32<TOut>(xr[d] * r * gamma[d]);
}

// stream[i] += mult * rmsnorm(y[i]) * gamma; copy[i] = bfloat16(stream[i]) when copy is given.
// VEC: widths and row strides are multiples of 4 and every row starts on a 16-byte boundary
// (8-byte for the copy): 16-byte loads and stores.
template <bool VEC>
__global__ __launch_bounds__(256) void rmsnorm_add_kernel(const float* __restrict__ y, long ldy,
                                                          const float* __restrict__ gamma, float* __restrict__ stream,
                                                          long lds, __nv_bfloat16* __restrict__ copy, long ldc,
                                                          int n_rows, int width, float eps, float mult) {
  __shared__ float scratch[33];
  pdl_begin();
  const int i = blockIdx.x;
  if (i >= n_rows) return;
  const float* yr = y + (size_t)i * ldy;
  float* xr = stream + (size_t)i * lds;
  float s = 0.f;
  if (VEC) {
    const float4* y4 = reinterpret_cast<const float4*>(yr);
    for (int d = threadIdx.x; d < width / 4; d += blockDim.x) {
      const float4 v = y4[d];
      s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s))));
    }
  } else {
    for (int d = threadIdx.x; d < width; d += blockDim.x) s = fmaf(yr[d], yr[d], s);
  }
  const float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)width + eps);
  if (VEC) {
    const float4* y4 = reinterpret_cast<const float4*>(yr);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    float4* x4 = reinterpret_cast<float4*>(xr);
    for (int d = threadIdx.x; d < width / 4; d += blockDim.x) {
      const float4 v = y4[d], g = g4[d];
      float4 x = x4[d];
      x.x += mult * (v.x * r * g.x);
      x.y += mult * (v.y * r * g.y);
      x.z += mult * (v.z * r * g.z);
      x.w += mult * (v.w * r * g.w);
      x4[d] = x;
      if (copy != nullptr) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(copy + (size_t)i * ldc + 4 * d) = packed;
      }
    }
  } else {
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      const float v = xr[d] + mult * (yr[d] * r * gamma[d]);
      xr[d] = v;
      if (copy != nullptr) copy[(size_t)i * ldc + d] = __float2bfloat16_rn(v);
    }
  }
}

// stream[i] += rmsnorm(y[i]) * gamma, and next[i] = rmsnorm(stream[i]) * gamma_next of the new row, in one
// pass: the norm after one sublayer and the norm before the next (a layer that normalises its sublayers on
// both sides).  The row is kept in shared memory between the two statistics.
template <typename TOut>
__global__ __launch_bounds__(256) void rmsnorm_add_norm_kernel(const float* __restrict__ y, long ldy,
                                                               const float* __restrict__ gamma,
                                                               float* __restrict__ stream, long lds,
                                                               const float* __restrict__ gamma_next,
                                                               TOut* __restrict__ next, long ldn, int n_rows, int width,
                                                               float eps, float eps_next) {
  extern __shared__ float row_s[];  // [width] + 33
  float* scratch = row_s + width;
  pdl_begin();
  const int i = blockIdx.x;
  if (i >= n_rows) return;
  const float* yr = y + (size_t)i * ldy;
  float* xr = stream + (size_t)i * lds;
  float s = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = yr[d];
    row_s[d] = v;
    s = fmaf(v, v, s);
  }
  const float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)width + eps);
  float s2 = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = xr[d] + row_s[d] * r * gamma[d];
    xr[d] = v;
    row_s[d] = v;
    s2 = fmaf(v, v, s2);
  }
  const float r2 = 1.0f / sqrtf(block_sum(s2, scratch) / (float)width + eps_next);
  TOut* o = next + (size_t)i * ldn;
  for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = from_f32<TOut>(row_s[d] * r2 * gamma_next[d]);
}

__global__ void cast_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long n) {
  pdl_begin();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}

// stream[i] = rmsnorm(alpha * stream[i] + sigmoid(z[i] + zb) * (s0 * y0[i] + s1 * y1[i])) * gamma: the norm AFTER the sum
// of a layer that normalises the stream itself, with the sublayer's result (of one mixer, or of two side by
// side with a weight each) passing a gate whose logits z the caller computed from the sublayer's input (zb: the
// logits' bias, one entry a column, where the product that made z did not add it; null: none).  The new
// row also goes out in bfloat16 (copy) for the products of the next sublayer.  The row is kept in shared memory
// between the statistic and the scaling where it fits (KEEP), else worked out a second time.
template <bool KEEP>
__global__ __launch_bounds__(256) void gated_join_norm_kernel(const float* __restrict__ y0, long ld0, float s0,
                                                              const float* __restrict__ y1, long ld1, float s1,
                                                              const float* __restrict__ z, long ldz,
                                                              const float* __restrict__ zb,
                                                              const float* __restrict__ gamma, float* __restrict__ stream,
                                                              long lds, __nv_bfloat16* __restrict__ copy, long ldc,
                                                              int n_rows, int width, float eps, float alpha) {
  extern __shared__ float join_row_s[];
  __shared__ float scratch[33];
  pdl_begin();
  const int i = blockIdx.x;
  if (i >= n_rows) return;
  float* xr = stream + (size_t)i * lds;
  const float* a = y0 + (size_t)i * ld0;
  const float* b = y1 != nullptr ? y1 + (size_t)i * ld1 : nullptr;
  const float* zr = z != nullptr ? z + (size_t)i * ldz : nullptr;  // no logits: no gate
  auto joined = [&](int d) {
    float y = s0 * a[d];
    if (b != nullptr) y = fmaf(s1, b[d], y);
    const float g = zr != nullptr ? 1.0f / (1.0f + expf(-(zr[d] + (zb != nullptr ? zb[d] : 0.f)))) : 1.0f;
    return fmaf(alpha, xr[d], g * y);
  };
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = joined(d);
    if (KEEP) join_row_s[d] = v;
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x) {  // a thread meets the entries it wrote itself
    const float v = (KEEP ? join_row_s[d] : joined(d)) * r * gamma[d];
    xr[d] = v;
    if (copy != nullptr) copy[(size_t)i * ldc + d] = __float2bfloat16_rn(v);
  }
}

static inline int norm_threads(int width) {
  int t = (width + 3) / 4;
  t = (t + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 256 ? 256 : t);
}

}  // namespace rl

// out[i] = rmsnorm(x[rows[i]] or x[i]) * gamma.  out_dtype: RL_F32 or RL_BF16.
RL_EXPORT int rl_rmsnorm(int out_dtype, const float* x, long ldx, const int* rows, const float* gamma, void* out,
                         long ldo, int n_out, int width, float eps, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (width <= 0) return -2;
  const int threads = rl::norm_threads(width);
  if (out_dtype == RL_F32)
    rl::launch_pdl(rl::rmsnorm_store_kernel<float>, n_out, threads, 0, stream, x, ldx, rows, gamma, (float*)out, ldo,
                   n_out, width, eps);
  else
    rl::launch_pdl(rl::rmsnorm_store_kernel<__nv_bfloat16>, n_out, threads, 0, stream, x, ldx, rows, gamma,
                   (__nv_bfloat16*)out, ldo, n_out, width, eps);
  RL_CHECK_LAUNCH();
  return 0;
}

// stream += mult * rmsnorm(y) * gamma, with an optional bfloat16 copy of the stream's new rows.
RL_EXPORT int rl_rmsnorm_add(const float* y, long ldy, const float* gamma, float* stream_rows, long lds, void* copy,
                             long ldc, int n_rows, int width, float eps, float mult, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0) return -2;
  const bool vec = width % 4 == 0 && ldy % 4 == 0 && lds % 4 == 0 && ldc % 4 == 0 && (uintptr_t)y % 16 == 0 &&
                   (uintptr_t)stream_rows % 16 == 0 && (uintptr_t)gamma % 16 == 0 && (uintptr_t)copy % 8 == 0;
  rl::launch_pdl(vec ? rl::rmsnorm_add_kernel<true> : rl::rmsnorm_add_kernel<false>, n_rows, rl::norm_threads(width), 0,
                 stream, y, ldy, gamma, stream_rows, lds, (__nv_bfloat16*)copy, ldc, n_rows, width, eps, mult);
  RL_CHECK_LAUNCH();
  return 0;
}

// out = bfloat16(x), n elements.
RL_EXPORT int rl_cast_rows(const float* x, void* out, long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  rl::launch_pdl(rl::cast_rows_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, (__nv_bfloat16*)out, n);
  RL_CHECK_LAUNCH();
  return 0;
}

// stream += rmsnorm(y) * gamma; next = rmsnorm(new stream rows) * gamma_next (out_dtype: RL_F32 or RL_BF16).
RL_EXPORT int rl_rmsnorm_add_norm(int out_dtype, const float* y, long ldy, const float* gamma, float* stream_rows,
                                  long lds, const float* gamma_next, void* next, long ldn, int n_rows, int width,
                                  float eps, float eps_next, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0 || width > 48 * 1024 / 4 - 64) return -2;
  const size_t smem = (size_t)(width + 33) * sizeof(float);
  if (out_dtype == RL_F32)
    rl::launch_pdl(rl::rmsnorm_add_norm_kernel<float>, n_rows, rl::norm_threads(width), smem, stream, y, ldy, gamma,
                   stream_rows, lds, gamma_next, (float*)next, ldn, n_rows, width, eps, eps_next);
  else
    rl::launch_pdl(rl::rmsnorm_add_norm_kernel<__nv_bfloat16>, n_rows, rl::norm_threads(width), smem, stream, y, ldy,
                   gamma, stream_rows, lds, gamma_next, (__nv_bfloat16*)next, ldn, n_rows, width, eps, eps_next);
  RL_CHECK_LAUNCH();
  return 0;
}

// stream = rmsnorm(alpha * stream + sigmoid(z + zb) * (s0 * y0 + s1 * y1)) * gamma (y1 may be null; z null: no gate; zb null: no bias), with an optional
// bfloat16 copy of the new rows; see the kernel.
RL_EXPORT int rl_gated_join_norm(const float* y0, long ld0, float s0, const float* y1, long ld1, float s1, const float* z,
                                 long ldz, const float* zb, const float* gamma, float* stream_rows, long lds, void* copy, long ldc,
                                 int n_rows, int width, float eps, float alpha, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0 || y0 == nullptr) return -2;
  const int threads = rl::norm_threads(width);
  const size_t row_bytes = (size_t)width * sizeof(float);
  if (row_bytes <= 40 * 1024)
    rl::launch_pdl(rl::gated_join_norm_kernel<true>, n_rows, threads, row_bytes, stream, y0, ld0, s0, y1, ld1, s1, z, ldz,
                   zb, gamma, stream_rows, lds, (__nv_bfloat16*)copy, ldc, n_rows, width, eps, alpha);
  else
    rl::launch_pdl(rl::gated_join_norm_kernel<false>, n_rows, threads, 0, stream, y0, ld0, s0, y1, ld1, s1, z, ldz, zb, gamma,
                   stream_rows, lds, (__nv_bfloat16*)copy, ldc, n_rows, width, eps, alpha);
  RL_CHECK_LAUNCH();
  return 0;
}
