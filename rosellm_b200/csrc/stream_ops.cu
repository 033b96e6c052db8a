// Element-wise work on the residual stream and on a mixer's merged heads.
//
// `stream_inject_kernel`: what a stack adds to the stream between two runs of layers, in float32:
//     keep <- x                      (keep given: the rows as they are now, for a later run to add again)
//     x    <- x + vec + again        (vec: one row [width] for all tokens; again: rows kept earlier; either absent)
// One pass over the rows whatever the combination.  `stream_inject_norm_kernel` does the same a block a row and
// leaves, in the same launch, the RMS norm of the new rows for the layer that runs next (fused: what is added ahead
// of a pass and that pass's first norm): h = x / sqrt(mean(x^2) + eps) * gamma in float32, stored in the activation type.
//
// `gate_mul_kernel`: o <- o * sigmoid(g) element by element, o in the activation type, g float32 logits (a view
// with a row stride will do): the output gate of a mixer whose heads' results are made by a product of their own.
#include "common.cuh"

namespace rl {

__global__ __launch_bounds__(256) void stream_inject_kernel(float* __restrict__ x, long ldx, const float* __restrict__ vec,
                                                            const float* __restrict__ again, long lda,
                                                            float* __restrict__ keep, long ldk, int n_rows, int width) {
  pdl_begin();
  const long total = (long)n_rows * width;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / width;
    const int c = (int)(i - r * width);
    float v = x[r * ldx + c];
    if (keep != nullptr) keep[r * ldk + c] = v;
    if (vec != nullptr) v += vec[c];
    if (again != nullptr) v += again[r * lda + c];
    x[r * ldx + c] = v;
  }
}

template <typename TOut>
__global__ __launch_bounds__(256) void stream_inject_norm_kernel(float* __restrict__ x, long ldx, const float* __restrict__ vec,
                                                                 const float* __restrict__ again, long lda,
                                                                 float* __restrict__ keep, long ldk,
                                                                 const float* __restrict__ gamma, float eps,
                                                                 TOut* __restrict__ out, long ldo, int n_rows, int width) {
  __shared__ float scratch[33];
  pdl_begin();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  float* xr = x + (size_t)r * ldx;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = xr[c];
    if (keep != nullptr) keep[(size_t)r * ldk + c] = v;
    if (vec != nullptr) v += vec[c];
    if (again != nullptr) v += again[(size_t)r * lda + c];
    xr[c] = v;
    s = fmaf(v, v, s);
  }
  const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)width + eps);
  TOut* o = out + (size_t)r * ldo;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_f32<TOut>(xr[c] * inv * gamma[c]);  // its own writes
}

template <typename T>
__global__ __launch_bounds__(256) void gate_mul_kernel(T* __restrict__ o, long ldo, const float* __restrict__ g, long ldg,
                                                       int n_rows, int width) {
  pdl_begin();
  const long total = (long)n_rows * width;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / width;
    const int c = (int)(i - r * width);
    const float v = to_f32(o[r * ldo + c]) * (1.0f / (1.0f + expf(-g[r * ldg + c])));
    o[r * ldo + c] = from_f32<T>(v);
  }
}

static int elementwise_blocks(long total) {
  const long want = (total + 255) / 256;
  return (int)(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
}

}  // namespace rl

// x: float32 [n_rows, width] (row stride ldx); vec: float32 [width] or null; again: float32 rows or null;
// keep: float32 rows or null (receives x as it was).  again and keep may be the same buffer only if one is null.
RL_EXPORT int rl_stream_inject(float* x, long ldx, const float* vec, const float* again, long lda, float* keep, long ldk,
                               int n_rows, int width, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return 0;
  if (x == nullptr || (again != nullptr && again == keep)) return -2;
  rl::launch_pdl(rl::stream_inject_kernel, rl::elementwise_blocks((long)n_rows * width), 256, 0, stream, x, ldx, vec, again,
                 lda, keep, ldk, n_rows, width);
  RL_CHECK_LAUNCH();
  return 0;
}

// The same, and out (float32 or bfloat16 by out_dtype, row stride ldo) = rmsnorm(new x) * gamma.
RL_EXPORT int rl_stream_inject_norm(int out_dtype, float* x, long ldx, const float* vec, const float* again, long lda,
                                    float* keep, long ldk, const float* gamma, float eps, void* out, long ldo, int n_rows,
                                    int width, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return 0;
  if (x == nullptr || gamma == nullptr || out == nullptr || (again != nullptr && again == keep)) return -2;
  if (out_dtype == RL_F32)
    rl::launch_pdl(rl::stream_inject_norm_kernel<float>, n_rows, 256, 0, stream, x, ldx, vec, again, lda, keep, ldk, gamma,
                   eps, (float*)out, ldo, n_rows, width);
  else
    rl::launch_pdl(rl::stream_inject_norm_kernel<__nv_bfloat16>, n_rows, 256, 0, stream, x, ldx, vec, again, lda, keep,
                   ldk, gamma, eps, (__nv_bfloat16*)out, ldo, n_rows, width);
  RL_CHECK_LAUNCH();
  return 0;
}

// o: [n_rows, width] float32 or bfloat16 (row stride ldo), multiplied in place by sigmoid(g), g float32 (row stride ldg).
RL_EXPORT int rl_gate_mul(int dtype, void* o, long ldo, const float* g, long ldg, int n_rows, int width,
                          cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return 0;
  if (o == nullptr || g == nullptr) return -2;
  const int blocks = rl::elementwise_blocks((long)n_rows * width);
  if (dtype == RL_F32)
    rl::launch_pdl(rl::gate_mul_kernel<float>, blocks, 256, 0, stream, (float*)o, ldo, g, ldg, n_rows, width);
  else
    rl::launch_pdl(rl::gate_mul_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)o, ldo, g, ldg, n_rows,
                   width);
  RL_CHECK_LAUNCH();
  return 0;
}
