// A residual stream that is kept in float whatever the engine's dtype, for layers whose norms sit on the sublayers'
// OUTPUTS:  x <- x + N(y),  N(y) = (y + bias) / sqrt(mean((y + bias)^2) + eps) * w.
//
//   norm_add      the update above for every token; x (float) is changed in place, and if `cast_out` is given it also
//                 receives x rounded once to the engine's dtype (what the next sublayer's first product reads), so the
//                 stream is never read again just to be rounded.  y: float or the engine's dtype; bias: float, per
//                 column, or none (an output projection's bias, added here in float instead of in a kernel of its own).
//   norm_rows     out[r] = N(x[rows[r]]) without the add (the model's last norm, at the rows whose logits are wanted).
//
// One block a token; a row's sum of squares is added in an order fixed by the thread layout, so a token's result does
// not depend on what else is in the step.
#include "common.cuh"

constexpr int PN_THREADS = 256;

template <typename TY, typename TO>
__global__ void __launch_bounds__(PN_THREADS)
norm_add_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ bias,
                const float* __restrict__ w, float eps, TO* __restrict__ cast_out, int width) {
  __shared__ float scratch[33];
  extern __shared__ float row[];                     // width floats: y + bias
  const size_t t = blockIdx.x;
  const TY* src = y + t * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_f32<TY>(src[c]);
    if (bias != nullptr) v += bias[c];
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  float* xr = x + t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float s = xr[c] + row[c] * r * w[c];
    xr[c] = s;
    if (cast_out != nullptr) cast_out[t * width + c] = from_f32<TO>(s);
  }
}

template <typename TO>
__global__ void __launch_bounds__(PN_THREADS)
norm_rows_kernel(TO* __restrict__ out, const float* __restrict__ x, const int* __restrict__ rows,
                 const float* __restrict__ w, float eps, int width) {
  __shared__ float scratch[33];
  const size_t r_out = blockIdx.x;
  const size_t t = rows != nullptr ? static_cast<size_t>(rows[r_out]) : r_out;
  const float* src = x + t * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[r_out * width + c] = from_f32<TO>(src[c] * r * w[c]);
}

// y_dtype: dtype of y; out_dtype: dtype of cast_out (ignored when cast_out is null).
B200_EXPORT int b200_norm_add(float* x, const void* y, int y_dtype, const float* bias, const float* w, float eps,
                              void* cast_out, int out_dtype, int tokens, int width, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || width * sizeof(float) > 200 * 1024) return B200_BAD_SIZE;
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
#define B200_NORM_ADD(TY, TO)                                                                                  \
  do {                                                                                                         \
    if (smem > 48 * 1024) {                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(norm_add_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           static_cast<int>(smem));                                            \
      if (e != cudaSuccess) return static_cast<int>(e);                                                        \
    }                                                                                                          \
    norm_add_kernel<TY, TO><<<tokens, PN_THREADS, smem, stream>>>(x, static_cast<const TY*>(y), bias, w, eps,   \
                                                                  static_cast<TO*>(cast_out), width);          \
  } while (0)
  const bool to_bf16 = cast_out != nullptr && out_dtype == B200_BF16;
  if (cast_out != nullptr && out_dtype != B200_BF16 && out_dtype != B200_F32) return B200_BAD_DTYPE;
  if (y_dtype == B200_F32) {
    if (to_bf16) B200_NORM_ADD(float, __nv_bfloat16); else B200_NORM_ADD(float, float);
  } else if (y_dtype == B200_BF16) {
    if (to_bf16) B200_NORM_ADD(__nv_bfloat16, __nv_bfloat16); else B200_NORM_ADD(__nv_bfloat16, float);
  } else {
    return B200_BAD_DTYPE;
  }
#undef B200_NORM_ADD
  return b200_check_launch();
}

B200_EXPORT int b200_norm_rows(void* out, int out_dtype, const float* x, const int* rows, const float* w, float eps,
                               int n, int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  if (out_dtype == B200_F32)
    norm_rows_kernel<float><<<n, PN_THREADS, 0, stream>>>(static_cast<float*>(out), x, rows, w, eps, width);
  else if (out_dtype == B200_BF16)
    norm_rows_kernel<__nv_bfloat16><<<n, PN_THREADS, 0, stream>>>(static_cast<__nv_bfloat16*>(out), x, rows, w, eps, width);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}
