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

constexpr int PN_THREADS = 256, PN_MAX_THREADS = 1024;

template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&lo);
  v.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

// Up to PN_MAX_THREADS threads a block (the launcher gives a step of few tokens more threads each); a width that is a
// multiple of four is taken four columns at a time.
template <typename TY, typename TO>
__global__ void __launch_bounds__(PN_MAX_THREADS)
norm_add_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ bias,
                const float* __restrict__ w, float eps, TO* __restrict__ cast_out, int width) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  __shared__ float scratch[33];
  extern __shared__ float row[];                     // width floats: y + bias
  const size_t t = blockIdx.x;
  const TY* src = y + t * width;
  float* xr = x + t * width;
  float ss = 0.0f;
  if (width % 4 == 0) {
#pragma unroll 2
    for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
      float v[4];
      load_floats<TY, 4>(src + c, v);
      if (bias != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(bias + c);
        v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
      }
      *reinterpret_cast<float4*>(row + c) = make_float4(v[0], v[1], v[2], v[3]);
      ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
#pragma unroll 2
    for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
      const float4 a = *reinterpret_cast<const float4*>(xr + c);
      const float4 g = *reinterpret_cast<const float4*>(w + c);
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      const float s0 = a.x + v.x * r * g.x, s1 = a.y + v.y * r * g.y, s2 = a.z + v.z * r * g.z, s3 = a.w + v.w * r * g.w;
      *reinterpret_cast<float4*>(xr + c) = make_float4(s0, s1, s2, s3);
      if (cast_out != nullptr) store4<TO>(cast_out + t * width + c, s0, s1, s2, s3);
    }
    return;
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_f32<TY>(src[c]);
    if (bias != nullptr) v += bias[c];
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
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
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
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
  // a step of few tokens: as many threads a block as the row has groups of four columns, up to PN_MAX_THREADS
  const int threads = tokens <= 64 ? min(PN_MAX_THREADS, max(PN_THREADS, (width / 4 + 31) / 32 * 32)) : PN_THREADS;
#define B200_NORM_ADD(TY, TO)                                                                                  \
  do {                                                                                                         \
    if (smem > 48 * 1024) {                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(norm_add_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           static_cast<int>(smem));                                            \
      if (e != cudaSuccess) return static_cast<int>(e);                                                        \
    }                                                                                                          \
    const int rc = b200_launch(norm_add_kernel<TY, TO>, dim3(tokens), dim3(threads), smem, stream, 0, x,         \
                               static_cast<const TY*>(y), bias, w, eps, static_cast<TO*>(cast_out), width);     \
    if (rc != 0) return rc;                                                                                    \
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
    return b200_launch(norm_rows_kernel<float>, dim3(n), dim3(PN_THREADS), 0, stream, 0, static_cast<float*>(out), x, rows, w,
                       eps, width);
  else if (out_dtype == B200_BF16)
    return b200_launch(norm_rows_kernel<__nv_bfloat16>, dim3(n), dim3(PN_THREADS), 0, stream, 0,
                       static_cast<__nv_bfloat16*>(out), x, rows, w, eps, width);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}
