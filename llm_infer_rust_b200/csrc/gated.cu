// Element-wise ends of gated mixers and of the PolyNorm feed-forward, all sums in float.
//
//   poly_norm            out = a N(z) + b N(z^2) + c N(z^3) + e,  N(y) = y / sqrt(mean(y^2) + eps) over a token's
//                        vector, powers taken element by element; (a, b, c, e) are four floats on the device
//   head_unit_norm_gate  out[t][h][:] = o[t][h][:] / sqrt(mean(o[t][h][:]^2) + eps) * silu(g[t][h][:])
//   sigmoid_gate_mul     out[t][c] = a[t][c] * sigmoid(g[t][c / per])   (per 1: a gate a column; a head's size: a gate a head)
//   activate_columns     x[t][c] <- act(x[t][c]) for the first `columns` columns of rows `stride` wide (in place), or
//                        out[t][c] = act(x[t][c]); act: 1 silu, 2 gelu with erf, 3 gelu with tanh
//   row_norm_gate        out[t][:] = o[t][:] / sqrt(mean(o[t][:]^2) + eps) * w[:] * sigmoid(g[t][:])   (o in float)
//   tanh_cap             z <- cap * tanh(z / cap) in place on floats
//
// `g` is a column range of a wider matrix (row stride g_stride), so a gate that was projected together with
// other things is read where it lies.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(T* __restrict__ out, const T* __restrict__ z, const float* __restrict__ coef, float eps, int width) {
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(z[base + c]);
    const float v2 = v * v, v3 = v2 * v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float n = static_cast<float>(width);
  const float r1 = coef[0] / sqrtf(s2 / n + eps), r2 = coef[1] / sqrtf(s4 / n + eps), r3 = coef[2] / sqrtf(s6 / n + eps);
  const float e = coef[3];
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(z[base + c]);
    const float v2 = v * v;
    out[base + c] = from_f32<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))));
  }
}

// The same for rows of whole 16-byte pieces: eight elements a thread and turn; a row of up to 8,192 elements
// stays in registers between the sums and the result.
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_vec_kernel(T* __restrict__ out, const T* __restrict__ z, const float* __restrict__ coef, float eps, int width) {
  __shared__ float scratch[33];
  constexpr int KEEP = 4;
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float kept[KEEP][8];
  float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
  int turn = 0;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8, ++turn) {
    float v[8];
    load_floats<T, 8>(z + base + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v2 = v[i] * v[i], v3 = v2 * v[i];
      s2 += v2;
      s4 = fmaf(v2, v2, s4);
      s6 = fmaf(v3, v3, s6);
    }
#pragma unroll
    for (int k = 0; k < KEEP; ++k)
      if (k == turn) {
#pragma unroll
        for (int i = 0; i < 8; ++i) kept[k][i] = v[i];
      }
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float n = static_cast<float>(width);
  const float r1 = coef[0] / sqrtf(s2 / n + eps), r2 = coef[1] / sqrtf(s4 / n + eps), r3 = coef[2] / sqrtf(s6 / n + eps);
  const float e = coef[3];
  turn = 0;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8, ++turn) {
    float v[8];
    bool have = false;
#pragma unroll
    for (int k = 0; k < KEEP; ++k)
      if (k == turn) {
        have = true;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = kept[k][i];
      }
    if (!have) load_floats<T, 8>(z + base + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v2 = v[i] * v[i];
      v[i] = fmaf(r1, v[i], fmaf(r2, v2, fmaf(r3, v2 * v[i], e)));
    }
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(out + base + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(out + base + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint4 u;
      __nv_bfloat162 h;
      h = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&h);
      *reinterpret_cast<uint4*>(out + base + c) = u;
    }
  }
}

// one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
head_unit_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ g, int g_stride,
                           int heads, int dv, float eps, long long vectors) {
  const long long vec = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (vec >= vectors) return;
  const int lane = threadIdx.x & 31;
  const long long t = vec / heads;
  const int h = static_cast<int>(vec - t * heads);
  const float* src = o + (t * heads + h) * dv;
  float ss = 0.0f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(src[j], src[j], ss);
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
  const T* gate = g + t * g_stride + static_cast<size_t>(h) * dv;
  T* dst = out + (t * heads + h) * dv;
  for (int j = lane; j < dv; j += 32) {
    const float x = to_f32<T>(gate[j]);
    dst[j] = from_f32<T>(src[j] * r * (x / (1.0f + expf(-x))));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_mul_kernel(T* out, const T* a, const T* __restrict__ g, int g_stride, int width, int per) {   // out may be a
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_f32<T>(g[t * g_stride + (per == 1 ? c : c / per)]);
    out[t * width + c] = from_f32<T>(to_f32<T>(a[t * width + c]) / (1.0f + expf(-x)));
  }
}

B200_EXPORT int b200_poly_norm(void* out, const void* z, const float* coef, float eps, int tokens, int width,
                               int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  if (width % 8 == 0 && (reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(z)) % 16 == 0 &&
      (dtype == B200_F32 || dtype == B200_BF16)) {
    if (dtype == B200_F32)
      poly_norm_vec_kernel<float><<<tokens, 256, 0, stream>>>(static_cast<float*>(out), static_cast<const float*>(z),
                                                              coef, eps, width);
    else
      poly_norm_vec_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
          static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(z), coef, eps, width);
    return b200_check_launch();
  }
  if (dtype == B200_F32)
    poly_norm_kernel<float><<<tokens, 256, 0, stream>>>(static_cast<float*>(out), static_cast<const float*>(z), coef,
                                                        eps, width);
  else if (dtype == B200_BF16)
    poly_norm_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(out),
                                                                static_cast<const __nv_bfloat16*>(z), coef, eps, width);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

B200_EXPORT int b200_head_unit_norm_gate(void* out, const float* o, const void* g, int g_stride, int tokens, int heads,
                                         int dv, float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || dv <= 0) return B200_BAD_SIZE;
  const long long vectors = static_cast<long long>(tokens) * heads;
  const unsigned blocks = static_cast<unsigned>((vectors + 3) / 4);
  if (dtype == B200_F32)
    head_unit_norm_gate_kernel<float><<<blocks, 128, 0, stream>>>(static_cast<float*>(out), o,
                                                                   static_cast<const float*>(g), g_stride, heads, dv, eps,
                                                                   vectors);
  else if (dtype == B200_BF16)
    head_unit_norm_gate_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), o, static_cast<const __nv_bfloat16*>(g), g_stride, heads, dv, eps, vectors);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

B200_EXPORT int b200_sigmoid_gate_mul(void* out, const void* a, const void* g, int g_stride, int tokens, int width,
                                      int per, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || per <= 0 || width % per) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return b200_launch(sigmoid_gate_mul_kernel<float>, dim3(tokens), dim3(256), 0, stream, 0, static_cast<float*>(out),
                       static_cast<const float*>(a), static_cast<const float*>(g), g_stride, width, per);
  if (dtype == B200_BF16)
    return b200_launch(sigmoid_gate_mul_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, 0,
                       static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(a),
                       static_cast<const __nv_bfloat16*>(g), g_stride, width, per);
  return B200_BAD_DTYPE;
}

// ------------------------------------------------------------------ activations, a joint norm with a gate, a cap
enum : int { ACT_SILU = 1, ACT_GELU_ERF = 2, ACT_GELU_TANH = 3, ACT_RELU_SQUARED = 4 };

__device__ __forceinline__ float activate(float z, int act) {
  if (act == ACT_SILU) return z / (1.0f + expf(-z));
  if (act == ACT_GELU_ERF) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (act == ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (act == ACT_RELU_SQUARED) { const float r = fmaxf(z, 0.0f); return r * r; }
  return z;
}

template <typename T>
__global__ void __launch_bounds__(256)
activate_columns_kernel(T* out, int out_stride, const T* x, int stride, int columns, int act) {   // out may be x
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < columns) out[t * out_stride + c] = from_f32<T>(activate(to_f32<T>(x[t * stride + c]), act));
}

// the same, eight elements a thread with 16-byte accesses (rows and column counts of whole 16-byte pieces)
template <typename T>
__global__ void __launch_bounds__(256)
activate_columns_vec_kernel(T* out, int out_stride, const T* x, int stride, int columns, int act) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= columns) return;
  float v[8];
  load_floats<T, 8>(x + t * stride + c, v);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = activate(v[i], act);
  T* dst = out + t * out_stride + c;
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 u;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(dst) = u;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
row_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                     const T* __restrict__ g, int g_stride, int width, float eps) {
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const float* src = o + t * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_f32<T>(g[t * g_stride + c]);
    out[t * width + c] = from_f32<T>(src[c] * r * w[c] / (1.0f + expf(-x)));
  }
}

__global__ void __launch_bounds__(256) tanh_cap_kernel(float* z, long long n, float cap) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

B200_EXPORT int b200_activate_columns(void* out, int out_stride, const void* x, int stride, int tokens, int columns,
                                      int act, int dtype, cudaStream_t stream) {
  int launch_rc = 0;
  if (tokens <= 0 || columns <= 0) return 0;
  if (act < ACT_SILU || act > ACT_RELU_SQUARED || stride < columns || out_stride < columns) return B200_BAD_SIZE;
  if (columns % 8 == 0 && stride % 8 == 0 && out_stride % 8 == 0 && (dtype == B200_F32 || dtype == B200_BF16) &&
      (reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) % 32 == 0) {
    const dim3 vgrid(tokens, (columns / 8 + 255) / 256);
    if (dtype == B200_F32)
      launch_rc = b200_launch(activate_columns_vec_kernel<float>, dim3(vgrid), dim3(256), 0, stream, 0, static_cast<float*>(out), out_stride,
                                                                    static_cast<const float*>(x), stride, columns, act);
    else
      launch_rc = b200_launch(activate_columns_vec_kernel<__nv_bfloat16>, dim3(vgrid), dim3(256), 0, stream, 0, 
          static_cast<__nv_bfloat16*>(out), out_stride, static_cast<const __nv_bfloat16*>(x), stride, columns, act);
    return launch_rc;
  }
  const dim3 grid(tokens, (columns + 255) / 256);
  if (dtype == B200_F32)
    launch_rc = b200_launch(activate_columns_kernel<float>, dim3(grid), dim3(256), 0, stream, 0, static_cast<float*>(out), out_stride,
                                                             static_cast<const float*>(x), stride, columns, act);
  else if (dtype == B200_BF16)
    launch_rc = b200_launch(activate_columns_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, 0, 
        static_cast<__nv_bfloat16*>(out), out_stride, static_cast<const __nv_bfloat16*>(x), stride, columns, act);
  else
    return B200_BAD_DTYPE;
  return launch_rc;
}

B200_EXPORT int b200_row_norm_gate(void* out, const float* o, const float* w, const void* g, int g_stride, int tokens,
                                   int width, float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    row_norm_gate_kernel<float><<<tokens, 256, 0, stream>>>(static_cast<float*>(out), o, w,
                                                            static_cast<const float*>(g), g_stride, width, eps);
  else if (dtype == B200_BF16)
    row_norm_gate_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), o, w, static_cast<const __nv_bfloat16*>(g), g_stride, width, eps);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

B200_EXPORT int b200_tanh_cap(float* z, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.0f)) return B200_BAD_SIZE;
  tanh_cap_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(z, n, cap);
  return b200_check_launch();
}

// ------------------------------------------------------------------ gate and up joined; an activation times a table row
// out[t][c] = glu(gate_up[t][c], gate_up[t][ff + c]).  kind 0: silu(g) u.  kind 1: g' sigmoid(alpha g') (u' + 1) with
// g' = min(g, limit), u' = clamp(u, -limit, limit).  Computed in float, rounded once.
__device__ __forceinline__ float glu_join(float g, float u, int kind, float limit, float alpha) {
  if (kind == 0) return g / (1.0f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename T>
__global__ void __launch_bounds__(256)
glu_columns_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int ff, int kind, float limit, float alpha) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= ff) return;
  const float g = to_f32<T>(gate_up[t * 2 * ff + c]), u = to_f32<T>(gate_up[t * 2 * ff + ff + c]);
  out[t * ff + c] = from_f32<T>(glu_join(g, u, kind, limit, alpha));
}

// The same eight columns a thread, for ff a multiple of eight (every row piece starts on 16 bytes): 16-byte loads
// and stores.  grid (tokens, ceil(ff / 2048)).
template <typename T>
__global__ void __launch_bounds__(256)
glu_columns_vec_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int ff, int kind, float limit, float alpha) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= ff) return;
  float g[8], u[8], r[8];
  load_floats<T, 8>(gate_up + t * 2 * ff + c, g);
  load_floats<T, 8>(gate_up + t * 2 * ff + ff + c, u);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = glu_join(g[i], u[i], kind, limit, alpha);
  T* dst = out + t * ff + c;
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(r[4], r[5], r[6], r[7]);
  } else {
    __nv_bfloat162 p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
  }
}

// out[t][c] = act(z[t][c]) * table[ids[t]][column + c]: a gate on a token's row of a second embedding table.
// An id outside the table sets the error bit and reads row 0.
template <typename T>
__global__ void __launch_bounds__(128)
act_table_mul_kernel(T* __restrict__ out, const T* __restrict__ z, const T* __restrict__ table, const int* __restrict__ ids,
                     int vocab, int table_width, int column, int dim, int act, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, B200_ERR_TOKEN_RANGE);
    id = 0;
  }
  const T* row = table + static_cast<size_t>(id) * table_width + column;
  for (int c = threadIdx.x; c < dim; c += blockDim.x)
    out[t * dim + c] = from_f32<T>(activate(to_f32<T>(z[t * dim + c]), act) * to_f32<T>(row[c]));
}

B200_EXPORT int b200_glu_columns(void* out, const void* gate_up, int tokens, int ff, int kind, float limit, float alpha,
                                 int dtype, cudaStream_t stream) {
  int launch_rc = 0;
  if (tokens <= 0 || ff <= 0) return 0;
  if (kind < 0 || kind > 1) return B200_BAD_SIZE;
  if (ff % 8 == 0) {
    const dim3 wide(tokens, (ff / 8 + 255) / 256);
    if (dtype == B200_F32)
      launch_rc = b200_launch(glu_columns_vec_kernel<float>, dim3(wide), dim3(256), 0, stream, 0, static_cast<float*>(out),
                                                              static_cast<const float*>(gate_up), ff, kind, limit, alpha);
    else if (dtype == B200_BF16)
      launch_rc = b200_launch(glu_columns_vec_kernel<__nv_bfloat16>, dim3(wide), dim3(256), 0, stream, 0, 
          static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), ff, kind, limit, alpha);
    else
      return B200_BAD_DTYPE;
    return launch_rc;
  }
  const dim3 grid(tokens, (ff + 255) / 256);
  if (dtype == B200_F32)
    launch_rc = b200_launch(glu_columns_kernel<float>, dim3(grid), dim3(256), 0, stream, 0, static_cast<float*>(out), static_cast<const float*>(gate_up), ff,
                                                        kind, limit, alpha);
  else if (dtype == B200_BF16)
    launch_rc = b200_launch(glu_columns_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, 0, 
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), ff, kind, limit, alpha);
  else
    return B200_BAD_DTYPE;
  return launch_rc;
}

B200_EXPORT int b200_act_table_mul(void* out, const void* z, const void* table, const int* ids, int tokens, int vocab,
                                   int table_width, int column, int dim, int act, int dtype, int* err,
                                   cudaStream_t stream) {
  int launch_rc = 0;
  if (tokens <= 0 || dim <= 0) return 0;
  if (act < ACT_SILU || act > ACT_RELU_SQUARED || vocab <= 0 || column < 0 || column + dim > table_width)
    return B200_BAD_SIZE;
  if (dtype == B200_F32)
    launch_rc = b200_launch(act_table_mul_kernel<float>, dim3(tokens), dim3(128), 0, stream, 0, static_cast<float*>(out), static_cast<const float*>(z),
                                                            static_cast<const float*>(table), ids, vocab, table_width,
                                                            column, dim, act, err);
  else if (dtype == B200_BF16)
    launch_rc = b200_launch(act_table_mul_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, 0, 
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(table),
        ids, vocab, table_width, column, dim, act, err);
  else
    return B200_BAD_DTYPE;
  return launch_rc;
}

// The whole gated read of a second token table for a step of few tokens, one cluster of SIDE_CLUSTER blocks a token,
// where four launches would each move a few kilobytes:
//   z = Wg x (rounded to T);  g = act(z) * table[id][column ..] (rounded to T);  y = Wp g (float)
//   stream <- stream + y / sqrt(mean(y^2) + eps) * norm;   cast_out <- the new stream rounded to T (if given)
// x [tokens, width] is the stream rounded to T (the stream itself in float32: every block has read it before the
// first barrier of the cluster, and writes come after the second).  Wg [dim, width], Wp [width, dim].
// Block r of the cluster takes rows r, r + SIDE_CLUSTER, .. of Wg (a warp a row, its lanes eight columns each and
// then 256 further on, in order) and sends each g to every block's shared memory; then it takes its slice of the
// columns of y (a thread a row of Wp), sends its part of the sum of squares to every block, and all add the parts in
// the order of the blocks.  Shared memory: dim + slice floats.
constexpr int SIDE_THREADS = 256, SIDE_CLUSTER = 8;

template <typename T>
__global__ void __launch_bounds__(SIDE_THREADS)
token_side_few_kernel(float* stream, const T* x, const T* __restrict__ gate, const T* __restrict__ table,
                      const int* __restrict__ ids, const T* __restrict__ proj, const float* __restrict__ norm_w,
                      float eps, T* __restrict__ cast_out, int vocab, int table_width, int column, int dim, int width,
                      int slice, int act, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  constexpr int NW = SIDE_THREADS / 32;
  __shared__ float warp_part[NW];
  __shared__ float part[SIDE_CLUSTER];
  extern __shared__ float side_sm[];
  float* g = side_sm;                                // dim
  float* y = side_sm + dim;                          // slice
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const size_t t = blockIdx.x / SIDE_CLUSTER;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && rank == 0) atomicOr(err, B200_ERR_TOKEN_RANGE);
    id = 0;
  }
  const T* e = table + static_cast<size_t>(id) * table_width + column;
  const T* xr = x + t * width;
  const bool wide = width % 8 == 0;
  cluster.sync();                                    // every block of the cluster runs: its shared memory can be written
  for (int j = rank + SIDE_CLUSTER * warp; j < dim; j += SIDE_CLUSTER * NW) {
    const T* w = gate + static_cast<size_t>(j) * width;
    float acc = 0.0f;
    if (wide) {
#pragma unroll 4
      for (int k = lane * 8; k < width; k += 256) {
        float a[8], b[8];
        load_floats<T, 8>(w + k, a);
        load_floats<T, 8>(xr + k, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
      }
    } else {
      for (int k8 = lane * 8; k8 < width; k8 += 256) {
        const int end = min(k8 + 8, width);
        for (int k = k8; k < end; ++k) acc = fmaf(to_f32<T>(w[k]), to_f32<T>(xr[k]), acc);
      }
    }
    acc = warp_sum(acc);
    const float z = to_f32<T>(from_f32<T>(acc));
    const float gj = to_f32<T>(from_f32<T>(activate(z, act) * to_f32<T>(e[j])));
    if (lane < SIDE_CLUSTER) *cluster.map_shared_rank(&g[j], lane) = gj;
  }
  cluster.sync();
  const int lo = rank * slice, hi = min(width, lo + slice);
  float ss = 0.0f;
  const bool wide_dim = dim % 8 == 0;
  for (int c = lo + threadIdx.x; c < hi; c += SIDE_THREADS) {
    const T* w = proj + static_cast<size_t>(c) * dim;
    float acc = 0.0f;
    if (wide_dim) {
#pragma unroll 4
      for (int k = 0; k < dim; k += 8) {
        float a[8];
        load_floats<T, 8>(w + k, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(a[i], g[k + i], acc);
      }
    } else {
      for (int k = 0; k < dim; ++k) acc = fmaf(to_f32<T>(w[k]), g[k], acc);
    }
    y[c - lo] = acc;
    ss = fmaf(acc, acc, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (threadIdx.x < SIDE_CLUSTER) {
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < NW; ++i) mine += warp_part[i];
    *cluster.map_shared_rank(&part[rank], threadIdx.x) = mine;
  }
  cluster.sync();
  ss = 0.0f;
#pragma unroll
  for (int i = 0; i < SIDE_CLUSTER; ++i) ss += part[i];
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  float* sr = stream + t * width;
  for (int c = lo + threadIdx.x; c < hi; c += SIDE_THREADS) {
    const float s = sr[c] + y[c - lo] * r * norm_w[c];
    sr[c] = s;
    if (cast_out != nullptr) cast_out[t * width + c] = from_f32<T>(s);
  }
}

// dtype: of x, gate, table, proj and cast_out (null: none is written; in float32 x may be the stream itself).
B200_EXPORT int b200_token_side_few(float* stream, const void* x, const void* gate, const void* table, const int* ids,
                                    const void* proj, const float* norm_w, float eps, void* cast_out, int tokens,
                                    int vocab, int table_width, int column, int dim, int width, int act, int dtype,
                                    int* err, cudaStream_t stream_) {
  if (tokens <= 0) return 0;
  if (act < ACT_SILU || act > ACT_RELU_SQUARED || vocab <= 0 || dim <= 0 || width <= 0 || column < 0 ||
      column + dim > table_width)
    return B200_BAD_SIZE;
  const int slice = (width + SIDE_CLUSTER - 1) / SIDE_CLUSTER;
  const size_t smem = (static_cast<size_t>(dim) + slice) * sizeof(float);
  if (smem > 200 * 1024) return B200_BAD_SIZE;
#define B200_SIDE(T)                                                                                               \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(token_side_few_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                           static_cast<int>(smem));                                                \
      if (e != cudaSuccess) return static_cast<int>(e);                                                            \
    }                                                                                                              \
    const int rc = b200_launch(token_side_few_kernel<T>, dim3(tokens * SIDE_CLUSTER), dim3(SIDE_THREADS), smem,    \
                               stream_, SIDE_CLUSTER, stream, static_cast<const T*>(x), static_cast<const T*>(gate), \
                               static_cast<const T*>(table), ids, static_cast<const T*>(proj), norm_w, eps,        \
                               static_cast<T*>(cast_out), vocab, table_width, column, dim, width, slice, act, err); \
    if (rc != 0) return rc;                                                                                        \
  } while (0)
  if (dtype == B200_F32) B200_SIDE(float);
  else if (dtype == B200_BF16) B200_SIDE(__nv_bfloat16);
  else return B200_BAD_DTYPE;
#undef B200_SIDE
  return b200_check_launch();
}

// y[t][c] += bias[c], the sum taken in float and rounded once (a projection's bias where nothing else can take it).
template <typename T>
__global__ void __launch_bounds__(256) add_row_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, int width) {
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    y[t * width + c] = from_f32<T>(to_f32<T>(y[t * width + c]) + bias[c]);
}

B200_EXPORT int b200_add_row_bias(void* y, const float* bias, int tokens, int width, int dtype, cudaStream_t stream) {
  if (tokens <= 0 || width <= 0) return 0;
  if (dtype == B200_F32) add_row_bias_kernel<float><<<tokens, 256, 0, stream>>>(static_cast<float*>(y), bias, width);
  else if (dtype == B200_BF16)
    add_row_bias_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(y), bias, width);
  else return B200_BAD_DTYPE;
  return b200_check_launch();
}
