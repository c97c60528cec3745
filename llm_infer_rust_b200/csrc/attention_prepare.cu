// What stands between a packed projection and attention, for two kinds of mixer.  One warp owns one vector of a
// token; values are read once, worked on in float in shared memory and rounded once when stored.
//
// (1) heads_prepare: grouped-query attention whose keys are `d` wide and whose values are `dv` wide.  The packed
//     row holds q (nh * d), k (nkv * d), v (nkv * dv) from column 0.  Optional, in this order: a bias per column;
//     a per-head RMS norm of q and of k (x / sqrt(mean(x^2) + eps) * w, one weight vector for all heads);
//     a rotation of the first rot_dims coordinates of every q and k head.  q goes to q_out [tokens, nh * d], k and
//     v to the paged cache at the token's slot.  `flags`: PREP_NORM_PLAIN: q and k are normed without a weight
//     (x / sqrt(mean(x^2) + eps)); PREP_NORM_AFTER_ROTATION: the norm follows the rotation instead of preceding it;
//     PREP_VALUES_ARE_KEYS: the row holds no v columns and a token's value is its key as projected (with its bias,
//     before norm and rotation; dv = d).
//
// (2) latent_prepare: attention over a narrow latent.  The packed row holds per head [d plain | r rotated] query
//     coordinates (nh * (d + r)), and a second row (`down`, which may be a column range of the same matrix or of
//     another one) the down projection [c_dim latent | r rotated key part].  The latent is
//     RMS-normed (weight w_c) and, with the rotated key part behind it, is the ONE key of the token
//     (c_dim + r wide, shared by all heads); the latent alone is its value (stored a second time only if a value cache
//     is given: attention can read it out of the key rows).  The query against that key is
//     [q_lat (c_dim) | rotated (r)], where q_lat[h] = W_uk[h]^T q_plain[h] was multiplied before
//     (q_lat: [nh, tokens, c_dim]), since q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c.
//
// (3) joint_heads_prepare: as (1), but the RMS norm of q runs over ALL of the token's q columns at once (nh * d, before
//     they are split into heads; weights of that size), and so does the norm of k (nkv * d).  One block a token.  A
//     layer that reads another layer's keys and values has only the q columns (`has_kv` 0) and stores nothing.
//
// Rotation: the pair (u, v) of a token at position p becomes (u cos a - v sin a, v cos a + u sin a) with
// a = p * inv_freq[i] in float; pairs are (2i, 2i + 1) (`interleaved`) or (i, i + rot_dims / 2).
// A slot outside the pool sets an error bit and the store is skipped; slot 0 (padding rows) stores nothing.
#include "common.cuh"

constexpr int MAX_VEC = 1024;       // widest vector a warp takes
constexpr int WARPS = 4;
enum : int { PREP_NORM_PLAIN = 1, PREP_NORM_AFTER_ROTATION = 2, PREP_VALUES_ARE_KEYS = 4 };

__device__ __forceinline__ void rotate_row(float* row, int rot_dims, float pos, const float* __restrict__ inv_freq,
                                           bool interleaved, int lane) {
  const int half = rot_dims >> 1;
  for (int i = lane; i < half; i += 32) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const float u = row[a], v = row[b];
    row[a] = u * cs - v * sn;
    row[b] = v * cs + u * sn;
  }
}

// cache[page][kv head][offset in page][width]: the row of `slot` for KV head kvh, or null (with the error bit set
// for a slot outside the pool)
template <typename T>
__device__ __forceinline__ T* cache_row(T* cache, int slot, int kvh, int nkv, int page_size, long long cache_slots,
                                        int width, int lane, int* err) {
  if (slot == 0) return nullptr;
  if (slot < 0 || slot >= cache_slots) {
    if (lane == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
    return nullptr;
  }
  const int page = slot / page_size, offset = slot - page * page_size;
  return cache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * width;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
heads_prepare_kernel(const T* __restrict__ x, int in_stride, const float* __restrict__ bias,
                     const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                     const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                     const int* __restrict__ positions, const int* __restrict__ slots, int tokens, int nh, int nkv,
                     int d, int dv, int flags, int page_size, long long cache_slots, T* __restrict__ q_out,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  __shared__ float buf[WARPS][MAX_VEC];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vectors = nh + 2 * nkv;
  const bool v_is_k = (flags & PREP_VALUES_ARE_KEYS) != 0;
  const long long work = static_cast<long long>(blockIdx.x) * WARPS + warp;
  if (work >= static_cast<long long>(tokens) * vectors) return;
  const int t = static_cast<int>(work / vectors);
  const int h = static_cast<int>(work - static_cast<long long>(t) * vectors);
  const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
  const int kvh = is_q ? 0 : (is_k ? h - nh : h - nh - nkv);
  const int width = (is_q || is_k) ? d : dv;
  const int col = is_q ? h * d : ((is_k || v_is_k) ? nh * d + kvh * d : (nh + nkv) * d + kvh * dv);
  T* dst;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(t) * nh + h) * d;
  } else {
    if (slots == nullptr) return;
    dst = cache_row(is_k ? k_cache : v_cache, slots[t], kvh, nkv, page_size, cache_slots, width, lane, err);
    if (dst == nullptr) return;
  }
  const T* src = x + static_cast<size_t>(t) * in_stride + col;
  float* row = buf[warp];
  float ss = 0.0f;
  for (int i = lane; i < width; i += 32) {
    float v = to_f32<T>(src[i]);
    if (bias != nullptr) v += bias[col + i];
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
  const bool normed = (is_q || is_k) && (w != nullptr || (flags & PREP_NORM_PLAIN) != 0);
  const bool rotated = (is_q || is_k) && inv_freq != nullptr && rot_dims > 0;
  const bool norm_last = (flags & PREP_NORM_AFTER_ROTATION) != 0;
  if (normed && !norm_last) {
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
    for (int i = lane; i < width; i += 32) row[i] = w != nullptr ? row[i] * r * w[i] : row[i] * r;
  }
  __syncwarp();
  if (rotated) {
    rotate_row(row, rot_dims, static_cast<float>(positions[t]), inv_freq, interleaved != 0, lane);
    __syncwarp();
  }
  if (normed && norm_last) {
    ss = 0.0f;                                       // of the rotated row: the same sum up to rounding, taken as written
    for (int i = lane; i < width; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
    for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>(w != nullptr ? row[i] * r * w[i] : row[i] * r);
    return;
  }
  for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>(row[i]);
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_prepare_kernel(const T* __restrict__ x, int in_stride, const T* __restrict__ down, int down_stride,
                      const T* __restrict__ q_lat,
                      const float* __restrict__ w_c, float eps, const float* __restrict__ inv_freq, int rot_dims,
                      int interleaved, const int* __restrict__ positions, const int* __restrict__ slots, int tokens,
                      int nh, int d, int r, int c_dim, int page_size, long long cache_slots, T* __restrict__ q_out,
                      T* __restrict__ k_cache, T* __restrict__ v_cache, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  __shared__ float buf[WARPS][MAX_VEC];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vectors = nh + 1;
  const long long work = static_cast<long long>(blockIdx.x) * WARPS + warp;
  if (work >= static_cast<long long>(tokens) * vectors) return;
  const int t = static_cast<int>(work / vectors);
  const int h = static_cast<int>(work - static_cast<long long>(t) * vectors);
  const float pos = static_cast<float>(positions[t]);
  float* row = buf[warp];
  if (h < nh) {
    // a query head: its latent part was multiplied before; its rotated part is turned here
    const T* src = x + static_cast<size_t>(t) * in_stride + static_cast<size_t>(h) * (d + r) + d;
    for (int i = lane; i < r; i += 32) row[i] = to_f32<T>(src[i]);
    __syncwarp();
    if (inv_freq != nullptr && rot_dims > 0) {
      rotate_row(row, rot_dims, pos, inv_freq, interleaved != 0, lane);
      __syncwarp();
    }
    T* dst = q_out + (static_cast<size_t>(t) * nh + h) * (c_dim + r);
    const T* lat = q_lat + (static_cast<size_t>(h) * tokens + t) * c_dim;
    for (int i = lane; i < c_dim; i += 32) dst[i] = lat[i];
    for (int i = lane; i < r; i += 32) dst[c_dim + i] = from_f32<T>(row[i]);
    return;
  }
  // the down projection: the normed latent and the rotated key part that all heads share
  if (slots == nullptr) return;
  const T* src = down + static_cast<size_t>(t) * down_stride;
  float ss = 0.0f;
  for (int i = lane; i < c_dim + r; i += 32) {
    const float v = to_f32<T>(src[i]);
    row[i] = v;
    if (i < c_dim) ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float rs = 1.0f / sqrtf(ss / static_cast<float>(c_dim) + eps);
  for (int i = lane; i < c_dim; i += 32) row[i] = row[i] * rs * w_c[i];
  __syncwarp();
  if (inv_freq != nullptr && rot_dims > 0) {
    rotate_row(row + c_dim, rot_dims, pos, inv_freq, interleaved != 0, lane);
    __syncwarp();
  }
  const int slot = slots[t];
  T* kd = cache_row(k_cache, slot, 0, 1, page_size, cache_slots, c_dim + r, lane, err);
  if (kd == nullptr) return;
  for (int i = lane; i < c_dim + r; i += 32) kd[i] = from_f32<T>(row[i]);
  if (v_cache != nullptr) {                          // a cache that keeps the values apart (else they are read from the key rows)
    T* vd = cache_row(v_cache, slot, 0, 1, page_size, cache_slots, c_dim, lane, err);
    for (int i = lane; i < c_dim; i += 32) vd[i] = from_f32<T>(row[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
joint_heads_prepare_kernel(const T* __restrict__ x, int in_stride, const float* __restrict__ bias,
                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                           const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                           const int* __restrict__ positions, const int* __restrict__ slots, int nh, int nkv, int d,
                           int dv, int has_kv, int page_size, long long cache_slots, T* __restrict__ q_out,
                           T* __restrict__ k_cache, T* __restrict__ v_cache, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  __shared__ float sums[2][32];
  extern __shared__ float jrow[];                    // q (nh * d), then k (nkv * d), then v (nkv * dv), then cos, sin
  const int t = blockIdx.x;
  const int nq = nh * d, nk = has_kv ? nkv * d : 0, nv = has_kv ? nkv * dv : 0;
  const T* src = x + static_cast<size_t>(t) * in_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  // the token's angles once for all heads (read after the barrier below)
  const bool rotate = inv_freq != nullptr && rot_dims > 0;
  const int half = rot_dims >> 1;
  float* cos_t = jrow + nq + nk + nv;
  float* sin_t = cos_t + half;
  if (rotate) {
    const float pos = static_cast<float>(positions[t]);
    for (int p = threadIdx.x; p < half; p += blockDim.x) sincosf(pos * inv_freq[p], &sin_t[p], &cos_t[p]);
  }
  // every size is even: the row is read two columns at a time where it starts on a pair
  const bool paired = (in_stride & 1) == 0 && (reinterpret_cast<uintptr_t>(x) & (2 * sizeof(T) - 1)) == 0;
  float ssq = 0.0f, ssk = 0.0f;
#pragma unroll 4
  for (int i = 2 * threadIdx.x; i < nq + nk + nv; i += 2 * blockDim.x) {
    float v0, v1;
    if (paired) {
      if constexpr (sizeof(T) == 4) {
        const float2 p = *reinterpret_cast<const float2*>(src + i);
        v0 = p.x; v1 = p.y;
      } else {
        const uint32_t p = *reinterpret_cast<const uint32_t*>(src + i);
        v0 = __uint_as_float(p << 16); v1 = __uint_as_float(p & 0xffff0000u);
      }
    } else {
      v0 = to_f32<T>(src[i]); v1 = to_f32<T>(src[i + 1]);
    }
    if (bias != nullptr) { v0 += bias[i]; v1 += bias[i + 1]; }
    jrow[i] = v0;
    jrow[i + 1] = v1;
    const float sq = fmaf(v1, v1, v0 * v0);
    if (i < nq) ssq += sq;
    else if (i < nq + nk) ssk += sq;
  }
  // both sums of squares through one pair of barriers; the additions' order is fixed by the thread layout
  ssq = warp_sum(ssq);
  ssk = warp_sum(ssk);
  if (lane == 0) { sums[0][warp] = ssq; sums[1][warp] = ssk; }
  __syncthreads();
  ssq = ssk = 0.0f;
  for (int w = 0; w < warps; ++w) { ssq += sums[0][w]; ssk += sums[1][w]; }
  const float rq = q_w != nullptr ? 1.0f / sqrtf(ssq / static_cast<float>(nq) + eps) : 1.0f;
  const float rk = (has_kv && k_w != nullptr) ? 1.0f / sqrtf(ssk / static_cast<float>(nk) + eps) : 1.0f;
  if (rotate && !interleaved) {
    // pairs (p, p + half) lie apart: norm in place, then the rotation, then the stores below read the row
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
      if (i < nq) { if (q_w != nullptr) jrow[i] = jrow[i] * rq * q_w[i]; }
      else if (k_w != nullptr) jrow[i] = jrow[i] * rk * k_w[i - nq];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (nh + (has_kv ? nkv : 0)) * half; i += blockDim.x) {
      const int h = i / half, p = i - h * half;
      float* row = jrow + h * d;                    // q heads, then k heads: all d wide and contiguous
      const float sn = sin_t[p], cs = cos_t[p];
      const float u = row[p], v = row[p + half];
      row[p] = u * cs - v * sn;
      row[p + half] = v * cs + u * sn;
    }
    __syncthreads();
  }
  const bool finish = !(rotate && !interleaved);    // norm and rotation of a neighbouring pair happen on the way out
  int slot = 0;
  if (has_kv && slots != nullptr) {
    slot = slots[t];
    if (slot < 0 || slot >= cache_slots) {
      if (threadIdx.x == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
      slot = 0;
    }
  }
  const int page = slot / page_size, offset = slot - page * page_size;
  T* qd = q_out + static_cast<size_t>(t) * nq;
#pragma unroll 2
  for (int i = 2 * threadIdx.x; i < nq + nk + nv; i += 2 * blockDim.x) {
    float v0 = jrow[i], v1 = jrow[i + 1];           // this thread's own pair in the interleaved form
    T* dst;
    if (i < nq + nk) {
      const bool is_q = i < nq;
      const int j = is_q ? i : i - nq;               // column within q or within k
      const int c = j % d;                           // column within the head
      if (finish) {
        const float* w = is_q ? q_w : k_w;
        if (w != nullptr) {
          const float r = is_q ? rq : rk;
          v0 = v0 * r * w[j];
          v1 = v1 * r * w[j + 1];
        }
        if (rotate && c < rot_dims) {
          const float sn = sin_t[c >> 1], cs = cos_t[c >> 1];
          const float u = v0, v = v1;
          v0 = u * cs - v * sn;
          v1 = v * cs + u * sn;
        }
      }
      if (is_q) {
        dst = qd + i;
      } else {
        if (slot == 0) continue;
        const int kvh = j / d;
        dst = k_cache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * d + c;
      }
    } else {
      if (slot == 0) continue;
      const int j = i - nq - nk, kvh = j / dv, c = j - kvh * dv;
      dst = v_cache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * dv + c;
    }
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
    }
  }
}


B200_EXPORT int b200_heads_prepare(const void* x, int dtype, int in_stride, const float* bias, const float* q_w,
                                   const float* k_w, float eps, const float* inv_freq, int rot_dims, int interleaved,
                                   const int* positions, const int* slots, int tokens, int nh, int nkv, int d, int dv,
                                   int flags, int page_size, long long cache_slots, void* q_out, void* k_cache,
                                   void* v_cache, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || d > MAX_VEC || dv > MAX_VEC || rot_dims < 0 || rot_dims > d ||
      (rot_dims & 1) || page_size <= 0 || ((flags & PREP_VALUES_ARE_KEYS) && dv != d))
    return B200_BAD_SIZE;
  const long long work = static_cast<long long>(tokens) * (nh + 2 * nkv);
  const unsigned blocks = static_cast<unsigned>((work + WARPS - 1) / WARPS);
  if (dtype == B200_F32)
    return b200_launch(heads_prepare_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
        static_cast<const float*>(x), in_stride, bias, q_w, k_w, eps, inv_freq, rot_dims, interleaved, positions, slots,
        tokens, nh, nkv, d, dv, flags, page_size, cache_slots, static_cast<float*>(q_out), static_cast<float*>(k_cache),
        static_cast<float*>(v_cache), err);
  else if (dtype == B200_BF16)
    return b200_launch(heads_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
        static_cast<const __nv_bfloat16*>(x), in_stride, bias, q_w, k_w, eps, inv_freq, rot_dims, interleaved,
        positions, slots, tokens, nh, nkv, d, dv, flags, page_size, cache_slots, static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), err);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

// x: the query rows (row stride in_stride); down: the down projection's rows [c_dim | r] (row stride down_stride).
B200_EXPORT int b200_latent_prepare(const void* x, int dtype, int in_stride, const void* down, int down_stride,
                                    const void* q_lat, const float* w_c,
                                    float eps, const float* inv_freq, int rot_dims, int interleaved,
                                    const int* positions, const int* slots, int tokens, int nh, int d, int r, int c_dim,
                                    int page_size, long long cache_slots, void* q_out, void* k_cache, void* v_cache,
                                    int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nh <= 0 || d <= 0 || r < 0 || c_dim <= 0 || c_dim + r > MAX_VEC || rot_dims < 0 || rot_dims > r ||
      (rot_dims & 1) || page_size <= 0)
    return B200_BAD_SIZE;
  const long long work = static_cast<long long>(tokens) * (nh + 1);
  const unsigned blocks = static_cast<unsigned>((work + WARPS - 1) / WARPS);
  if (dtype == B200_F32)
    return b200_launch(latent_prepare_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
        static_cast<const float*>(x), in_stride, static_cast<const float*>(down), down_stride,
        static_cast<const float*>(q_lat), w_c, eps, inv_freq, rot_dims,
        interleaved, positions, slots, tokens, nh, d, r, c_dim, page_size, cache_slots, static_cast<float*>(q_out),
        static_cast<float*>(k_cache), static_cast<float*>(v_cache), err);
  else if (dtype == B200_BF16)
    return b200_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
        static_cast<const __nv_bfloat16*>(x), in_stride, static_cast<const __nv_bfloat16*>(down), down_stride,
        static_cast<const __nv_bfloat16*>(q_lat), w_c, eps, inv_freq, rot_dims, interleaved, positions, slots, tokens,
        nh, d, r, c_dim, page_size, cache_slots,
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
        err);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

// (3): norms over the whole q and the whole k projection.  has_kv 0: x holds q columns only, nothing is stored.
B200_EXPORT int b200_joint_heads_prepare(const void* x, int dtype, int in_stride, const float* bias, const float* q_w,
                                         const float* k_w, float eps, const float* inv_freq, int rot_dims,
                                         int interleaved, const int* positions, const int* slots, int tokens, int nh,
                                         int nkv, int d, int dv, int has_kv, int page_size, long long cache_slots,
                                         void* q_out, void* k_cache, void* v_cache, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || rot_dims < 0 || rot_dims > d || (rot_dims & 1) || page_size <= 0 ||
      (d & 1) || (dv & 1))                            // columns are taken two at a time
    return B200_BAD_SIZE;
  const size_t smem = (static_cast<size_t>(nh) * d + (has_kv ? static_cast<size_t>(nkv) * (d + dv) : 0) + rot_dims) *
                      sizeof(float);
  const int threads = tokens <= 64 ? 1024 : 256;     // few tokens: more threads each, the step waits for the slowest
  if (smem > 200 * 1024) return B200_BAD_SIZE;
#define B200_JOINT(T)                                                                                               \
  do {                                                                                                              \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(joint_heads_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           static_cast<int>(smem));                                                 \
      if (e != cudaSuccess) return static_cast<int>(e);                                                             \
    }                                                                                                               \
    const int rc = b200_launch(joint_heads_prepare_kernel<T>, dim3(tokens), dim3(threads), smem, stream, 0,          \
        static_cast<const T*>(x), in_stride, bias, q_w, k_w, eps, inv_freq, rot_dims, interleaved, positions, slots, \
        nh, nkv, d, dv, has_kv, page_size, cache_slots, static_cast<T*>(q_out), static_cast<T*>(k_cache),           \
        static_cast<T*>(v_cache), err);                                                                             \
    if (rc != 0) return rc;                                                                                         \
  } while (0)
  if (dtype == B200_F32) B200_JOINT(float);
  else if (dtype == B200_BF16) B200_JOINT(__nv_bfloat16);
  else return B200_BAD_DTYPE;
#undef B200_JOINT
  return b200_check_launch();
}


// (4) columns_rms_norm: out[t][:] = x[t][0 .. width) / sqrt(mean(x^2) + eps) * w, the rows of x `in_stride` apart
//     (a column range of a wider projection), out contiguous.  One warp a row; sums in float in an order fixed by the
//     lane layout.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
columns_rms_norm_kernel(const T* __restrict__ x, int in_stride, const float* __restrict__ w, float eps, int tokens,
                        int width, T* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= tokens) return;
  const T* src = x + static_cast<size_t>(t) * in_stride;
  float ss = 0.0f;
  for (int i = lane; i < width; i += 32) {
    const float v = to_f32<T>(src[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  T* dst = out + static_cast<size_t>(t) * width;
  for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>(to_f32<T>(src[i]) * r * w[i]);
}

B200_EXPORT int b200_columns_rms_norm(const void* x, int dtype, int in_stride, const float* w, float eps, int tokens,
                                      int width, void* out, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || in_stride < width) return B200_BAD_SIZE;
  const unsigned blocks = (tokens + WARPS - 1) / WARPS;
  if (dtype == B200_F32)
    return b200_launch(columns_rms_norm_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
                       static_cast<const float*>(x), in_stride, w, eps, tokens, width, static_cast<float*>(out));
  if (dtype == B200_BF16)
    return b200_launch(columns_rms_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, stream, 0,
                       static_cast<const __nv_bfloat16*>(x), in_stride, w, eps, tokens, width,
                       static_cast<__nv_bfloat16*>(out));
  return B200_BAD_DTYPE;
}
