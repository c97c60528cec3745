// A mixture of small gated feed-forward experts.  A token's experts come from a table lookup (the row of its id in
// an integer table [vocab, top], each expert with weight 1 / top) or from a router (expert_router_kernel: 32-bit
// logits, softmax or sigmoid scores, the best groups of neighbouring experts, the top experts among them, each with
// its score as weight).
//
//   expert e:  y = W_down[e] glu(W_gate[e] x, W_up[e] x)          out[t] = sum_k weight_(t, k) y_(t, k) [+ add[t]]
//   glu(g, u) = silu(g) u,  or  g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)
//
// Four kernels behind the choice, nothing goes through the host (a step can be captured in a graph):
//   expert_route       (token, choice) pairs sorted by expert: sorted_token[pos], pos_of_pair[pair], the experts'
//                      ranges and the list of row tiles (expert, first row) that the products walk
//   expert_gate_up     H[pos] = glu(gate, up) for every sorted pair, rows of x gathered by token
//   expert_down        Y[pos] = W_down[e] H[pos], in float
//   expert_combine     out[t] = sum over k in order of weight(t, k) Y[pos_of_pair[t * top + k]] (+ add[t]), in float
//
// Weights: gate_up [experts, 2 * ff, width] (an expert's gate rows, then its up rows), down [experts, width, ff].
// float32: FFMA, every output accumulated over k in order (a pair's result does not depend on its place in a tile,
// so the order in which pairs of one expert were sorted does not show).  bfloat16: tensor cores with float
// accumulation, H rounded once to bfloat16; a step of at most 64 pairs (a decode step) takes expert_rows_few_kernel
// instead, which streams every weight row once for the few rows that need it.
#include <mma.h>

#include "common.cuh"

constexpr int TM = 64, TN = 64;      // rows (sorted pairs) and columns of a tile

// ------------------------------------------------------------------ routing
// The expert of pair i = token * top + k: the router's choice if there is one, else the table's entry for the token id
// (-1 for an id outside the table).
__device__ __forceinline__ int pair_expert(const int* __restrict__ token_ids, const int* __restrict__ table, int vocab,
                                           int top, const int* __restrict__ choice, int i) {
  if (choice != nullptr) return choice[i];
  const int id = token_ids[i / top];
  return (id >= 0 && id < vocab) ? table[static_cast<size_t>(id) * top + i % top] : -1;
}

// one block; shared memory: 2 * experts + 1 ints
__global__ void __launch_bounds__(1024)
expert_route_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int vocab, int top, int experts,
                    const int* __restrict__ choice, int tokens, int* __restrict__ sorted_token, int* __restrict__ pos_of_pair,
                    int* __restrict__ expert_start, int* __restrict__ tile_expert, int* __restrict__ tile_first,
                    int* __restrict__ num_tiles, int tile_rows, int* err) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  extern __shared__ int sm[];
  int* count = sm;                    // [experts]
  int* start = sm + experts;          // [experts + 1]
  const int pairs = tokens * top;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int e = pair_expert(token_ids, table, vocab, top, choice, i);
    if (e < 0 || e >= experts) { atomicOr(err, B200_ERR_TOKEN_RANGE); e = 0; }
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, n = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      expert_start[e] = at;
      for (int r = at; r < at + count[e]; r += tile_rows) { tile_expert[n] = e; tile_first[n] = r; ++n; }
      at += count[e];
    }
    start[experts] = at;
    expert_start[experts] = at;
    *num_tiles = n;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int e = pair_expert(token_ids, table, vocab, top, choice, i);
    if (e < 0 || e >= experts) e = 0;
    const int pos = start[e] + atomicAdd(&count[e], 1);
    sorted_token[pos] = i / top;
    pos_of_pair[i] = pos;
  }
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// What joins an expert's gate and up projections.  kind 0: silu(g) u.  kind 1: g' sigmoid(alpha g') (u' + 1) with
// g' = min(g, limit), u' = clamp(u, -limit, limit).
struct GluAct {
  int kind;
  float limit, alpha;
};
__device__ __forceinline__ float glu_f(float g, float u, const GluAct a) {
  if (a.kind == 0) return silu_f(g) * u;
  g = fminf(g, a.limit);
  u = fminf(fmaxf(u, -a.limit), a.limit);
  return g / (1.0f + expf(-a.alpha * g)) * (u + 1.0f);
}

// ------------------------------------------------------------------ float32 products
// GATED: C[pos][n] = silu(A . Wg[n]) * (A . Wu[n]) with A rows gathered by sorted_token; else C[pos][n] = A[pos] . W[n].
// grid (column tiles, row tiles); 256 threads, 4 x 4 outputs a thread; k in steps of 16.
template <bool GATED>
__global__ void __launch_bounds__(256)
expert_gemm_f32_kernel(const float* __restrict__ A, int lda, const int* __restrict__ gather,
                       const float* __restrict__ W, long long w_expert_stride, int up_row_offset,
                       float* __restrict__ C, int N, int K, const int* __restrict__ expert_start,
                       const int* __restrict__ tile_expert, const int* __restrict__ tile_first,
                       const int* __restrict__ num_tiles, const GluAct act) {
  constexpr int BK = 16;
  if (static_cast<int>(blockIdx.y) >= *num_tiles) return;
  __shared__ float As[BK][TM + 4];
  __shared__ float Ws[GATED ? 2 : 1][BK][TN + 4];
  const int e = tile_expert[blockIdx.y], r0 = tile_first[blockIdx.y];
  const int r_end = min(r0 + TM, expert_start[e + 1]);
  const int n0 = blockIdx.x * TN;
  const float* We = W + e * w_expert_stride;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int arow = r0 + lrow;
  const float* a_src = nullptr;
  if (arow < r_end) a_src = A + static_cast<size_t>(gather ? gather[arow] : arow) * lda;
  const int wn = n0 + lrow;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4], w[GATED ? 2 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k0 + lk + i;
      a[i] = (a_src != nullptr && kk < K) ? a_src[kk] : 0.0f;
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
        w[g][i] = (wn < N && kk < K) ? We[static_cast<size_t>(wn + g * up_row_offset) * K + kk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = a[i];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) Ws[g][lk + i][lrow] = w[g][i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) {
        const float4 wv = *reinterpret_cast<const float4*>(&Ws[g][k][tx * 4]);
        const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(ar[i], wr[j], acc[g][i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= r_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if constexpr (GATED) C[static_cast<size_t>(r) * N + n] = glu_f(acc[0][i][j], acc[1][i][j], act);
      else C[static_cast<size_t>(r) * N + n] = acc[0][i][j];
    }
  }
}

// ------------------------------------------------------------------ bfloat16 products on tensor cores
// The same tiles; 8 warps, warp w owns rows 16 * (w / 2) .. and columns 32 * (w % 2) .. of the tile (two 16 x 16
// accumulators, four when GATED); k in steps of 64 through shared memory, the next step's operands fetched into
// registers while the tensor cores work on this one (a decode step's products are a chain of such fetches: few rows
// an expert, all of its weights).  TO: bfloat16 (H) or float (Y).
template <bool GATED, typename TO>
__global__ void __launch_bounds__(256)
expert_gemm_bf16_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ gather,
                        const __nv_bfloat16* __restrict__ W, long long w_expert_stride, int up_row_offset,
                        TO* __restrict__ C, int N, int K, const int* __restrict__ expert_start,
                        const int* __restrict__ tile_expert, const int* __restrict__ tile_first,
                        const int* __restrict__ num_tiles, const GluAct act) {
  using namespace nvcuda;
  constexpr int BK = 64, LD = BK + 8, G = GATED ? 2 : 1;
  if (static_cast<int>(blockIdx.y) >= *num_tiles) return;
  __shared__ __align__(32) __nv_bfloat16 As[TM][LD];
  __shared__ __align__(32) __nv_bfloat16 Ws[G][TN][LD];
  __shared__ __align__(32) float Cs[8][16][32 + 4];
  const int e = tile_expert[blockIdx.y], r0 = tile_first[blockIdx.y];
  const int r_end = min(r0 + TM, expert_start[e + 1]);
  const int n0 = blockIdx.x * TN;
  const __nv_bfloat16* We = W + e * w_expert_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wr = warp >> 1, wc = warp & 1;
  // loads: thread -> row tid / 4, sixteen k from (tid % 4) * 16, as two pieces of eight
  const int lrow = tid >> 2, lk = (tid & 3) * 16;
  const int arow = r0 + lrow;
  const __nv_bfloat16* a_src = nullptr;
  if (arow < r_end) a_src = A + static_cast<size_t>(gather ? gather[arow] : arow) * lda;
  const int wn = n0 + lrow;
  const __nv_bfloat16* w_src[G];
#pragma unroll
  for (int g = 0; g < G; ++g) w_src[g] = wn < N ? We + static_cast<size_t>(wn + g * up_row_offset) * K : nullptr;
  const bool vec = (K % 8 == 0) && (lda % 8 == 0) && (reinterpret_cast<uintptr_t>(A) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(W) % 16 == 0);
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[G][2];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[g][j], 0.0f);

  // eight elements of a row from k on, zeros beyond K or for a row that does not exist
  auto fetch8 = [&](const __nv_bfloat16* row, int k) -> uint4 {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row == nullptr || k >= K) return v;
    if (vec && k + 8 <= K) return *reinterpret_cast<const uint4*>(row + k);
    __align__(16) __nv_bfloat16 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = k + i < K ? row[k + i] : __float2bfloat16_rn(0.0f);
    return *reinterpret_cast<const uint4*>(t);
  };
  uint4 ra[2], rw[G][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    ra[h] = fetch8(a_src, lk + 8 * h);
#pragma unroll
    for (int g = 0; g < G; ++g) rw[g][h] = fetch8(w_src[g], lk + 8 * h);
  }
  for (int k0 = 0; k0 < K; k0 += BK) {
    __syncthreads();                                   // the step before is no longer read
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<uint4*>(&As[lrow][lk + 8 * h]) = ra[h];
#pragma unroll
      for (int g = 0; g < G; ++g) *reinterpret_cast<uint4*>(&Ws[g][lrow][lk + 8 * h]) = rw[g][h];
    }
    __syncthreads();
    if (k0 + BK < K) {                                 // the next step's operands are on their way during the products
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ra[h] = fetch8(a_src, k0 + BK + lk + 8 * h);
#pragma unroll
        for (int g = 0; g < G; ++g) rw[g][h] = fetch8(w_src[g], k0 + BK + lk + 8 * h);
      }
    }
#pragma unroll
    for (int ks = 0; ks < BK; ks += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, &As[wr * 16][ks], LD);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
          wmma::load_matrix_sync(fb, &Ws[g][wc * 32 + j * 16][ks], LD);
          wmma::mma_sync(acc[g][j], fa, fb, acc[g][j]);
        }
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if constexpr (GATED) {          // both accumulators have one layout: element i of one meets element i of the other
#pragma unroll
      for (int i = 0; i < acc[0][j].num_elements; ++i) acc[0][j].x[i] = glu_f(acc[0][j].x[i], acc[G - 1][j].x[i], act);
    }
    wmma::store_matrix_sync(&Cs[warp][0][j * 16], acc[0][j], 32 + 4, wmma::mem_row_major);
  }
  __syncwarp();
  for (int i = lane; i < 16 * 32; i += 32) {
    const int rr = i >> 5, cc = i & 31;
    const int r = r0 + wr * 16 + rr, n = n0 + wc * 32 + cc;
    if (r >= r_end || n >= N) continue;
    C[static_cast<size_t>(r) * N + n] = from_f32<TO>(Cs[warp][rr][cc]);
  }
}

// ------------------------------------------------------------------ bfloat16 products of a step of few pairs
// A decode step has a handful of rows an expert and must read all of that expert's weights: the tensor cores have
// nothing to do, and the time is the weights' way out of memory.  So each warp takes ONE output column n of ONE
// expert (its gate row and its up row when GATED), streams the rows in 16-byte pieces (lane l takes columns
// 8 l .. 8 l + 7, then 256 further on, in order; the lanes' sums meet in a butterfly) and multiplies them with up to
// FEW_ROWS of the expert's rows at a time (more rows: another pass over the same weight rows, which the caches still
// hold).  grid (ceil(N / FEW_WARPS), experts); blocks of experts without rows return at once.  A row's result does
// not depend on what else the step holds.  K a multiple of 8.
constexpr int FEW_PAIRS = 64, FEW_ROWS = 4, FEW_WARPS = 8;

template <bool GATED, typename TO>
__global__ void __launch_bounds__(FEW_WARPS * 32)
expert_rows_few_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ sorted_token,
                       const __nv_bfloat16* __restrict__ W, long long w_stride, int ff, TO* __restrict__ C, int ldc,
                       int N, int K, const int* __restrict__ expert_start, const GluAct act) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const int e = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * FEW_WARPS + warp;
  const int first = expert_start[e], last = expert_start[e + 1];
  if (first >= last || n >= N) return;
  const __nv_bfloat16* w0 = W + static_cast<size_t>(e) * w_stride + static_cast<size_t>(n) * K;
  const __nv_bfloat16* w1 = GATED ? w0 + static_cast<size_t>(ff) * K : w0;
  for (int r0 = first; r0 < last; r0 += FEW_ROWS) {
    const int nr = min(FEW_ROWS, last - r0);
    const __nv_bfloat16* a[FEW_ROWS];
#pragma unroll
    for (int i = 0; i < FEW_ROWS; ++i) {             // a row beyond the last reads the last one; its sums are dropped
      const int r = r0 + min(i, nr - 1);
      a[i] = A + static_cast<size_t>(GATED ? sorted_token[r] : r) * lda;
    }
    float acc0[FEW_ROWS], acc1[FEW_ROWS];
#pragma unroll
    for (int i = 0; i < FEW_ROWS; ++i) acc0[i] = acc1[i] = 0.0f;
#pragma unroll 2
    for (int k = lane * 8; k < K; k += 256) {
      float g[8], u[8];
      load_floats<__nv_bfloat16, 8>(w0 + k, g);
      if (GATED) load_floats<__nv_bfloat16, 8>(w1 + k, u);
#pragma unroll
      for (int i = 0; i < FEW_ROWS; ++i) {
        float v[8];
        load_floats<__nv_bfloat16, 8>(a[i] + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc0[i] = fmaf(g[j], v[j], acc0[i]);
          if (GATED) acc1[i] = fmaf(u[j], v[j], acc1[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < FEW_ROWS; ++i) {
      const float s0 = warp_sum(acc0[i]);
      const float s1 = GATED ? warp_sum(acc1[i]) : 0.0f;
      if (lane == 0 && i < nr)
        C[static_cast<size_t>(r0 + i) * ldc + n] = from_f32<TO>(GATED ? glu_f(s0, s1, act) : s0);
    }
  }
}

// ------------------------------------------------------------------ the experts' outputs back to the tokens
// weight: one per pair, or null for `uniform` each.  add [tokens, width] (TA; a shared expert's output) joins the sum,
// times add_scale[t] if that is given (a gate of the shared expert, one float a token).
// grid (tokens, column tiles of 1,024): a thread takes four neighbouring columns (one where the width is no multiple
// of four); the sum over k runs in order either way.
template <typename TA>
__global__ void __launch_bounds__(256)
expert_combine_kernel(float* __restrict__ out, const float* __restrict__ Y, const int* __restrict__ pos_of_pair,
                      int top, int width, float uniform, const float* __restrict__ weight,
                      const TA* __restrict__ add, const float* __restrict__ add_scale) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  const size_t t = blockIdx.x;
  const float as = (add != nullptr && add_scale != nullptr) ? add_scale[t] : 1.0f;
  if (width % 4 == 0) {
    const int c = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (c >= width) return;
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int k = 0; k < top; ++k) {
      const float4 v = *reinterpret_cast<const float4*>(Y + static_cast<size_t>(pos_of_pair[t * top + k]) * width + c);
      if (weight == nullptr) {
        s[0] += v.x; s[1] += v.y; s[2] += v.z; s[3] += v.w;
      } else {
        const float g = weight[t * top + k];
        s[0] = fmaf(g, v.x, s[0]); s[1] = fmaf(g, v.y, s[1]); s[2] = fmaf(g, v.z, s[2]); s[3] = fmaf(g, v.w, s[3]);
      }
    }
    if (weight == nullptr) { s[0] *= uniform; s[1] *= uniform; s[2] *= uniform; s[3] *= uniform; }
    if (add != nullptr) {
      float a[4];
      load_floats<TA, 4>(add + t * width + c, a);
      s[0] = fmaf(as, a[0], s[0]); s[1] = fmaf(as, a[1], s[1]); s[2] = fmaf(as, a[2], s[2]); s[3] = fmaf(as, a[3], s[3]);
    }
    *reinterpret_cast<float4*>(out + t * width + c) = make_float4(s[0], s[1], s[2], s[3]);
    return;
  }
  for (int c = blockIdx.y * 1024 + threadIdx.x; c < min(width, (static_cast<int>(blockIdx.y) + 1) * 1024); c += blockDim.x) {
    float s = 0.0f;
    if (weight == nullptr) {
      for (int k = 0; k < top; ++k) s += Y[static_cast<size_t>(pos_of_pair[t * top + k]) * width + c];
      s *= uniform;
    } else {
      for (int k = 0; k < top; ++k)
        s = fmaf(weight[t * top + k], Y[static_cast<size_t>(pos_of_pair[t * top + k]) * width + c], s);
    }
    if (add != nullptr) s = fmaf(as, to_f32<TA>(add[t * width + c]), s);
    out[t * width + c] = s;
  }
}

// ------------------------------------------------------------------ the router
// z[t][e] = W[e] . x[t] in float (FFMA, whatever the dtype of x and W), scores s = softmax over all experts (or a
// sigmoid of each).  The CHOICE looks at c = s + correction (one float an expert; null: c = s): experts in `groups`
// equal groups of neighbours, a group's score the sum of its `group_members` largest c (1: its largest), only experts
// of the `keep` best groups can be chosen (the others are shut out whatever their c, which may be negative), the `top`
// largest c of them are.  The WEIGHTS are the chosen experts' s (without the correction), divided by their sum if
// `renormalize`, times `gain_scale`.  Ties go to the lower index.
// An extra row `gate_w` (null: none) gives gate_out[t] = sigmoid(gate_w . x[t]): the gate of something that every
// token takes besides its experts.  All warps share that row (warp w takes every eighth piece of 256 columns; the
// warps' sums are added in warp order), so that it does not cost one warp a second round of rows.
// A block takes TT tokens (1 for a step of few tokens, so that they spread over the SMs; 4 otherwise): warp w
// multiplies rows 2w, 2w + 1, then 2w + 16, .. for all of them (a row of W is read once a block), then warp t
// chooses for token t.  A logit is summed the same way whatever the block holds: lane l takes columns
// 8 l .. 8 l + 7, then 256 further on and so on, in order, and the lanes' sums meet in a butterfly.  Rows that start
// on 16 bytes are read in 16-byte pieces.  Shared memory a token: experts + 1 floats (logits, then scores), experts
// floats (what the choice looks at) and experts ints.
constexpr int ROUTER_WARPS = 8;

template <typename TX, typename TW, int TT>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
expert_router_kernel(const TX* __restrict__ x, const TW* __restrict__ W, int tokens, int width, int experts,
                     int groups, int keep, int top, int sigmoid_scores, int renormalize,
                     const float* __restrict__ correction, int group_members, float gain_scale,
                     const TW* __restrict__ gate_w, float* __restrict__ gate_out, int* __restrict__ choice,
                     float* __restrict__ weight) {
  pdl_launch_dependents();                          // the kernel after this one may be scheduled; it waits before it reads
  pdl_wait();                                        // what this kernel reads belongs to the kernels before it
  extern __shared__ float rsm[];
  __shared__ float gate_part[TT][ROUTER_WARPS];
  const int zs = experts + 1;                                       // a token's logits (one spare place)
  float* z = rsm;                                                   // [TT][experts + 1]
  float* look = rsm + TT * zs;                                      // [TT][experts]: what the choice compares
  int* open = reinterpret_cast<int*>(look + TT * experts);          // [TT][experts]: may still be chosen
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * TT;
  const int nt = min(TT, tokens - t0);
  const bool wide = width % 8 == 0 && (gate_w == nullptr || reinterpret_cast<uintptr_t>(gate_w) % 16 == 0);
  const int rows = experts;
  if (gate_w != nullptr) {
    float acc[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) acc[i] = 0.0f;
    const TX* xs = x + static_cast<size_t>(t0) * width;
    for (int k8 = lane * 8 + 256 * warp; k8 < width; k8 += 256 * ROUTER_WARPS) {
      if (wide) {
        float a[8];
        load_floats<TW, 8>(gate_w + k8, a);
#pragma unroll
        for (int i = 0; i < TT; ++i) {
          float v[8];
          load_floats<TX, 8>(xs + static_cast<size_t>(min(i, nt - 1)) * width + k8, v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i] = fmaf(a[j], v[j], acc[i]);
        }
      } else {
        const int end = min(k8 + 8, width);
        for (int k = k8; k < end; ++k) {
          const float a = to_f32<TW>(gate_w[k]);
#pragma unroll
          for (int i = 0; i < TT; ++i)
            if (i < nt) acc[i] = fmaf(a, to_f32<TX>(xs[static_cast<size_t>(i) * width + k]), acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) {
      const float v = warp_sum(acc[i]);
      if (lane == 0) gate_part[i][warp] = v;
    }
  }
  for (int e0 = 2 * warp; e0 < rows; e0 += 2 * ROUTER_WARPS) {
    const bool two = e0 + 1 < rows;
    float acc[2][TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) acc[0][i] = acc[1][i] = 0.0f;
    const int e1 = two ? e0 + 1 : e0;
    const TW* w0 = W + static_cast<size_t>(e0) * width;
    const TW* w1 = W + static_cast<size_t>(e1) * width;
    const TX* xs = x + static_cast<size_t>(t0) * width;
    if (wide) {
#pragma unroll 2
      for (int k = lane * 8; k < width; k += 256) {
        float a[8], b[8];
        load_floats<TW, 8>(w0 + k, a);
        load_floats<TW, 8>(w1 + k, b);
#pragma unroll
        for (int i = 0; i < TT; ++i) {               // a token beyond the last reads the last one's row; its sums are dropped
          float v[8];
          load_floats<TX, 8>(xs + static_cast<size_t>(min(i, nt - 1)) * width + k, v);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[0][i] = fmaf(a[j], v[j], acc[0][i]);
            acc[1][i] = fmaf(b[j], v[j], acc[1][i]);
          }
        }
      }
    } else {
      for (int k8 = lane * 8; k8 < width; k8 += 256) {
        const int end = min(k8 + 8, width);
        for (int k = k8; k < end; ++k) {
          const float a = to_f32<TW>(w0[k]), b = to_f32<TW>(w1[k]);
#pragma unroll
          for (int i = 0; i < TT; ++i)
            if (i < nt) {
              const float v = to_f32<TX>(xs[static_cast<size_t>(i) * width + k]);
              acc[0][i] = fmaf(a, v, acc[0][i]);
              acc[1][i] = fmaf(b, v, acc[1][i]);
            }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) {
      const float v0 = warp_sum(acc[0][i]), v1 = warp_sum(acc[1][i]);
      if (lane == 0 && i < nt) {
        z[i * zs + e0] = v0;
        if (two) z[i * zs + e0 + 1] = v1;
      }
    }
  }
  __syncthreads();
  if (warp >= nt) return;
  float* s = z + warp * zs;
  float* c = look + warp * experts;
  int* can = open + warp * experts;
  const int t = t0 + warp;
  if (gate_w != nullptr && lane == 0) {
    float g = 0.0f;
    for (int w = 0; w < ROUTER_WARPS; ++w) g += gate_part[warp][w];
    gate_out[t] = 1.0f / (1.0f + expf(-g));
  }
  if (sigmoid_scores) {
    for (int e = lane; e < experts; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
  } else {
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, s[e]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int e = lane; e < experts; e += 32) { s[e] = expf(s[e] - m); sum += s[e]; }
    sum = warp_sum(sum);
    for (int e = lane; e < experts; e += 32) s[e] = s[e] / sum;
  }
  for (int e = lane; e < experts; e += 32) {
    can[e] = groups <= 1 ? 1 : 0;
    c[e] = correction != nullptr ? s[e] + correction[e] : s[e];
  }
  __syncwarp();
  const int per = experts / max(groups, 1);
  // argmax over lanes of (value, lower index first)
  auto best_of = [&](float v, int i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    return i;
  };
  if (groups > 1) {
    // the keep best groups, one at a time; `can` of a group's first expert doubles as "group taken"
    const int members = min(max(group_members, 1), per);
    for (int r = 0; r < keep; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        if (can[g * per] != 0) continue;
        const float* cg = c + g * per;
        float gm;
        if (members == 1) {
          gm = -INFINITY;
          for (int j = 0; j < per; ++j) gm = fmaxf(gm, cg[j]);
        } else {
          // the sum of the group's `members` largest, taken in the order (larger first, lower index first)
          gm = 0.0f;
          float pv = INFINITY;
          int pj = -1;
          for (int n = 0; n < members; ++n) {
            float mv = -INFINITY;
            int mj = per;
            for (int j = 0; j < per; ++j) {
              const float v = cg[j];
              const bool after = v < pv || (v == pv && j > pj);          // not yet taken
              if (after && (v > mv || (v == mv && j < mj))) { mv = v; mj = j; }
            }
            if (mj == per) break;
            gm += mv;
            pv = mv; pj = mj;
          }
        }
        if (gm > bv || (gm == bv && g < bi)) { bv = gm; bi = g; }
      }
      const int g = best_of(bv, bi);
      __syncwarp();
      if (g != 0x7fffffff)
        for (int j = lane; j < per; j += 32) can[g * per + j] = 1;
      __syncwarp();
    }
  }
  float total = 0.0f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32)
      if (can[e] == 1 && (c[e] > bv || (c[e] == bv && e < bi))) { bv = c[e]; bi = e; }
    const int e = best_of(bv, bi);
    __syncwarp();
    if (lane == 0) {
      choice[static_cast<size_t>(t) * top + r] = e == 0x7fffffff ? -1 : e;
      weight[static_cast<size_t>(t) * top + r] = e == 0x7fffffff ? 0.0f : s[e];
      if (e != 0x7fffffff) can[e] = 2;
    }
    if (e != 0x7fffffff) total += s[e];
    __syncwarp();
  }
  if (lane == 0) {
    const float f = (renormalize && total > 0.0f) ? gain_scale / total : gain_scale;
    if (f != 1.0f)
      for (int r = 0; r < top; ++r) weight[static_cast<size_t>(t) * top + r] *= f;
  }
}

// ------------------------------------------------------------------ C interface
// Ints of scratch that the routing needs for (tokens, top, experts); row tiles of at least 64 rows.
B200_EXPORT long long b200_expert_route_ints(int tokens, int top, int experts) {
  const long long pairs = static_cast<long long>(tokens) * top;
  const long long tiles = (pairs + TM - 1) / TM + experts;
  return 2 * pairs + (experts + 1) + 2 * tiles + 1;
}

// Where the parts of the routing scratch lie.
struct RouteLayout {
  int *sorted_token, *pos_of_pair, *expert_start, *tile_expert, *tile_first, *num_tiles;
  int tiles;
};
static RouteLayout route_layout(int* route, int pairs, int experts) {
  RouteLayout r;
  r.tiles = (pairs + TM - 1) / TM + experts;
  r.sorted_token = route;
  r.pos_of_pair = r.sorted_token + pairs;
  r.expert_start = r.pos_of_pair + pairs;
  r.tile_expert = r.expert_start + experts + 1;
  r.tile_first = r.tile_expert + r.tiles;
  r.num_tiles = r.tile_first + r.tiles;
  return r;
}

// Who names a token's experts and how their outputs are summed: a table row by token id with equal weights, or a
// router's choices [tokens, top] with a weight each; `add` [tokens, width] (dtype add_dtype) joins the sum.
struct ExpertChoice {
  const int *token_ids, *table;
  int vocab;
  const int* choice;
  const float* weight;
  const void* add;
  int add_dtype;
  const float* add_scale;      // null, or one factor a token for `add`
};

static int launch_combine(float* out, const float* y, const int* pos_of_pair, int tokens, int top, int width,
                          const ExpertChoice& c, cudaStream_t stream) {
  const float uniform = 1.0f / static_cast<float>(top);
  const dim3 combine_grid(tokens, (width + 1023) / 1024);
  if (c.add != nullptr && c.add_dtype == B200_BF16)
    return b200_launch(expert_combine_kernel<__nv_bfloat16>, combine_grid, dim3(256), 0, stream, 0, out, y, pos_of_pair,
                       top, width, uniform, c.weight, static_cast<const __nv_bfloat16*>(c.add), c.add_scale);
  return b200_launch(expert_combine_kernel<float>, combine_grid, dim3(256), 0, stream, 0, out, y, pos_of_pair, top, width,
                     uniform, c.weight, static_cast<const float*>(c.add), c.add_scale);
}

// x [tokens, width] -> out [tokens, width] float32.  `h` holds pairs * ff elements of x's dtype, `y` pairs * width
// floats, `route` b200_expert_route_ints(...) ints.
static int run_experts(const void* x, int dtype, const ExpertChoice& c, int top, int experts, const void* gate_up,
                       const void* down, int tokens, int width, int ff, const GluAct act, void* h, float* y, int* route,
                       float* out, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0 || experts <= 0 || width <= 0 || ff <= 0 || (c.choice == nullptr && c.vocab <= 0)) return B200_BAD_SIZE;
  const long long pairs_ll = static_cast<long long>(tokens) * top;
  if (pairs_ll > (1ll << 30) || (2 * experts + 1) * sizeof(int) > 48 * 1024) return B200_BAD_SIZE;
  const int pairs = static_cast<int>(pairs_ll);
  const RouteLayout rl = route_layout(route, pairs, experts);
  const int tiles = rl.tiles;
  if (tiles > 65535) return B200_BAD_SIZE;
  int *sorted_token = rl.sorted_token, *pos_of_pair = rl.pos_of_pair, *expert_start = rl.expert_start;
  int *tile_expert = rl.tile_expert, *tile_first = rl.tile_first, *num_tiles = rl.num_tiles;
  int rc = b200_launch(expert_route_kernel, dim3(1), dim3(1024), (2 * experts + 1) * sizeof(int), stream, 0,
                       c.token_ids, c.table, c.vocab, top, experts, c.choice, tokens, sorted_token, pos_of_pair,
                       expert_start, tile_expert, tile_first, num_tiles, TM, err);
  if (rc != 0) return rc;
  const dim3 g1((ff + TN - 1) / TN, tiles), g2((width + TN - 1) / TN, tiles);
  const long long gu_stride = 2ll * ff * width, dn_stride = static_cast<long long>(width) * ff;
  if (dtype == B200_F32) {
    expert_gemm_f32_kernel<true><<<g1, 256, 0, stream>>>(
        static_cast<const float*>(x), width, sorted_token, static_cast<const float*>(gate_up), gu_stride, ff,
        static_cast<float*>(h), ff, width, expert_start, tile_expert, tile_first, num_tiles, act);
    expert_gemm_f32_kernel<false><<<g2, 256, 0, stream>>>(
        static_cast<const float*>(h), ff, nullptr, static_cast<const float*>(down), dn_stride, 0, y, width, ff,
        expert_start, tile_expert, tile_first, num_tiles, act);
  } else if (dtype == B200_BF16 && pairs <= FEW_PAIRS && width % 8 == 0 && ff % 8 == 0) {
    const dim3 f1((ff + FEW_WARPS - 1) / FEW_WARPS, experts), f2((width + FEW_WARPS - 1) / FEW_WARPS, experts);
    rc = b200_launch(expert_rows_few_kernel<true, __nv_bfloat16>, f1, dim3(FEW_WARPS * 32), 0, stream, 0,
                     static_cast<const __nv_bfloat16*>(x), width, sorted_token, static_cast<const __nv_bfloat16*>(gate_up),
                     gu_stride, ff, static_cast<__nv_bfloat16*>(h), ff, ff, width, expert_start, act);
    if (rc != 0) return rc;
    rc = b200_launch(expert_rows_few_kernel<false, float>, f2, dim3(FEW_WARPS * 32), 0, stream, 0,
                     static_cast<const __nv_bfloat16*>(h), ff, static_cast<const int*>(nullptr),
                     static_cast<const __nv_bfloat16*>(down), dn_stride, 0, y, width, width, ff, expert_start, act);
    if (rc != 0) return rc;
  } else if (dtype == B200_BF16) {
    expert_gemm_bf16_kernel<true, __nv_bfloat16><<<g1, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), width, sorted_token, static_cast<const __nv_bfloat16*>(gate_up),
        gu_stride, ff, static_cast<__nv_bfloat16*>(h), ff, width, expert_start, tile_expert, tile_first, num_tiles, act);
    expert_gemm_bf16_kernel<false, float><<<g2, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(h), ff, nullptr, static_cast<const __nv_bfloat16*>(down), dn_stride, 0, y,
        width, ff, expert_start, tile_expert, tile_first, num_tiles, act);
  } else {
    return B200_BAD_DTYPE;
  }
  rc = b200_check_launch();
  if (rc != 0) return rc;
  return launch_combine(out, y, pos_of_pair, tokens, top, width, c, stream);
}

B200_EXPORT int b200_table_experts(const void* x, int dtype, const int* token_ids, const int* table, int vocab, int top,
                                   int experts, const void* gate_up, const void* down, int tokens, int width, int ff,
                                   void* h, float* y, int* route, float* out, int* err, cudaStream_t stream) {
  const ExpertChoice c = {token_ids, table, vocab, nullptr, nullptr, nullptr, B200_F32, nullptr};
  return run_experts(x, dtype, c, top, experts, gate_up, down, tokens, width, ff, GluAct{0, 0.0f, 0.0f}, h, y, route,
                     out, err, stream);
}

// The router alone: choice [tokens, top] ints and weight [tokens, top] floats.  x_dtype / w_dtype: B200_F32 or
// B200_BF16 each; the products are FFMA either way.  correction (null or [experts] floats), group_members, gain_scale,
// gate_w (null or one more row of w's dtype) and gate_out ([tokens] floats): see the kernel.
B200_EXPORT int b200_expert_router(const void* x, int x_dtype, const void* w, int w_dtype, int tokens, int width,
                                   int experts, int groups, int keep, int top, int sigmoid_scores, int renormalize,
                                   const float* correction, int group_members, float gain_scale, const void* gate_w,
                                   float* gate_out, int* choice, float* weight, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || experts <= 0 || groups <= 0 || experts % groups || keep <= 0 || keep > groups || top <= 0 ||
      top > keep * (experts / groups) || group_members <= 0 || (gate_w != nullptr && gate_out == nullptr))
    return B200_BAD_SIZE;
  const int per_block = tokens <= 148 ? 1 : 4;
  const size_t per_token = (static_cast<size_t>(experts) + 1) * sizeof(float) + experts * (sizeof(float) + sizeof(int));
  const size_t smem = per_block * per_token;
  if (8 * per_token > 48 * 1024) return B200_BAD_SIZE;
  const unsigned blocks = (tokens + per_block - 1) / per_block;
  int router_rc = 0;
#define B200_ROUTER_TT(TX, TW, TT)                                                                                   \
  router_rc = b200_launch(expert_router_kernel<TX, TW, TT>, dim3(blocks), dim3(ROUTER_WARPS * 32), smem, stream, 0,  \
      static_cast<const TX*>(x), static_cast<const TW*>(w), tokens, width, experts, groups, keep, top, sigmoid_scores, \
      renormalize, correction, group_members, gain_scale, static_cast<const TW*>(gate_w), gate_out, choice, weight)
#define B200_ROUTER(TX, TW)                                                                                          \
  do {                                                                                                               \
    if (per_block == 1) B200_ROUTER_TT(TX, TW, 1);                                                                   \
    else B200_ROUTER_TT(TX, TW, 4);                                                                                  \
  } while (0)
  if (x_dtype == B200_F32 && w_dtype == B200_F32) B200_ROUTER(float, float);
  else if (x_dtype == B200_BF16 && w_dtype == B200_BF16) B200_ROUTER(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == B200_BF16 && w_dtype == B200_F32) B200_ROUTER(__nv_bfloat16, float);
  else if (x_dtype == B200_F32 && w_dtype == B200_BF16) B200_ROUTER(float, __nv_bfloat16);
  else return B200_BAD_DTYPE;
#undef B200_ROUTER_TT
#undef B200_ROUTER
  return router_rc;
}

// Experts chosen by a router: choice and weight [tokens, top] (b200_expert_router), glu kind `act_kind` with `limit`
// and `alpha`, `add` (null, or [tokens, width] of add_dtype: what every token gets besides, e.g. a shared expert),
// `add_scale` (null, or one float a token that multiplies its row of `add`).
B200_EXPORT int b200_routed_experts(const void* x, int dtype, const int* choice, const float* weight, int top,
                                    int experts, const void* gate_up, const void* down, int tokens, int width, int ff,
                                    int act_kind, float limit, float alpha, const void* add, int add_dtype,
                                    const float* add_scale, void* h, float* y, int* route, float* out, int* err,
                                    cudaStream_t stream) {
  if (choice == nullptr || weight == nullptr || act_kind < 0 || act_kind > 1) return B200_BAD_SIZE;
  const ExpertChoice c = {nullptr, nullptr, 0, choice, weight, add, add_dtype, add_scale};
  return run_experts(x, dtype, c, top, experts, gate_up, down, tokens, width, ff, GluAct{act_kind, limit, alpha}, h, y,
                     route, out, err, stream);
}
