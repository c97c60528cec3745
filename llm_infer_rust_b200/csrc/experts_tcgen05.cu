// The experts' two products on the fifth-generation tensor cores, for steps with many (token, expert) pairs.
//
// The pairs are sorted by expert (expert_route_kernel of experts.cu, row tiles of 128) and their rows of x gathered
// into one matrix X' [pairs, width], so that an expert's rows are a contiguous range.  Each product is then ONE
// persistent kernel over all experts, built like gemm_tcgen05_kernel (TMA ring of four stages, tcgen05.mma
// 128 x 256 x 16 from shared-memory descriptors, two accumulators in tensor memory, tcgen05.ld epilogue); what
// differs is where a tile's operands come from:
//   a tile is (row tile rt, column tile): rows tile_first[rt] .. of X' (or of H) for the A operand, and the rows of
//   expert tile_expert[rt] in the experts' stacked weights ([experts * rows per expert, K] as one matrix) for B;
//   rows of the tile that belong to the next expert (or lie beyond the last pair) are computed and not stored.
//   GATED  H[pos] = glu(gate, up) (silu(gate) * up or the clamped form, see experts.cu): 128 gate columns and the same 128 up columns per tile, bfloat16 out
//   else   Y[pos] = H[pos] . W_down[e]^T: 256 columns per tile, float out
// Every wait is bounded by the clock, as in the kernel it is built from.
#include "experts.cu"
#include "gemm_tcgen05.cu"

constexpr int TC_ROWS = BM;          // rows of a row tile

__global__ void __launch_bounds__(256)
gather_rows_kernel(bf16* __restrict__ dst, const bf16* __restrict__ src, const int* __restrict__ index, int width) {
  const size_t r = blockIdx.x;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(index[r]) * width);
  uint4* d = reinterpret_cast<uint4*>(dst + r * width);
  for (int c = threadIdx.x; c < width / 8; c += blockDim.x) d[c] = s[c];
}

template <bool GATED, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
expert_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap wmap,
                           TO* __restrict__ out, int cols, int K, int w_rows_per_expert,
                           const int* __restrict__ expert_start, const int* __restrict__ tile_expert,
                           const int* __restrict__ tile_first, const int* __restrict__ num_row_tiles, int* err,
                           const GluAct act) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;          // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + BK - 1) / BK;
  const int n_tiles = GATED ? (cols + 127) / 128 : (cols + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {                                                          // the whole warp allocates tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(2 * TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                                                               // the routing and A come from kernels before
  const int row_tiles = *num_row_tiles;
  const int tiles = row_tiles * n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int rt = tile % row_tiles, tile_n = tile / row_tiles;         // CTAs that run together share few experts
        const int w_base = tile_expert[rt] * w_rows_per_expert;
        const int w_row0 = w_base + (GATED ? tile_n * 128 : tile_n * BN);
        const int w_row1 = GATED ? w_base + cols + tile_n * 128 : w_row0 + 128;
        const int a_row = tile_first[rt];
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES, use = it / STAGES;
          if (use > 0 && !mbar_wait(empty + s, (use - 1) & 1, err)) { ok = false; break; }
          unsigned char* st = ring + s * STAGE_BYTES;
          mbar_expect_tx(full + s, STAGE_BYTES);
          tma_load_2d(st, &amap, kb * BK, a_row, full + s);
          tma_load_2d(st + A_BYTES, &wmap, kb * BK, w_row0, full + s);
          tma_load_2d(st + A_BYTES + B_BYTES / 2, &wmap, kb * BK, w_row1, full + s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1, use = local >> 1;
        if (use > 0) ok = mbar_wait(acc_empty + acc, (use - 1) & 1, err);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_c = tmem_base + acc * TMEM_COLS;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full + s, (it / STAGES) & 1, err);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_c, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);
        }
        umma_commit(acc_full + acc);
      }
    }
  } else {
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int rt = tile % row_tiles, tile_n = tile / row_tiles;
      const int acc = local & 1;
      const int row = tile_first[rt] + quarter * 32 + lane;
      const bool row_ok = row < expert_start[tile_expert[rt] + 1];          // the rest of the tile is another expert's
      if (!mbar_wait(acc_full + acc, (local >> 1) & 1, err)) break;
      tc_fence_after();
      const uint32_t lane_base = tmem_base + acc * TMEM_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (!GATED) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld32(lane_base + c * 32, v);
          const int col0 = tile_n * BN + c * 32;
          if (row_ok && col0 < cols) {
            TO* dst = out + static_cast<size_t>(row) * cols + col0;
            if (col0 + 32 <= cols && (cols % 4) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
              for (int e = 0; e < 32 && col0 + e < cols; ++e) dst[e] = v[e];
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {                                       // gate columns c * 32 .., up columns 128 + c * 32 ..
          float g[32], u[32];
          tmem_ld32(lane_base + c * 32, g);
          tmem_ld32(lane_base + 128 + c * 32, u);
          const int col0 = tile_n * 128 + c * 32;
          if (row_ok && col0 < cols) {
            TO* dst = out + static_cast<size_t>(row) * cols + col0;
            __align__(16) bf16 r[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float2bfloat16_rn(glu_f(g[e], u[e], act));
            if (col0 + 32 <= cols && (cols % 8) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = *reinterpret_cast<const uint4*>(r + q * 8);
            } else {
              for (int e = 0; e < 32 && col0 + e < cols; ++e) dst[e] = r[e];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + acc);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * TMEM_COLS) : "memory");
  }
}

// The same as run_experts for bfloat16 with width and ff multiples of 8; `xs` holds pairs * width more elements (the
// gathered rows).  gate_up [experts * 2 ff, width] and down [experts * width, ff] as stacked matrices.
static int run_experts_tcgen05(const void* x, const ExpertChoice& c, int top, int experts, const void* gate_up,
                               const void* down, int tokens, int width, int ff, const GluAct act, void* xs, void* h,
                               float* y, int* route, float* out, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0 || experts <= 0 || width <= 0 || ff <= 0 || (c.choice == nullptr && c.vocab <= 0) || width % 8 || ff % 8)
    return B200_BAD_SIZE;
  const long long pairs_ll = static_cast<long long>(tokens) * top;
  if (pairs_ll > (1ll << 30) || (2 * experts + 1) * sizeof(int) > 48 * 1024) return B200_BAD_SIZE;
  const int pairs = static_cast<int>(pairs_ll);
  const RouteLayout rl = route_layout(route, pairs, experts);
  expert_route_kernel<<<1, 1024, (2 * experts + 1) * sizeof(int), stream>>>(
      c.token_ids, c.table, c.vocab, top, experts, c.choice, tokens, rl.sorted_token, rl.pos_of_pair, rl.expert_start,
      rl.tile_expert, rl.tile_first, rl.num_tiles, TC_ROWS, err);
  int rc = b200_check_launch();
  if (rc != 0) return rc;
  gather_rows_kernel<<<pairs, 256, 0, stream>>>(static_cast<bf16*>(xs), static_cast<const bf16*>(x), rl.sorted_token, width);
  rc = b200_check_launch();
  if (rc != 0) return rc;
  CUtensorMap xs_map, h_map, gu_map, dn_map;
  if ((rc = b200_gemm_tensor_map(&xs_map, xs, pairs, width)) != 0) return rc;
  if ((rc = b200_gemm_tensor_map(&h_map, h, pairs, ff)) != 0) return rc;
  if ((rc = b200_gemm_tensor_map(&gu_map, gate_up, static_cast<long long>(experts) * 2 * ff, width)) != 0) return rc;
  if ((rc = b200_gemm_tensor_map(&dn_map, down, static_cast<long long>(experts) * width, ff)) != 0) return rc;
  const size_t smem = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(expert_gemm_tcgen05_kernel<true, bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(expert_gemm_tcgen05_kernel<false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int most_row_tiles = (pairs + TC_ROWS - 1) / TC_ROWS + experts;    // the real count is known on the device only
  const int g1 = min(sms, most_row_tiles * ((ff + 127) / 128)), g2 = min(sms, most_row_tiles * ((width + BN - 1) / BN));
  rc = b200_launch(expert_gemm_tcgen05_kernel<true, bf16>, dim3(g1), dim3(THREADS), smem, stream, 0, xs_map, gu_map,
                   static_cast<bf16*>(h), ff, width, 2 * ff, rl.expert_start, rl.tile_expert, rl.tile_first, rl.num_tiles,
                   err, act);
  if (rc != 0) return rc;
  rc = b200_launch(expert_gemm_tcgen05_kernel<false, float>, dim3(g2), dim3(THREADS), smem, stream, 0, h_map, dn_map, y,
                   width, ff, width, rl.expert_start, rl.tile_expert, rl.tile_first, rl.num_tiles, err, act);
  if (rc != 0) return rc;
  return launch_combine(out, y, rl.pos_of_pair, tokens, top, width, c, stream);
}

B200_EXPORT int b200_table_experts_tcgen05(const void* x, const int* token_ids, const int* table, int vocab, int top,
                                           int experts, const void* gate_up, const void* down, int tokens, int width,
                                           int ff, void* xs, void* h, float* y, int* route, float* out, int* err,
                                           cudaStream_t stream) {
  const ExpertChoice c = {token_ids, table, vocab, nullptr, nullptr, nullptr, B200_F32, nullptr};
  return run_experts_tcgen05(x, c, top, experts, gate_up, down, tokens, width, ff, GluAct{0, 0.0f, 0.0f}, xs, h, y,
                             route, out, err, stream);
}

// b200_routed_experts on the tcgen05 products (bfloat16, width and ff multiples of 8).
B200_EXPORT int b200_routed_experts_tcgen05(const void* x, const int* choice, const float* weight, int top, int experts,
                                            const void* gate_up, const void* down, int tokens, int width, int ff,
                                            int act_kind, float limit, float alpha, const void* add, int add_dtype,
                                            const float* add_scale, void* xs, void* h, float* y, int* route, float* out, int* err,
                                            cudaStream_t stream) {
  if (choice == nullptr || weight == nullptr || act_kind < 0 || act_kind > 1) return B200_BAD_SIZE;
  const ExpertChoice c = {nullptr, nullptr, 0, choice, weight, add, add_dtype, add_scale};
  return run_experts_tcgen05(x, c, top, experts, gate_up, down, tokens, width, ff, GluAct{act_kind, limit, alpha}, xs,
                             h, y, route, out, err, stream);
}
