// Products per group of rows on the 5th-generation tensor cores (sm_100a): the per-expert
// products of a routed feed-forward for steps with many rows (a prompt), bf16 operands, fp32
// accumulation in tensor memory.  The contract of nb_moe_gemm for rows that already lie in the
// order of their places (the caller gathers them first: nb_moe_gather), so that a group's rows
// are consecutive and a tile of 128 of them is one TMA box.
//
// A CTA computes one tile of 128 places x 128 outputs of one expert.  Warp 0: one thread
// issues the TMA loads (128 x 64 boxes of the rows and of the expert's weight rows, 128-byte
// swizzled; the weights of all experts are one [experts * N, K] matrix to the tensor map)
// into a ring of four stages guarded by full/empty mbarriers.  Warp 1 owns the tensor memory
// and one of its threads issues `tcgen05.mma` (M = 128, N = 128, K = 16; four per stage), with
// a second weight set into a second accumulator from the same staged rows; `tcgen05.commit`
// hands a stage back and, after the last block of K, signals the accumulators.  Warps 2 to 5
// read their quarter of the accumulators with `tcgen05.ld` (a lane per row, 32 columns at a
// time), apply act(a) * b where there are two, and store their row's 32 columns if the row
// belongs to the group (a tile may reach into the next group's rows; those results are
// dropped) and the columns exist.
//
// Every wait on an mbarrier is bounded by the clock budget of the tensor-core kernels; a wait
// that runs out raises the product kernels' error word, all roles leave their loops, and the
// CTA frees its tensor memory and returns.
#include "tc05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BN = 128, BK = 64, UMMA_K = 16, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;

template <bool DUAL>
struct Layout {
  static constexpr int STAGE_BYTES = A_BYTES + (DUAL ? 2 : 1) * B_BYTES;
  static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
  static constexpr int N_BARRIERS = 2 * STAGES + 1;
  static constexpr int TOTAL = TILES_BYTES + N_BARRIERS * 8 + 16 + 1024 /* alignment slack */;
  static constexpr uint32_t TMEM_COLS = DUAL ? 256 : 128;
};

template <bool DUAL, typename TY>
__global__ void __launch_bounds__(THREADS)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
              const __grid_constant__ CUtensorMap map_w2, const int* offsets, int n_experts, TY* y,
              int y_stride, int N, int K, int act, float act_param, int* err_word) {
  using L = Layout<DUAL>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;      // swizzle atoms want 1024-byte alignment
  unsigned char* gen = smem_dyn + (base - raw);
  const uint32_t bars = base + L::TILES_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * STAGES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + L::TILES_BYTES + L::N_BARRIERS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_kb = (K + BK - 1) / BK;

  if (tid == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    if (DUAL) prefetch_tensormap(&map_w2);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(L::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc05_fence_before();
  __syncthreads();
  tc05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  nb_grid_dependency_wait();      // the rows and the grouping are the predecessors' work
  nb_launch_dependents();

  // which expert and which of its tiles this CTA has
  int tile = blockIdx.x, e = 0, begin = 0, end = 0;
  for (; e < n_experts; ++e) {
    begin = offsets[e];
    end = offsets[e + 1];
    const int t = (end - begin + BM - 1) / BM;
    if (tile < t) break;
    tile -= t;
  }
  const bool have = e < n_experts;
  const int m0 = begin + tile * BM, n0 = blockIdx.y * BN;

  if (have && warp == 0) {
    if (lane == 0) {   // ------------------------------------------------------- TMA producer
      const int w_row = e * N + n0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
        if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag)) break;
        const uint32_t dst = base + s * L::STAGE_BYTES;
        mbar_expect_tx(full_bar(s), (uint32_t)L::STAGE_BYTES);
        tma_load_2d(dst, &map_x, kb * BK, m0, full_bar(s));
        tma_load_2d(dst + A_BYTES, &map_w, kb * BK, w_row, full_bar(s));
        if (DUAL) tma_load_2d(dst + A_BYTES + B_BYTES, &map_w2, kb * BK, w_row, full_bar(s));
      }
    }
  } else if (have && warp == 1) {
    if (lane == 0) {   // ------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(full_bar(s), (uint32_t)(kb / STAGES) & 1u, abort_flag);
        if (!ok) break;
        tc05_fence_after();
        const uint32_t a_addr = base + s * L::STAGE_BYTES;
        const uint64_t da = smem_desc_sw128(a_addr);
        const uint64_t db = smem_desc_sw128(a_addr + A_BYTES);
        const uint64_t db2 = smem_desc_sw128(a_addr + A_BYTES + B_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing K by 16 elements inside the swizzle atom = 32 bytes = 2 address units
          const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
          tc05_mma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, accumulate);
          if (DUAL)
            tc05_mma_bf16(tmem_base + (uint32_t)BN, da + (uint64_t)(2 * k), db2 + (uint64_t)(2 * k), idesc,
                          accumulate);
        }
        tc05_commit(empty_bar(s));     // the stage is free once these MMAs have read it
      }
      if (ok) tc05_commit(acc_full);   // complete once all MMAs issued so far are done
    }
  } else if (have) {   // ---------------------------------------------------------- epilogue
    const int quarter = warp & 3;      // the 32 tensor-memory lanes this warp may read
    const bool ready = __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full, 0u, abort_flag), 0) != 0;
    if (ready) {
      tc05_fence_after();
      const int p = m0 + quarter * 32 + lane;
      TY* row = y + (size_t)p * y_stride;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32);
        tc05_ld_32x32b_x32(taddr, v);
        if (DUAL) {
          uint32_t w[32];
          tc05_ld_32x32b_x32(taddr + (uint32_t)BN, w);
          tc05_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(nb_gate_up<true>(__uint_as_float(v[j]), __uint_as_float(w[j]), act, act_param));
        }
        tc05_wait_ld();
        if (!DUAL && act != NB_ACT_NONE) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(nb_apply_act_fast(__uint_as_float(v[j]), act));
        }
        const int col0 = n0 + c * 32;
        if (p < end && col0 < N) {
          const bool whole = col0 + 32 <= N;
          if constexpr (sizeof(TY) == 2) {
            if (whole && (y_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                pk.x = *reinterpret_cast<uint32_t*>(&h0);
                pk.y = *reinterpret_cast<uint32_t*>(&h1);
                pk.z = *reinterpret_cast<uint32_t*>(&h2);
                pk.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(row + col0 + j) = pk;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) row[col0 + j] = nb_from_f32<TY>(__uint_as_float(v[j]));
            }
          } else {
            if (whole && (y_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(row + col0 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) row[col0 + j] = nb_from_f32<TY>(__uint_as_float(v[j]));
            }
          }
        }
      }
    }
  }

  tc05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) {
      nb_report_timeout(err_word);
      // let TMA copies that are still in flight land before the shared memory goes away
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) {
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                 "r"(L::TMEM_COLS)
                 : "memory");
  }
}

// xs[place] = x[order[place] / row_div] for the places that are taken (below offsets[n_experts]).
__global__ void moe_gather_kernel(const bf16* x, int x_stride, const int* order, int row_div,
                                  const int* offsets, int n_experts, bf16* xs, int K) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int place = blockIdx.x;
  if (place >= offsets[n_experts]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(order[place] / row_div) * x_stride);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)place * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}

int* error_word() {
  int* w = nb_error_words();
  return w ? w + NB_ERRW_GEMM_TCGEN05 : nullptr;
}

template <bool DUAL, typename TY>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mw2, dim3 grid,
           const int* offsets, int n_experts, TY* y, int y_stride, int N, int K, int act, float act_param,
           cudaStream_t stream) {
  auto kern = moe_tc_kernel<DUAL, TY>;
  const int smem = Layout<DUAL>::TOTAL;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  NB_CUDA(nb_launch(kern, grid, dim3(THREADS), (size_t)smem, stream, mx, mw, mw2, offsets, n_experts, y,
                    y_stride, N, K, act, act_param, error_word()));
  return 0;
}

}  // namespace

NB_EXPORT int nb_moe_gemm_tc_set_wait_budget(long long cycles) { return set_wait_budget(cycles); }

// Whether the kernel takes this shape: bf16 rows and weights, K a multiple of 8 and at least a
// box wide, at least a box of rows of x and of stacked weight rows.
NB_EXPORT int nb_moe_gemm_tc_supported(int x_dtype, int w_dtype, int x_rows, int n_experts, int N,
                                       int K) {
  return x_dtype == NB_BF16 && w_dtype == NB_BF16 && K % 8 == 0 && K >= BK && x_rows >= BM &&
         (long long)n_experts * N >= BN;
}

NB_EXPORT int nb_moe_gather(const void* x, int x_stride, const int* order, int row_div,
                            const int* offsets, int n_experts, void* xs, int n_places, int K,
                            cudaStream_t stream) {
  if (n_places == 0) return 0;
  NB_REQUIRE(K % 8 == 0 && x_stride % 8 == 0 && row_div >= 1, NB_ERR_BAD_ARG,
             "moe_gather: rows must be multiples of 16 bytes");
  NB_REQUIRE(((uintptr_t)x | (uintptr_t)xs) % 16 == 0, NB_ERR_BAD_ARG,
             "moe_gather: pointers must be 16-byte aligned");
  NB_CUDA(nb_launch(moe_gather_kernel, dim3(n_places), dim3(128), 0, stream, (const bf16*)x, x_stride,
                    order, row_div, offsets, n_experts, (bf16*)xs, K));
  NB_CHECK_LAUNCH("moe_gather");
  return 0;
}

// x: bf16 [x_rows][K], the rows of place p at row p; W, W2: bf16 [n_experts][N][K] (W2 may be
// null); y: [>= n_places][y_stride].
NB_EXPORT int nb_moe_gemm_tc(const void* x, int x_rows, const int* offsets, int n_experts, int n_places,
                             const void* W, const void* W2, void* y, int y_dtype, int y_stride, int N,
                             int K, int act, float act_param, cudaStream_t stream) {
  if (n_places == 0) return 0;
  NB_REQUIRE(nb_moe_gemm_tc_supported(NB_BF16, NB_BF16, x_rows, n_experts, N, K), NB_ERR_UNSUPPORTED,
             "moe_gemm_tc: shape not supported (rows=%d experts=%d N=%d K=%d)", x_rows, n_experts, N, K);
  NB_REQUIRE(((uintptr_t)x | (uintptr_t)W | (uintptr_t)W2) % 16 == 0, NB_ERR_BAD_ARG,
             "moe_gemm_tc: pointers must be 16-byte aligned");
  CUtensorMap mx, mw, mw2;
  int rc = make_map(&mx, x, x_rows, K, BM, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  rc = make_map(&mw, W, (long long)n_experts * N, K, BN, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  if (W2 != nullptr) {
    rc = make_map(&mw2, W2, (long long)n_experts * N, K, BN, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
    if (rc) return rc;
  } else {
    mw2 = mw;   // unused
  }
  const int tiles = (n_places + BM - 1) / BM + (n_experts < n_places ? n_experts : n_places);
  const dim3 grid(tiles, (N + BN - 1) / BN);
  NB_REQUIRE(grid.y <= 65535, NB_ERR_UNSUPPORTED, "moe_gemm_tc: %d outputs are too many", N);
  if (y_dtype == NB_BF16)
    rc = W2 ? launch<true, bf16>(mx, mw, mw2, grid, offsets, n_experts, (bf16*)y, y_stride, N, K, act, act_param, stream)
            : launch<false, bf16>(mx, mw, mw2, grid, offsets, n_experts, (bf16*)y, y_stride, N, K, act, act_param, stream);
  else if (y_dtype == NB_F32)
    rc = W2 ? launch<true, float>(mx, mw, mw2, grid, offsets, n_experts, (float*)y, y_stride, N, K, act, act_param, stream)
            : launch<false, float>(mx, mw, mw2, grid, offsets, n_experts, (float*)y, y_stride, N, K, act, act_param, stream);
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "moe_gemm_tc: unknown output dtype %d", y_dtype);
  if (rc) return rc;
  NB_CHECK_LAUNCH("moe_gemm_tc");
  return 0;
}
