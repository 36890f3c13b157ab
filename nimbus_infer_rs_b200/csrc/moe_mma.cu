// Products per group of rows on the tensor cores (bf16 operands, fp32 accumulation): the
// per-expert products of a routed feed-forward (the contract of nb_moe_gemm, for bf16 rows and
// weights with K % 8 == 0; a group = the places of one expert), and the per-head linear maps of
// the latent attention (the contract of nb_head_linear; a group = one head, every row of the
// step belongs to every group, each group reads and writes its own columns).
//
// Two shapes of the same kernel.  Many rows: a CTA takes 128 places of one group and 64
// outputs; eight warps, each 32 places x 32 outputs (two by four MMA tiles, so an operand
// fetched from shared memory feeds several MMAs), a ring of three stages.  Few rows (a
// one-token step: a handful of places per expert, the product is a stream of the chosen
// experts' weights): a CTA takes 16 places and 64 outputs, four warps of 16 outputs each, and
// what a tile of 128 places would spend on rows that are not there goes into a ring of four
// stages and more CTAs per SM, so that more weight bytes are in flight.  In both, rows
// (gathered through `order`) and weight rows come into shared memory in K-blocks of 64 by
// 16-byte asynchronous copies, zero-filled beyond the group's end, the last output and K;
// operands are read with ldmatrix.  With a second weight set both products share the staged
// rows and the epilogue writes act(a) * b.
#include "mma_common.cuh"

namespace {

using namespace nbmma;
typedef __nv_bfloat16 bf16;

constexpr int BN = 64, BK = 64, LD = BK + 8;

// MI: 16-row MMA tiles per warp; WM x WN warps; a warp takes 16 * MI places x 16 * NJ outputs.
template <int MI_, int WM_, int WN_, int NJ_, int STAGES_>
struct Shape {
  static constexpr int MI = MI_, WM = WM_, WN = WN_, NJ = NJ_, STAGES = STAGES_;
  static constexpr int BM = 16 * MI * WM, THREADS = 32 * WM * WN;
  static_assert(16 * NJ * WN == BN, "the warps cover the tile's outputs");
};
typedef Shape<2, 4, 2, 2, 3> Large;    // 128 places, 256 threads
typedef Shape<1, 1, 4, 1, 4> Small;    // 16 places, 128 threads

// Groups are either given by `offsets` (group e = places offsets[e] .. offsets[e+1]; a place's
// source row is order[place] / row_div, or the place itself) or, with `uniform_rows` > 0, every
// group has rows 0 .. uniform_rows - 1, reads columns e * x_gcol .. of x and writes columns
// e * y_gcol .. of y; rows with a negative `row_slot` then give zeros, and with `gate` the
// result is multiplied by sigmoid(gate[row][gate_col + e]).
template <typename S, bool DUAL, typename TX, typename TY>
__global__ void __launch_bounds__(S::THREADS)
moe_mma_kernel(const TX* x, int x_stride, const int* order, int row_div, const int* offsets,
               int n_experts, const bf16* __restrict__ W, const bf16* __restrict__ W2, TY* y,
               int y_stride, int N, int K, int act, float act_param, int uniform_rows, int x_gcol, int y_gcol,
               const int* row_slot, const float* gate, int gate_stride, int gate_col) {
  constexpr int BM = S::BM, THREADS = S::THREADS, STAGES = S::STAGES, MI = S::MI, NJ = S::NJ;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* As = reinterpret_cast<bf16*>(smem_raw);       // [STAGES][BM][LD]
  bf16* Ws = As + STAGES * BM * LD;                    // [STAGES][BN][LD]
  bf16* Ws2 = Ws + STAGES * BN * LD;                   // [STAGES][BN][LD] when DUAL
  __shared__ int a_row[BM];

  int tile = blockIdx.x, e = 0, begin = 0, end = 0;
  if (uniform_rows > 0) {
    const int per = (uniform_rows + BM - 1) / BM;
    e = tile / per;
    tile -= e * per;
    end = uniform_rows;
  } else {
    for (; e < n_experts; ++e) {
      begin = offsets[e];
      end = offsets[e + 1];
      const int t = (end - begin + BM - 1) / BM;
      if (tile < t) break;
      tile -= t;
    }
  }
  if (e >= n_experts) return;
  const int m0 = begin + tile * BM, n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < BM; i += THREADS) {
    const int p = m0 + i;
    int src = p < end ? (order != nullptr ? order[p] / row_div : p) : -1;
    if (src >= 0 && uniform_rows > 0 && row_slot[src] < 0) src = -1;
    a_row[i] = src;
  }
  __syncthreads();
  x += (size_t)e * x_gcol;
  y += (size_t)e * y_gcol;
  // 32-bit rows can be fetched 16 bytes at a time when every row's piece starts on such a boundary
  const bool x_vec4 = sizeof(TX) == 4 && x_stride % 4 == 0 && x_gcol % 4 == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const bf16* We = W + (size_t)e * N * K;
  const bf16* We2 = DUAL ? W2 + (size_t)e * N * K : nullptr;

  auto load_stage = [&](int stage, int k0) {
    if constexpr (sizeof(TX) == 2) {
      for (int i = tid; i < BM * (BK / 8); i += THREADS) {
        const int rr = i >> 3, k = k0 + (i & 7) * 8;
        const int src = a_row[rr];
        const bool ok = src >= 0 && k < K;
        cp_async16_zfill(As + (stage * BM + rr) * LD + (i & 7) * 8,
                         ok ? x + (size_t)src * x_stride + k : x, ok);
      }
    } else if (x_vec4) {   // 32-bit rows: rounded to bf16 on the way into shared memory
      constexpr int PER = (BM * BK / 4 + THREADS - 1) / THREADS;
      float4 v[PER];
#pragma unroll
      for (int u = 0; u < PER; ++u) {      // all loads first, then the stores
        const int i = tid + u * THREADS, rr = i / (BK / 4), k = k0 + (i % (BK / 4)) * 4;
        const int src = rr < BM ? a_row[rr] : -1;
        v[u] = (src >= 0 && k < K)
                   ? *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)src * x_stride + k)
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const int i = tid + u * THREADS, rr = i / (BK / 4), kk = (i % (BK / 4)) * 4;
        if (rr >= BM) continue;
        uint2 pk;
        pk.x = pack_bf16(v[u].x, v[u].y);
        pk.y = pack_bf16(v[u].z, v[u].w);
        *reinterpret_cast<uint2*>(As + (stage * BM + rr) * LD + kk) = pk;
      }
    } else {
      for (int i = tid; i < BM * BK; i += THREADS) {
        const int rr = i / BK, kk = i % BK;
        const int src = a_row[rr];
        const float v = (src >= 0 && k0 + kk < K) ? nb_to_f32(x[(size_t)src * x_stride + k0 + kk]) : 0.0f;
        As[(stage * BM + rr) * LD + kk] = __float2bfloat16_rn(v);
      }
    }
    for (int i = tid; i < BN * (BK / 8); i += THREADS) {
      const int rr = i >> 3, k = k0 + (i & 7) * 8;
      const bool ok = n0 + rr < N && k < K;
      const size_t off = (size_t)(n0 + rr) * K + k;
      cp_async16_zfill(Ws + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We + off : We, ok);
      if (DUAL) cp_async16_zfill(Ws2 + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We2 + off : We2, ok);
    }
  };

  const int wm = warp / S::WN, wn = warp % S::WN;      // the warp's places and outputs
  const int row_w = wm * 16 * MI, col_w = wn * 16 * NJ;
  float acc[MI][2 * NJ][4], acc2[DUAL ? MI : 1][2 * NJ][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < 2 * NJ; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
#pragma unroll
  for (int i = 0; i < (DUAL ? MI : 1); ++i)
#pragma unroll
    for (int j = 0; j < 2 * NJ; ++j) acc2[i][j][0] = acc2[i][j][1] = acc2[i][j][2] = acc2[i][j][3] = 0.0f;
  const bool warp_has_rows = m0 + row_w < end;

  const int n_k = (K + BK - 1) / BK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_k) load_stage(st, st * BK);
    cp_async_commit();
  }
  for (int kt = 0; kt < n_k; ++kt) {
    const int stage = kt % STAGES;
    cp_async_wait<STAGES - 2>();
    __syncthreads();          // block kt has landed, and every warp is done with block kt - 1
    if (kt + STAGES - 1 < n_k) load_stage((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * BK);
    cp_async_commit();
    if (warp_has_rows) {
      const bf16* A = As + stage * BM * LD;
      const bf16* B = Ws + stage * BN * LD;
      const bf16* B2 = Ws2 + stage * BN * LD;
#pragma unroll
      for (int kk = 0; kk < BK / 16; ++kk) {
        uint32_t a[MI][4];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
          ldmatrix_x4(a[mi], A + (row_w + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD +
                                 kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int off = (col_w + j * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 +
                          ((lane >> 3) & 1) * 8;
          uint32_t b[4];
          ldmatrix_x4(b, B + off);
#pragma unroll
          for (int mi = 0; mi < MI; ++mi) {
            mma_bf16(acc[mi][2 * j], a[mi], b[0], b[1]);
            mma_bf16(acc[mi][2 * j + 1], a[mi], b[2], b[3]);
          }
          if (DUAL) {
            ldmatrix_x4(b, B2 + off);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
              mma_bf16(acc2[mi][2 * j], a[mi], b[0], b[1]);
              mma_bf16(acc2[mi][2 * j + 1], a[mi], b[2], b[3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  if (!warp_has_rows) return;
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int local = row_w + mi * 16 + g + half * 8;
      const int p = m0 + local;
      if (p >= end) continue;
      float scale = 1.0f;
      if (uniform_rows > 0) {
        if (a_row[local] < 0) scale = 0.0f;
        else if (gate != nullptr) scale = nb_sigmoid(gate[(size_t)p * gate_stride + gate_col + e]);
      }
#pragma unroll
      for (int nt = 0; nt < 2 * NJ; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + col_w + nt * 8 + 2 * t4 + c;
          if (n >= N) continue;
          float v = acc[mi][nt][2 * half + c];
          if (DUAL) v = nb_gate_up<true>(v, acc2[mi][nt][2 * half + c], act, act_param);
          else v = nb_apply_act_fast(v, act);
          y[(size_t)p * y_stride + n] = nb_from_f32<TY>(scale == 0.0f ? 0.0f : v * scale);
        }
      }
    }
  }
}

struct Uniform {      // the per-head form (see the kernel)
  int rows = 0, x_gcol = 0, y_gcol = 0;
  const int* row_slot = nullptr;
  const float* gate = nullptr;
  int gate_stride = 0, gate_col = 0;
};

// Tiles of a launch: `places` places in `groups` groups (each group rounds up on its own).
template <typename S>
int tiles_of(int places, int groups) {
  return (places + S::BM - 1) / S::BM + (groups < places ? groups : places);
}

template <typename S, bool DUAL, typename TX, typename TY>
int launch(int tiles, cudaStream_t stream, const TX* x, int x_stride, const int* order, int row_div,
           const int* offsets, int n_experts, const bf16* W, const bf16* W2, TY* y, int y_stride,
           int N, int K, int act, float act_param, Uniform u = Uniform()) {
  const size_t smem = (size_t)S::STAGES * (S::BM + BN * (DUAL ? 2 : 1)) * LD * sizeof(bf16);
  static bool set = false;
  if (!set) {
    NB_CUDA(cudaFuncSetAttribute(moe_mma_kernel<S, DUAL, TX, TY>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  const dim3 grid(tiles, (N + BN - 1) / BN);
  NB_REQUIRE(grid.y <= 65535, NB_ERR_UNSUPPORTED, "grouped product: %d outputs are too many", N);
  NB_CUDA(nb_launch(moe_mma_kernel<S, DUAL, TX, TY>, grid, dim3(S::THREADS), smem, stream, x, x_stride,
                    order, row_div, offsets, n_experts, W, W2, y, y_stride, N, K, act, act_param, u.rows, u.x_gcol,
                    u.y_gcol, u.row_slot, u.gate, u.gate_stride, u.gate_col));
  return 0;
}

// Few places: the shape with 16-place tiles.
constexpr int SMALL_MAX_PLACES = 256;

}  // namespace

NB_EXPORT int nb_moe_gemm_mma_supported(int x_dtype, int w_dtype, int x_stride, int K) {
  return x_dtype == NB_BF16 && w_dtype == NB_BF16 && K % 8 == 0 && x_stride % 8 == 0;
}

NB_EXPORT int nb_moe_gemm_mma(const void* x, int x_stride, const int* order, int row_div,
                              const int* offsets, int n_experts, int n_pairs, const void* W,
                              const void* W2, void* y, int y_dtype, int y_stride, int N, int K, int act, float act_param,
                              cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  NB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0 && n_experts >= 1 && row_div >= 1,
             NB_ERR_BAD_ARG, "moe_gemm_mma: bad sizes N=%d K=%d stride=%d", N, K, x_stride);
  NB_REQUIRE(((uintptr_t)x | (uintptr_t)W | (uintptr_t)W2) % 16 == 0, NB_ERR_BAD_ARG,
             "moe_gemm_mma: pointers must be 16-byte aligned");
  NB_REQUIRE(y_dtype == NB_BF16 || y_dtype == NB_F32, NB_ERR_BAD_ARG,
             "moe_gemm_mma: unknown output dtype %d", y_dtype);
  int rc;
  const bf16* xb = (const bf16*)x;
  const bf16* w = (const bf16*)W;
  const bf16* w2 = (const bf16*)W2;
#define NB_GO(S_, DUAL_, TY_)                                                                       \
  rc = launch<S_, DUAL_, bf16, TY_>(tiles_of<S_>(n_pairs, n_experts), stream, xb, x_stride, order,   \
                                    row_div, offsets, n_experts, w, w2, (TY_*)y, y_stride, N, K, act, act_param)
  if (n_pairs <= SMALL_MAX_PLACES) {
    if (y_dtype == NB_BF16) { if (W2) NB_GO(Small, true, bf16); else NB_GO(Small, false, bf16); }
    else { if (W2) NB_GO(Small, true, float); else NB_GO(Small, false, float); }
  } else {
    if (y_dtype == NB_BF16) { if (W2) NB_GO(Large, true, bf16); else NB_GO(Large, false, bf16); }
    else { if (W2) NB_GO(Large, true, float); else NB_GO(Large, false, float); }
  }
#undef NB_GO
  if (rc) return rc;
  NB_CHECK_LAUNCH("moe_gemm_mma");
  return 0;
}

// The per-head linear map (the contract of nb_head_linear) for bf16 weights and bf16 results;
// x: bf16 or fp32 rows (fp32 is rounded to bf16 on the way in).
NB_EXPORT int nb_head_linear_mma_supported(int x_dtype, int w_dtype, int y_dtype, int x_stride,
                                           int x_col, int n_in) {
  return w_dtype == NB_BF16 && y_dtype == NB_BF16 && n_in % 8 == 0 &&
         (x_dtype == NB_F32 || (x_dtype == NB_BF16 && x_stride % 8 == 0 && x_col % 8 == 0));
}

NB_EXPORT int nb_head_linear_mma(const void* x, int x_dtype, int x_stride, int x_col, const void* W,
                                 void* y, int y_stride, const float* gate, int gate_stride,
                                 int gate_col, const int* row_slot, int n_rows, int n_heads, int n_in,
                                 int n_out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(nb_head_linear_mma_supported(x_dtype, NB_BF16, NB_BF16, x_stride, x_col, n_in),
             NB_ERR_UNSUPPORTED, "head_linear_mma: shape not supported (in=%d stride=%d col=%d)", n_in,
             x_stride, x_col);
  NB_REQUIRE((uintptr_t)W % 16 == 0 && (x_dtype == NB_F32 || (uintptr_t)x % 16 == 0), NB_ERR_BAD_ARG,
             "head_linear_mma: pointers must be 16-byte aligned");
  Uniform u;
  u.rows = n_rows; u.x_gcol = n_in; u.y_gcol = n_out; u.row_slot = row_slot;
  u.gate = gate; u.gate_stride = gate_stride; u.gate_col = gate_col;
  int rc;
#define NB_GO(S_, TX_)                                                                               \
  rc = launch<S_, false, TX_, bf16>(((n_rows + S_::BM - 1) / S_::BM) * n_heads, stream,               \
                                    (const TX_*)x + x_col, x_stride, nullptr, 1, nullptr, n_heads,    \
                                    (const bf16*)W, nullptr, (bf16*)y, y_stride, n_out, n_in, 0, 0.0f, u)
  if (n_rows <= 16) {
    if (x_dtype == NB_F32) NB_GO(Small, float); else NB_GO(Small, bf16);
  } else {
    if (x_dtype == NB_F32) NB_GO(Large, float); else NB_GO(Large, bf16);
  }
#undef NB_GO
  if (rc) return rc;
  NB_CHECK_LAUNCH("head_linear_mma");
  return 0;
}
