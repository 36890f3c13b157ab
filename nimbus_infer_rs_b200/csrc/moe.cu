// A feed-forward of routed experts: every token is run through `top` of `n_experts` small
// gated feed-forwards and the results are added up with per-token weights.
//
//   nb_moe_route    scores = softmax(router logits) over all experts (fp32); the `top`
//                   largest per row (of equal scores the lower index), with their scores as
//                   weights (optionally renormalised to sum 1)
//   nb_moe_route_sigmoid  scores = sigmoid(logits); chosen by score + bias among the experts of
//                   the best groups; weights are the scores, renormalised and scaled
//   nb_moe_group    the (row, choice) pairs grouped by expert: offsets[e] .. offsets[e+1] are
//                   the places of expert e's pairs, order[place] = pair, place[pair] = place
//   nb_moe_gemm     a product per expert over its group of rows, tiled; with two weight
//                   sets it gives act(x Wa^T) * (x Wb^T) (the gated first half of an expert),
//                   with one the plain product (the second half)
//   nb_moe_combine  residual[row] += sum_k weight[row, k] * y[place[row, k]], k in order
//
// Everything is read from device memory (no count comes back to the host), so a step with
// routed experts can be recorded in a CUDA graph.  A row's result does not depend on where
// its pair lands inside a group: every output element is one thread's sum over k in a fixed
// order.  This file is arithmetic in fp32 on the CUDA cores for any element types: the
// 32-bit path, and the bf16 path's fallback for shapes its tensor-core kernel leaves out.
#include "common.cuh"

namespace {

constexpr int ROUTE_MAX_PER_LANE = 32;   // n_experts <= 32 * this

// The `top` largest of the lane-distributed values v (entry i of a lane is expert lane + 32 i;
// NEG marks "none" or "taken"), of equal values the lower index: the k-th winner's index goes to
// out_e[k] of every lane and its entry is marked taken.
template <int PL>
__device__ __forceinline__ void route_take_best(float (&v)[PL], int lane, float neg,
                                                float& best, int& best_e) {
  best = neg;
  best_e = 0x7fffffff;
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    const int e = lane + 32 * i;
    if (v[i] > best) { best = v[i]; best_e = e; }     // ascending e within a lane: first wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
    if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
  }
#pragma unroll
  for (int i = 0; i < PL; ++i)
    if (lane + 32 * i == best_e) v[i] = neg;
}

__global__ void moe_route_kernel(const float* logits, int stride, int col, const int* row_slot,
                                 int n_rows, int n_experts, int top, int renormalize, int* idx,
                                 float* weight) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  if (row_slot[r] < 0) {
    for (int k = lane; k < top; k += 32) {
      idx[(size_t)r * top + k] = -1;
      weight[(size_t)r * top + k] = 0.0f;
    }
    return;
  }
  const float* z = logits + (size_t)r * stride + col;
  float v[ROUTE_MAX_PER_LANE];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < n_experts ? z[e] : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = nb_warp_max(m);
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < n_experts ? expf(v[i] - m) : -1.0f;   // scores are >= 0; -1 marks "none"/"taken"
    if (e < n_experts) sum += v[i];
  }
  sum = nb_warp_sum(sum);
  const float inv = 1.0f / sum;
  float chosen_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best;
    int best_e;
    route_take_best(v, lane, -1.0f, best, best_e);
    const float s = best * inv;
    chosen_sum += s;
    if (lane == 0) {
      idx[(size_t)r * top + k] = best_e;
      weight[(size_t)r * top + k] = s;
    }
  }
  if (renormalize) {
    __syncwarp();
    for (int k = lane; k < top; k += 32) weight[(size_t)r * top + k] /= chosen_sum;
  }
}

// Routing by sigmoid scores with a choice bias and groups of experts.  s = sigmoid(z); the choice
// score of expert e is c_e = s_e + bias_e (bias may be null).  With n_groups > 1 the experts form
// n_groups equal groups of neighbours; a group's score is the sum of its `group_top` largest
// choice scores; only the experts of the `keep_groups` groups with the largest scores (of equal
// scores the lower group) can be chosen.  The `top` allowed experts with the largest choice
// scores are chosen (of equal scores the lower index); their weights are their s (without the
// bias), divided by (their sum + norm_eps) when `renormalize`, times `out_scale`.
template <int PL>   // experts a lane holds: n_experts <= 32 * PL
__global__ void moe_route_sigmoid_kernel(const float* logits, int stride, int col,
                                         const float* __restrict__ bias, const int* row_slot,
                                         int n_rows, int n_experts, int top, int n_groups,
                                         int keep_groups, int group_top, int renormalize,
                                         float norm_eps, float out_scale, int* idx, float* weight) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  if (row_slot[r] < 0) {
    for (int k = lane; k < top; k += 32) {
      idx[(size_t)r * top + k] = -1;
      weight[(size_t)r * top + k] = 0.0f;
    }
    return;
  }
  const float* z = logits + (size_t)r * stride + col;
  float s[PL], c[PL];
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < n_experts ? 1.0f / (1.0f + expf(-z[e])) : 0.0f;
    c[i] = e < n_experts ? s[i] + (bias != nullptr ? bias[e] : 0.0f) : -INFINITY;
  }
  if (n_groups > 1 && keep_groups < n_groups) {
    // group scores: lane g (+ 32 j) owns group g; every group's `group_top` largest are taken
    // from a copy of the choice scores, one group after the other
    const int per = n_experts / n_groups;
    float gs[PL];     // gs[j]: score of group lane + 32 j
#pragma unroll
    for (int j = 0; j < PL; ++j) gs[j] = -INFINITY;
    for (int g = 0; g < n_groups; ++g) {
      float t[PL];
#pragma unroll
      for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        t[i] = (e >= g * per && e < (g + 1) * per) ? c[i] : -INFINITY;
      }
      float total = 0.0f;
      for (int k = 0; k < group_top && k < per; ++k) {
        float best;
        int best_e;
        route_take_best(t, lane, -INFINITY, best, best_e);
        total += best;
      }
#pragma unroll
      for (int j = 0; j < PL; ++j)
        if (lane + 32 * j == g) gs[j] = total;
    }
    // the kept groups, as a bit per group held by the lane that owns it
    unsigned kept_bits = 0u;          // bit j: group lane + 32 j is kept
    for (int k = 0; k < keep_groups; ++k) {
      float best;
      int best_g;
      route_take_best(gs, lane, -INFINITY, best, best_g);
      if (best_g != 0x7fffffff && (best_g & 31) == lane) kept_bits |= 1u << (best_g >> 5);
    }
#pragma unroll
    for (int i = 0; i < PL; ++i) {
      const int e = lane + 32 * i;
      const int g = min(e, n_experts - 1) / per;        // every lane takes part in the shuffle
      const unsigned bits = __shfl_sync(0xffffffffu, kept_bits, g & 31);
      if (e < n_experts && !((bits >> (g >> 5)) & 1u)) c[i] = -INFINITY;
    }
  }
  float chosen_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best;
    int best_e;
    route_take_best(c, lane, -INFINITY, best, best_e);
    float sv = 0.0f;
#pragma unroll
    for (int i = 0; i < PL; ++i)
      if (lane + 32 * i == best_e) sv = s[i];
    sv = nb_warp_sum(sv);             // one lane holds it, the others zero
    chosen_sum += sv;
    if (lane == 0) {
      idx[(size_t)r * top + k] = best_e == 0x7fffffff ? -1 : best_e;
      weight[(size_t)r * top + k] = sv;
    }
  }
  __syncwarp();
  const float f = (renormalize ? 1.0f / (chosen_sum + norm_eps) : 1.0f) * out_scale;
  for (int k = lane; k < top; k += 32) weight[(size_t)r * top + k] *= f;
}

// One CTA.  counts and cursors live in shared memory ([n_experts] ints each).
__global__ void moe_group_kernel(const int* idx, int n_pairs, int n_experts, int* offsets, int* order,
                                 int* place) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ int sm[];
  int* counts = sm;
  int* cursor = sm + n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += counts[e];
    }
    offsets[n_experts] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < n_experts) {
      const int at = atomicAdd(&cursor[e], 1);
      order[at] = p;
      place[p] = at;
    } else {
      place[p] = -1;
    }
  }
}

// Tiled product per expert group.  Tile: TM places x TN outputs, K in steps of TK.
constexpr int TM = 32, TN = 64, TK = 32, GEMM_THREADS = 256;

template <typename TX, typename TW, typename TY, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS)
moe_gemm_kernel(const TX* x, int x_stride, const int* order, int row_div, const int* offsets,
                int n_experts, const TW* __restrict__ W, const TW* __restrict__ W2, TY* y,
                int y_stride, int N, int K, int act, float act_param) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float As[TM][TK + 1];
  __shared__ float Ws[TN][TK + 1];
  __shared__ float Ws2[DUAL ? TN : 1][TK + 1];
  __shared__ int a_row[TM];

  // which expert and which of its tiles this CTA has
  int tile = blockIdx.x, e = 0, begin = 0, end = 0;
  for (; e < n_experts; ++e) {
    begin = offsets[e];
    end = offsets[e + 1];
    const int t = (end - begin + TM - 1) / TM;
    if (tile < t) break;
    tile -= t;
  }
  if (e >= n_experts) return;
  const int m0 = begin + tile * TM;
  const int n0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  if (tid < TM) {
    const int p = m0 + tid;
    a_row[tid] = p < end ? (order != nullptr ? order[p] / row_div : p) : -1;
  }
  __syncthreads();
  const TW* We = W + (size_t)e * N * K;
  const TW* We2 = DUAL ? W2 + (size_t)e * N * K : nullptr;

  const int ty = tid / 16, tx = tid % 16;     // rows ty*2, ty*2+1; columns tx + 16*c
  float acc[2][4], acc2[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = acc2[i][c] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = tid; i < TM * TK; i += GEMM_THREADS) {
      const int rr = i / TK, kk = i % TK;
      const int src = a_row[rr];
      As[rr][kk] = (src >= 0 && k0 + kk < K) ? nb_to_f32(x[(size_t)src * x_stride + k0 + kk]) : 0.0f;
    }
    for (int i = tid; i < TN * TK; i += GEMM_THREADS) {
      const int nn = i / TK, kk = i % TK;
      const bool ok = n0 + nn < N && k0 + kk < K;
      Ws[nn][kk] = ok ? nb_to_f32(We[(size_t)(n0 + nn) * K + k0 + kk]) : 0.0f;
      if (DUAL) Ws2[nn][kk] = ok ? nb_to_f32(We2[(size_t)(n0 + nn) * K + k0 + kk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float w = Ws[tx + 16 * c][kk];
        acc[0][c] = fmaf(a0, w, acc[0][c]);
        acc[1][c] = fmaf(a1, w, acc[1][c]);
        if (DUAL) {
          const float w2 = Ws2[tx + 16 * c][kk];
          acc2[0][c] = fmaf(a0, w2, acc2[0][c]);
          acc2[1][c] = fmaf(a1, w2, acc2[1][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = m0 + ty * 2 + i;
    if (p >= end) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx + 16 * c;
      if (n >= N) continue;
      float v = acc[i][c];
      if (DUAL) v = nb_gate_up<false>(v, acc2[i][c], act, act_param);
      else v = nb_apply_act(v, act);
      y[(size_t)p * y_stride + n] = nb_from_f32<TY>(v);
    }
  }
}

__global__ void moe_combine_kernel(const float* y, int width, const int* place, const float* weight,
                                   int top, float* residual) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int at = place[(size_t)r * top + k];
      if (at >= 0) s = fmaf(weight[(size_t)r * top + k], y[(size_t)at * width + i], s);
    }
    residual[(size_t)r * width + i] += s;
  }
}

}  // namespace

typedef __nv_bfloat16 bf16;

NB_EXPORT int nb_moe_route(const float* logits, int stride, int col, const int* row_slot, int n_rows,
                           int n_experts, int top, int renormalize, int* idx, float* weight,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_experts >= 1 && n_experts <= 32 * ROUTE_MAX_PER_LANE, NB_ERR_UNSUPPORTED,
             "moe_route: %d experts are outside 1..%d", n_experts, 32 * ROUTE_MAX_PER_LANE);
  NB_REQUIRE(top >= 1 && top <= n_experts, NB_ERR_BAD_ARG, "moe_route: top=%d of %d experts", top,
             n_experts);
  NB_REQUIRE(col >= 0 && stride >= col + n_experts, NB_ERR_BAD_ARG, "moe_route: bad columns");
  NB_CUDA(nb_launch(moe_route_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream, logits, stride,
                    col, row_slot, n_rows, n_experts, top, renormalize, idx, weight));
  NB_CHECK_LAUNCH("moe_route");
  return 0;
}

// bias: fp32 [n_experts] or null; n_groups <= 1: no groups.
NB_EXPORT int nb_moe_route_sigmoid(const float* logits, int stride, int col, const float* bias,
                                   const int* row_slot, int n_rows, int n_experts, int top,
                                   int n_groups, int keep_groups, int group_top, int renormalize,
                                   float norm_eps, float out_scale, int* idx, float* weight,
                                   cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_experts >= 1 && n_experts <= 32 * ROUTE_MAX_PER_LANE, NB_ERR_UNSUPPORTED,
             "moe_route_sigmoid: %d experts are outside 1..%d", n_experts, 32 * ROUTE_MAX_PER_LANE);
  NB_REQUIRE(top >= 1 && top <= n_experts, NB_ERR_BAD_ARG, "moe_route_sigmoid: top=%d of %d experts",
             top, n_experts);
  NB_REQUIRE(col >= 0 && stride >= col + n_experts, NB_ERR_BAD_ARG, "moe_route_sigmoid: bad columns");
  if (n_groups > 1)
    NB_REQUIRE(n_experts % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups &&
                   group_top >= 1 && keep_groups * (n_experts / n_groups) >= top,
               NB_ERR_BAD_ARG, "moe_route_sigmoid: %d groups (keep %d, top %d of each) of %d experts, top=%d",
               n_groups, keep_groups, group_top, n_experts, top);
#define NB_RS(PL_)                                                                               \
  NB_CUDA(nb_launch(moe_route_sigmoid_kernel<PL_>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, \
                    logits, stride, col, bias, row_slot, n_rows, n_experts, top, n_groups,       \
                    keep_groups, group_top, renormalize, norm_eps, out_scale, idx, weight))
  if (n_experts <= 32) NB_RS(1);
  else if (n_experts <= 64) NB_RS(2);
  else if (n_experts <= 256) NB_RS(8);
  else NB_RS(ROUTE_MAX_PER_LANE);
#undef NB_RS
  NB_CHECK_LAUNCH("moe_route_sigmoid");
  return 0;
}

NB_EXPORT int nb_moe_group(const int* idx, int n_pairs, int n_experts, int* offsets, int* order,
                           int* place, cudaStream_t stream) {
  NB_REQUIRE(n_pairs >= 0 && n_experts >= 1 && n_experts <= 4096, NB_ERR_BAD_ARG,
             "moe_group: bad sizes pairs=%d experts=%d", n_pairs, n_experts);
  NB_CUDA(nb_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * n_experts * sizeof(int),
                    stream, idx, n_pairs, n_experts, offsets, order, place));
  NB_CHECK_LAUNCH("moe_group");
  return 0;
}

// How many row tiles a launch over `n_pairs` pairs of `n_experts` experts can need at most.
NB_EXPORT int nb_moe_gemm_tiles(int n_pairs, int n_experts) {
  return (n_pairs + TM - 1) / TM + (n_experts < n_pairs ? n_experts : n_pairs);
}

// y[place, :] = f(x[row(place), :]) for every place of every expert's group, where
// row(place) = order[place] / row_div if `order` is given, else place itself;
// f = act(x We^T), or act(x We^T) * (x We2^T) when W2 is given.  W, W2: [n_experts][N][K].
NB_EXPORT int nb_moe_gemm(const void* x, int x_dtype, int x_stride, const int* order, int row_div,
                          const int* offsets, int n_experts, int n_pairs, const void* W,
                          const void* W2, int w_dtype, void* y, int y_dtype, int y_stride, int N,
                          int K, int act, float act_param, cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  NB_REQUIRE(N > 0 && K > 0 && n_experts >= 1 && row_div >= 1, NB_ERR_BAD_ARG,
             "moe_gemm: bad sizes N=%d K=%d experts=%d", N, K, n_experts);
  const dim3 grid(nb_moe_gemm_tiles(n_pairs, n_experts), (N + TN - 1) / TN);
  NB_REQUIRE(grid.y <= 65535, NB_ERR_UNSUPPORTED, "moe_gemm: %d outputs are too many", N);
#define NB_MG(TX, TW, TY)                                                                          \
  do {                                                                                             \
    if (W2 != nullptr)                                                                             \
      NB_CUDA(nb_launch(moe_gemm_kernel<TX, TW, TY, true>, grid, dim3(GEMM_THREADS), 0, stream,    \
                        (const TX*)x, x_stride, order, row_div, offsets, n_experts, (const TW*)W,  \
                        (const TW*)W2, (TY*)y, y_stride, N, K, act, act_param));                              \
    else                                                                                           \
      NB_CUDA(nb_launch(moe_gemm_kernel<TX, TW, TY, false>, grid, dim3(GEMM_THREADS), 0, stream,   \
                        (const TX*)x, x_stride, order, row_div, offsets, n_experts, (const TW*)W,  \
                        (const TW*)W2, (TY*)y, y_stride, N, K, act, act_param));                              \
  } while (0)
  const int key = x_dtype * 4 + w_dtype * 2 + y_dtype;
  switch (key) {
    case 0: NB_MG(float, float, float); break;
    case 1: NB_MG(float, float, bf16); break;
    case 2: NB_MG(float, bf16, float); break;
    case 3: NB_MG(float, bf16, bf16); break;
    case 4: NB_MG(bf16, float, float); break;
    case 5: NB_MG(bf16, float, bf16); break;
    case 6: NB_MG(bf16, bf16, float); break;
    case 7: NB_MG(bf16, bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "moe_gemm: unknown dtypes %d/%d/%d", x_dtype, w_dtype, y_dtype);
  }
#undef NB_MG
  NB_CHECK_LAUNCH("moe_gemm");
  return 0;
}

NB_EXPORT int nb_moe_combine(const float* y, int width, const int* place, const float* weight,
                             int top, float* residual, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(width > 0 && top >= 1, NB_ERR_BAD_ARG, "moe_combine: bad sizes");
  // a thread per element of the stream while the launch stays small; rows of a long prompt
  // walk over their width instead
  const int threads = 128;
  const int chunks = n_rows <= 256 ? (width + threads - 1) / threads : (width + 4 * threads - 1) / (4 * threads);
  NB_CUDA(nb_launch(moe_combine_kernel, dim3(n_rows, chunks), dim3(threads), 0, stream, y, width,
                    place, weight, top, residual));
  NB_CHECK_LAUNCH("moe_combine");
  return 0;
}
