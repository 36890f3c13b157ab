// Linear attention with a fixed decay per head: a matrix state S (key channels x value channels,
// fp32, zero at a sequence's start) that every token decays, feeds and reads,
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
//
// with q, k, v = act(projections) (the activation applied here, in fp32).  The state of a
// sequence lives in its fixed-size state row ([heads][d][dv]) between steps.
//
// A CTA takes one sequence, one head and a block of value columns, and walks the step's tokens
// in order.  A value column's d state numbers sit in the registers of LANES neighbouring lanes
// (d / LANES each, at most 32); a token costs a thread two multiply-adds per state number, and
// the lanes' parts of o are added up by shuffles.  Tokens are staged in chunks of 16: the
// chunk's activated queries and keys of the head and the values of the CTA's columns go to
// shared memory in one cooperative pass.
#include "common.cuh"

namespace {

constexpr int LA_CHUNK = 16;
constexpr int LA_PER = 32;        // state numbers a thread holds

template <int LANES>
__global__ void __launch_bounds__(256)
linear_attention_kernel(const float* src, int stride, int col_q, int col_k, int col_v, int act,
                        const float* __restrict__ decay, float* state, int state_stride,
                        const int* cu_rows, const int* seq_slot, int n_heads, int d, int dv,
                        int cols_per_cta, float* out) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ float la_smem[];
  float* q_s = la_smem;                       // [CHUNK][d]
  float* k_s = q_s + LA_CHUNK * d;            // [CHUNK][d]
  float* v_s = k_s + LA_CHUNK * d;            // [CHUNK][cols_per_cta]
  const int s = blockIdx.z, h = blockIdx.y;
  const int slot = seq_slot[s];
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (slot < 0 || n_q <= 0) return;
  const int tid = threadIdx.x;
  const int col_local = tid / LANES, part = tid % LANES;
  const int j0 = blockIdx.x * cols_per_cta;
  const int j = j0 + col_local;
  const bool live = col_local < cols_per_cta && j < dv;
  const int per = (d + LANES - 1) / LANES;    // key channels of this lane: part*per .. +per
  const int i0 = part * per;
  float S[LA_PER];
  float* st = state + (size_t)slot * state_stride + (size_t)h * d * dv;
#pragma unroll
  for (int a = 0; a < LA_PER; ++a) {
    const int i = i0 + a;
    S[a] = (live && a < per && i < d) ? st[(size_t)i * dv + j] : 0.0f;
  }
  const float w = decay[h];
  const int n_cols = min(cols_per_cta, dv - j0);

  for (int t0 = 0; t0 < n_q; t0 += LA_CHUNK) {
    const int nt = min(LA_CHUNK, n_q - t0);
    __syncthreads();
    for (int e = tid; e < nt * d; e += blockDim.x) {
      const int t = e / d, i = e - t * d;
      const float* row = src + (size_t)(row0 + t0 + t) * stride;
      q_s[e] = nb_apply_act(row[col_q + h * d + i], act);
      k_s[e] = nb_apply_act(row[col_k + h * d + i], act);
    }
    for (int e = tid; e < nt * n_cols; e += blockDim.x) {
      const int t = e / n_cols, c = e - t * n_cols;
      v_s[t * cols_per_cta + c] =
          nb_apply_act(src[(size_t)(row0 + t0 + t) * stride + col_v + h * dv + j0 + c], act);
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = live ? v_s[t * cols_per_cta + col_local] : 0.0f;
      const float* qt = q_s + t * d + i0;
      const float* kt = k_s + t * d + i0;
      float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
      for (int a = 0; a < LA_PER; a += 2) {
        if (a < per && i0 + a < d) {
          S[a] = fmaf(w, S[a], kt[a] * v);
          o0 = fmaf(S[a], qt[a], o0);
        }
        if (a + 1 < per && i0 + a + 1 < d) {
          S[a + 1] = fmaf(w, S[a + 1], kt[a + 1] * v);
          o1 = fmaf(S[a + 1], qt[a + 1], o1);
        }
      }
      float o = o0 + o1;
#pragma unroll
      for (int m = LANES / 2; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (live && part == 0)
        out[(size_t)(row0 + t0 + t) * n_heads * dv + (size_t)h * dv + j] = o;
    }
  }
  if (live)
#pragma unroll
    for (int a = 0; a < LA_PER; ++a) {
      const int i = i0 + a;
      if (a < per && i < d) st[(size_t)i * dv + j] = S[a];
    }
}

}  // namespace

NB_EXPORT int nb_linear_attention_supported(int d, int dv) {
  return d >= 1 && d <= 32 * LA_PER && dv >= 1 ? 1 : 0;
}

// src: fp32 [rows][stride], the heads' queries at col_q .. (n_heads*d), keys at col_k ..,
// values at col_v .. (n_heads*dv), all before their activation `act`; decay: fp32 [n_heads];
// state: a sequence's row at state + slot * state_stride holds [n_heads][d][dv]; out: fp32
// [rows][n_heads*dv] (the heads' results before any norm).
NB_EXPORT int nb_linear_attention(const float* src, int stride, int col_q, int col_k, int col_v,
                                  int act, const float* decay, float* state, int state_stride,
                                  const int* cu_rows, const int* seq_slot, int n_heads, int d,
                                  int dv, float* out, int n_seqs, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  NB_REQUIRE(n_heads > 0 && n_heads <= 65535 && n_seqs <= 65535 &&
                 nb_linear_attention_supported(d, dv) && state != nullptr && decay != nullptr,
             NB_ERR_BAD_ARG, "linear_attention: bad sizes heads=%d d=%d dv=%d", n_heads, d, dv);
  int lanes = 1;
  while (lanes * LA_PER < d) lanes *= 2;                 // 1, 2, 4, ..., 32
  const int max_cols = 256 / lanes;
  const int cols = dv < max_cols ? dv : max_cols;
  const int threads = ((cols * lanes + 31) / 32) * 32;
  const dim3 grid((dv + cols - 1) / cols, n_heads, n_seqs);
  const size_t smem = (size_t)LA_CHUNK * (2 * d + cols) * sizeof(float);
#define NB_LA(L_)                                                                                 \
  case L_: {                                                                                      \
    auto kern = linear_attention_kernel<L_>;                                                      \
    if (smem > 48 * 1024)                                                                         \
      NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    NB_CUDA(nb_launch_serial(kern, grid, dim3(threads), smem, stream, src, stride, col_q, col_k,  \
                             col_v, act, decay, state, state_stride, cu_rows, seq_slot, n_heads,  \
                             d, dv, cols, out));                                                  \
  } break;
  switch (lanes) {
    NB_LA(1) NB_LA(2) NB_LA(4) NB_LA(8) NB_LA(16) NB_LA(32)
    default: NB_REQUIRE(false, NB_ERR_UNSUPPORTED, "linear_attention: heads of %d", d);
  }
#undef NB_LA
  NB_CHECK_LAUNCH("linear_attention");
  return 0;
}
