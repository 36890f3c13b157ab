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
// (16 each, in groups of four consecutive key channels, so that a lane reads its part of a
// token's key and query as 16-byte pieces and the lanes of a column read consecutive pieces);
// a token costs a thread two multiply-adds per state number, and the lanes' parts of o are
// added up by shuffles.  Tokens are staged in chunks of 16 through two buffers of shared
// memory: while one chunk is walked, asynchronous copies bring the next one's queries and keys
// of the head and values of the CTA's columns; the activation is applied in place once the
// chunk has landed.  Rows of the buffers are LANES * 16 wide; what lies beyond d stays zero, so
// that the walk needs no bounds.  The columns of a CTA are chosen by the launcher so that the
// grid fills the GPU.
#include "common.cuh"

namespace {

constexpr int LA_CHUNK = 16;
constexpr int LA_PER = 16;        // state numbers a thread holds

__device__ __forceinline__ void la_copy4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void la_copy16(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}

template <int LANES>
__global__ void __launch_bounds__(256)
linear_attention_kernel(const float* src, int stride, int col_q, int col_k, int col_v, int act,
                        const float* __restrict__ decay, float* state, int state_stride,
                        const int* cu_rows, const int* seq_slot, int n_heads, int d, int dv,
                        int cols_per_cta, float* out) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  constexpr int DS = LANES * LA_PER;          // a staged row of queries or keys
  extern __shared__ __align__(16) float la_smem[];
  const int buf_floats = LA_CHUNK * (2 * DS + cols_per_cta);   // [CHUNK][DS] q, k; [CHUNK][cols] v
  const int s = blockIdx.z, h = blockIdx.y;
  const int slot = seq_slot[s];
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (slot < 0 || n_q <= 0) return;
  const int tid = threadIdx.x, n_threads = blockDim.x;
  const int col_local = tid / LANES, part = tid % LANES;
  const int j0 = blockIdx.x * cols_per_cta;
  const int j = j0 + col_local;
  const bool live = col_local < cols_per_cta && j < dv;
  const int n_cols = min(cols_per_cta, dv - j0);
  // state number a of this lane is key channel chan(a)
  auto chan = [&](int a) { return (a >> 2) * (LANES * 4) + part * 4 + (a & 3); };
  float S[LA_PER];
  float* st = state + (size_t)slot * state_stride + (size_t)h * d * dv;
#pragma unroll
  for (int a = 0; a < LA_PER; ++a) S[a] = (live && chan(a) < d) ? st[(size_t)chan(a) * dv + j] : 0.0f;
  const float w = decay[h];
  for (int i = tid; i < 2 * buf_floats; i += n_threads) la_smem[i] = 0.0f;
  __syncthreads();

  // 16-byte copies where every piece starts on a 16-byte boundary on both sides
  const bool wide_qk = (d % 4 == 0) && (stride % 4 == 0) && ((col_q + h * d) % 4 == 0) &&
                       ((col_k + h * d) % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  const bool wide_v = wide_qk && (n_cols % 4 == 0) && (cols_per_cta % 4 == 0) &&
                      ((col_v + h * dv + j0) % 4 == 0);
  auto issue = [&](int t0, float* buf) {
    const int nt = min(LA_CHUNK, n_q - t0);
    float* q_s = buf;
    float* k_s = q_s + LA_CHUNK * DS;
    float* v_s = k_s + LA_CHUNK * DS;
    if (wide_qk) {
      const int d4 = d >> 2;
      for (int e = tid; e < nt * d4; e += n_threads) {
        const int t = e / d4, i = (e - t * d4) * 4;
        const float* row = src + (size_t)(row0 + t0 + t) * stride;
        la_copy16(q_s + t * DS + i, row + col_q + h * d + i);
        la_copy16(k_s + t * DS + i, row + col_k + h * d + i);
      }
    } else {
      for (int e = tid; e < nt * d; e += n_threads) {
        const int t = e / d, i = e - t * d;
        const float* row = src + (size_t)(row0 + t0 + t) * stride;
        la_copy4(q_s + t * DS + i, row + col_q + h * d + i);
        la_copy4(k_s + t * DS + i, row + col_k + h * d + i);
      }
    }
    if (wide_v) {
      const int c4 = n_cols >> 2;
      for (int e = tid; e < nt * c4; e += n_threads) {
        const int t = e / c4, c = (e - t * c4) * 4;
        la_copy16(v_s + t * cols_per_cta + c, src + (size_t)(row0 + t0 + t) * stride + col_v + h * dv + j0 + c);
      }
    } else {
      for (int e = tid; e < nt * n_cols; e += n_threads) {
        const int t = e / n_cols, c = e - t * n_cols;
        la_copy4(v_s + t * cols_per_cta + c, src + (size_t)(row0 + t0 + t) * stride + col_v + h * dv + j0 + c);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  issue(0, la_smem);
  int which = 0;
  for (int t0 = 0; t0 < n_q; t0 += LA_CHUNK, which ^= 1) {
    const int nt = min(LA_CHUNK, n_q - t0);
    float* q_s = la_smem + which * buf_floats;
    float* k_s = q_s + LA_CHUNK * DS;
    float* v_s = k_s + LA_CHUNK * DS;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();     // the chunk is in; everyone is done with the other buffer
    if (t0 + LA_CHUNK < n_q) issue(t0 + LA_CHUNK, la_smem + (which ^ 1) * buf_floats);
    if (act != NB_ACT_NONE) {
      for (int e = tid; e < nt * d; e += n_threads) {
        const int t = e / d, i = e - t * d;
        q_s[t * DS + i] = nb_apply_act(q_s[t * DS + i], act);
        k_s[t * DS + i] = nb_apply_act(k_s[t * DS + i], act);
      }
      for (int e = tid; e < nt * n_cols; e += n_threads) {
        const int t = e / n_cols, c = e - t * n_cols;
        v_s[t * cols_per_cta + c] = nb_apply_act(v_s[t * cols_per_cta + c], act);
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float v = live ? v_s[t * cols_per_cta + col_local] : 0.0f;
      const float4* qt = reinterpret_cast<const float4*>(q_s + t * DS + part * 4);
      const float4* kt = reinterpret_cast<const float4*>(k_s + t * DS + part * 4);
      float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
      for (int g = 0; g < LA_PER / 4; ++g) {
        const float4 k4 = kt[g * LANES], q4 = qt[g * LANES];
        S[4 * g] = fmaf(w, S[4 * g], k4.x * v);
        o0 = fmaf(S[4 * g], q4.x, o0);
        S[4 * g + 1] = fmaf(w, S[4 * g + 1], k4.y * v);
        o1 = fmaf(S[4 * g + 1], q4.y, o1);
        S[4 * g + 2] = fmaf(w, S[4 * g + 2], k4.z * v);
        o0 = fmaf(S[4 * g + 2], q4.z, o0);
        S[4 * g + 3] = fmaf(w, S[4 * g + 3], k4.w * v);
        o1 = fmaf(S[4 * g + 3], q4.w, o1);
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
    for (int a = 0; a < LA_PER; ++a)
      if (chan(a) < d) st[(size_t)chan(a) * dv + j] = S[a];
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
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    NB_CUDA(cudaGetDevice(&dev));
    NB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  // as many columns a CTA as 256 threads hold (the CTAs of a head each stage and activate
  // its queries and keys); fewer, down to a warp's worth, while the grid has fewer CTAs than
  // the GPU has SMs
  int cols = 256 / lanes;
  if (cols > dv) cols = dv;
  while (cols * lanes > 32 && (long long)((dv + cols - 1) / cols) * n_heads * n_seqs < (long long)sms)
    cols = (cols + 1) / 2;
  const int threads = ((cols * lanes + 31) / 32) * 32;
  const dim3 grid((dv + cols - 1) / cols, n_heads, n_seqs);
  const size_t smem = (size_t)2 * LA_CHUNK * (2 * lanes * LA_PER + cols) * sizeof(float);
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
