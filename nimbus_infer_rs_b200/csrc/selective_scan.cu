// The selective scan: per channel c a state of N numbers that every token decays and feeds,
//
//   dt_c   = softplus(dt_lin_c + dt_bias_c)                 (the step size, per token and channel)
//   S[c,n] = exp(dt_c * A[c,n]) * S[c,n] + dt_c * x_c * B_n,      A = -exp(A_log)
//   y_c    = sum_n S[c,n] * C_n + D_c * x_c,      out_c = y_c * silu(z_c)
//
// with B and C (N numbers each) shared by all channels of a token.  All of it fp32; the state of
// a sequence lives in its fixed-size state row ([channels][N]) between steps.
//
// A CTA takes 128 channels of one sequence and walks the step's tokens in order; a thread owns
// a channel with its N state numbers and its row of A in registers.  Tokens are staged in
// chunks of 16: B and C of the chunk and the chunk's step sizes, inputs and gates of the CTA's
// channels go to shared memory in one cooperative pass (softplus applied there), then every
// thread runs the 16 tokens out of shared memory.  Results are written as they come (a warp's
// stores of one token are consecutive).
#include "common.cuh"

namespace {

constexpr int SS_THREADS = 128;
constexpr int SS_CHUNK = 16;

__device__ __forceinline__ float ss_softplus(float x) {
  return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x)));
}

template <int NMAX, typename TOut>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const float* x, const float* low, int low_stride, int col_b, int col_c,
                      const float* dt_lin, const float* __restrict__ dt_bias,
                      const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      const float* zsrc, int z_stride, int z_col, float* state, int state_stride,
                      const int* cu_rows, const int* seq_slot, int inner, int N, TOut* out) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ float ss_smem[];
  float* bc_s = ss_smem;                               // [CHUNK][2N]
  float* dt_s = bc_s + SS_CHUNK * 2 * N;               // [CHUNK][THREADS]
  float* x_s = dt_s + SS_CHUNK * SS_THREADS;
  float* z_s = x_s + SS_CHUNK * SS_THREADS;
  const int s = blockIdx.y;
  const int slot = seq_slot[s];
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (slot < 0 || n_q <= 0) return;     // rows of a sequence that has ended keep what they held
  const int c0 = blockIdx.x * SS_THREADS, tid = threadIdx.x;
  const int c = c0 + tid;
  const bool live = c < inner;
  float S[NMAX], A[NMAX];
  float* st = state + (size_t)slot * state_stride + (size_t)c * N;
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    S[n] = (live && n < N) ? st[n] : 0.0f;
    A[n] = (live && n < N) ? -expf(a_log[(size_t)c * N + n]) : 0.0f;
  }
  const float bias = live ? dt_bias[c] : 0.0f, dsk = live ? d_skip[c] : 0.0f;

  for (int t0 = 0; t0 < n_q; t0 += SS_CHUNK) {
    const int nt = min(SS_CHUNK, n_q - t0);
    __syncthreads();
    for (int i = tid; i < nt * 2 * N; i += SS_THREADS) {
      const int t = i / (2 * N), j = i - t * 2 * N;
      bc_s[i] = low[(size_t)(row0 + t0 + t) * low_stride + (j < N ? col_b + j : col_c + j - N)];
    }
    if (live)
      for (int t = 0; t < nt; ++t) {
        const size_t r = row0 + t0 + t;
        dt_s[t * SS_THREADS + tid] = ss_softplus(dt_lin[r * inner + c] + bias);
        x_s[t * SS_THREADS + tid] = x[r * inner + c];
        z_s[t * SS_THREADS + tid] = zsrc[r * z_stride + z_col + c];
      }
    __syncthreads();
    if (!live) continue;
    for (int t = 0; t < nt; ++t) {
      const float dt = dt_s[t * SS_THREADS + tid], xv = x_s[t * SS_THREADS + tid];
      const float z = z_s[t * SS_THREADS + tid];
      const float dx = dt * xv;
      const float* B = bc_s + t * 2 * N;
      const float* Cv = B + N;
      float y0 = 0.0f, y1 = 0.0f;
#pragma unroll
      for (int n = 0; n < NMAX; n += 2) {
        if (n < N) {
          S[n] = fmaf(expf(dt * A[n]), S[n], dx * B[n]);
          y0 = fmaf(S[n], Cv[n], y0);
        }
        if (n + 1 < N) {
          S[n + 1] = fmaf(expf(dt * A[n + 1]), S[n + 1], dx * B[n + 1]);
          y1 = fmaf(S[n + 1], Cv[n + 1], y1);
        }
      }
      const float y = fmaf(dsk, xv, y0 + y1);
      out[(size_t)(row0 + t0 + t) * inner + c] = nb_from_f32<TOut>(y * nb_silu(z));
    }
  }
  if (live)
#pragma unroll
    for (int n = 0; n < NMAX; ++n)
      if (n < N) st[n] = S[n];
}

template <int NMAX>
int launch_scan(const float* x, const float* low, int low_stride, int col_b, int col_c,
                const float* dt_lin, const float* dt_bias, const float* a_log, const float* d_skip,
                const float* z, int z_stride, int z_col, float* state, int state_stride,
                const int* cu_rows, const int* seq_slot, int inner, int N, void* out, int out_dtype,
                int n_seqs, cudaStream_t stream) {
  const dim3 grid((inner + SS_THREADS - 1) / SS_THREADS, n_seqs);
  const size_t smem = (size_t)(SS_CHUNK * 2 * N + 3 * SS_CHUNK * SS_THREADS) * sizeof(float);
  if (out_dtype == NB_F32) {
    auto kern = selective_scan_kernel<NMAX, float>;
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch_serial(kern, grid, dim3(SS_THREADS), smem, stream, x, low, low_stride, col_b,
                             col_c, dt_lin, dt_bias, a_log, d_skip, z, z_stride, z_col, state,
                             state_stride, cu_rows, seq_slot, inner, N, (float*)out));
  } else {
    auto kern = selective_scan_kernel<NMAX, __nv_bfloat16>;
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch_serial(kern, grid, dim3(SS_THREADS), smem, stream, x, low, low_stride, col_b,
                             col_c, dt_lin, dt_bias, a_log, d_skip, z, z_stride, z_col, state,
                             state_stride, cu_rows, seq_slot, inner, N, (__nv_bfloat16*)out));
  }
  return 0;
}

}  // namespace

NB_EXPORT int nb_selective_scan_supported(int n_state) { return n_state >= 1 && n_state <= 256 ? 1 : 0; }

// x: fp32 [rows][inner] (the channels' inputs after their convolution and activation); low: fp32
// [rows][low_stride] with B at columns col_b .. and C at col_c ..; dt_lin: fp32 [rows][inner];
// dt_bias, d_skip: fp32 [inner]; a_log: fp32 [inner][N]; z: fp32 rows of stride z_stride, the
// gates at columns z_col ..; state: a sequence's row at state + slot * state_stride holds
// [inner][N]; out: [rows][inner].
NB_EXPORT int nb_selective_scan(const float* x, const float* low, int low_stride, int col_b,
                                int col_c, const float* dt_lin, const float* dt_bias,
                                const float* a_log, const float* d_skip, const float* z,
                                int z_stride, int z_col, float* state, int state_stride,
                                const int* cu_rows, const int* seq_slot, int inner, int n_state,
                                void* out, int out_dtype, int n_seqs, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  NB_REQUIRE(inner > 0 && nb_selective_scan_supported(n_state) && n_seqs <= 65535 &&
                 (out_dtype == NB_F32 || out_dtype == NB_BF16) && state != nullptr,
             NB_ERR_BAD_ARG, "selective_scan: bad sizes inner=%d state=%d", inner, n_state);
#define NB_SS(NMAX_)                                                                              \
  rc = launch_scan<NMAX_>(x, low, low_stride, col_b, col_c, dt_lin, dt_bias, a_log, d_skip, z,    \
                          z_stride, z_col, state, state_stride, cu_rows, seq_slot, inner,         \
                          n_state, out, out_dtype, n_seqs, stream)
  int rc;
  if (n_state <= 8) NB_SS(8);
  else if (n_state <= 16) NB_SS(16);
  else if (n_state <= 32) NB_SS(32);
  else if (n_state <= 64) NB_SS(64);
  else if (n_state <= 128) NB_SS(128);
  else NB_SS(256);
#undef NB_SS
  if (rc) return rc;
  NB_CHECK_LAUNCH("selective_scan");
  return 0;
}
