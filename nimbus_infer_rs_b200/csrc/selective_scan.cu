// The selective scan: per channel c a state of N numbers that every token decays and feeds,
//
//   dt_c   = softplus(dt_lin_c + dt_bias_c)                 (the step size, per token and channel)
//   S[c,n] = exp(dt_c * A[c,n]) * S[c,n] + dt_c * x_c * B_n,      A = -exp(A_log)
//   y_c    = sum_n S[c,n] * C_n + D_c * x_c,      out_c = y_c * silu(z_c)
//
// with B and C (N numbers each) shared by all channels of a token.  All of it fp32; the state of
// a sequence lives in its fixed-size state row ([channels][N]) between steps.
//
// A CTA takes a block of channels of one sequence and walks the step's tokens in order.  A
// channel's N state numbers and its row of A sit in the registers of LANES neighbouring lanes
// (NPER each), so that a model with a small state still fills the GPU with CTAs; the lanes'
// parts of y are added up by shuffles.  Tokens are staged in chunks of 16 through two buffers of
// shared memory: while the threads run one chunk, asynchronous copies bring the next one's B
// and C, step sizes, inputs and gates.  The step sizes' softplus is applied once per token and
// channel, in place, before the chunk is used.
#include "common.cuh"

namespace {

constexpr int SS_THREADS = 128;
constexpr int SS_CHUNK = 16;

__device__ __forceinline__ float ss_softplus(float x) {
  return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x)));
}

__device__ __forceinline__ void ss_copy4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}

template <int NPER, int LANES, typename TOut>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const float* x, const float* low, int low_stride, int col_b, int col_c,
                      const float* dt_lin, const float* __restrict__ dt_bias,
                      const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      const float* zsrc, int z_stride, int z_col, float* state, int state_stride,
                      const int* cu_rows, const int* seq_slot, int inner, int N, TOut* out) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  constexpr int CH = SS_THREADS / LANES;               // channels of a CTA
  constexpr int NP = NPER * LANES;                     // a staged row of B or C, N and zeros
  static_assert(NPER % 4 == 0, "a lane reads its part of B and C as 16-byte pieces");
  extern __shared__ __align__(16) float ss_smem[];
  const int buf_floats = SS_CHUNK * (2 * NP + 3 * CH); // [CHUNK][2NP] B|C, then dt, x, z [CHUNK][CH]
  const int s = blockIdx.y;
  const int slot = seq_slot[s];
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (slot < 0 || n_q <= 0) return;     // rows of a sequence that has ended keep what they held
  const int tid = threadIdx.x;
  const int cl = tid / LANES, part = tid % LANES;
  const int c0 = blockIdx.x * CH, c = c0 + cl;
  const int n0 = part * NPER;
  const bool live = c < inner;
  const int n_ch = min(CH, inner - c0);
  float S[NPER], A[NPER];
  float* st = state + (size_t)slot * state_stride + (size_t)c * N;
#pragma unroll
  for (int a = 0; a < NPER; ++a) {
    const bool has = live && n0 + a < N;
    S[a] = has ? st[n0 + a] : 0.0f;
    A[a] = has ? -expf(a_log[(size_t)c * N + n0 + a]) : 0.0f;
  }
  const float dsk = live ? d_skip[c] : 0.0f;
  // the rows of B and C beyond N stay zero, so the walk below needs no bounds (a state number
  // beyond N has A = 0 and stays 0)
  for (int i = tid; i < 2 * buf_floats; i += SS_THREADS) ss_smem[i] = 0.0f;
  __syncthreads();

  auto issue = [&](int t0, float* buf) {
    const int nt = min(SS_CHUNK, n_q - t0);
    float* bc_s = buf;
    float* dt_s = buf + SS_CHUNK * 2 * NP;
    float* x_s = dt_s + SS_CHUNK * CH;
    float* z_s = x_s + SS_CHUNK * CH;
    for (int i = tid; i < nt * 2 * N; i += SS_THREADS) {
      const int t = i / (2 * N), j = i - t * 2 * N;
      const float* row = low + (size_t)(row0 + t0 + t) * low_stride;
      if (j < N) ss_copy4(bc_s + t * 2 * NP + j, row + col_b + j);
      else ss_copy4(bc_s + t * 2 * NP + NP + j - N, row + col_c + j - N);
    }
    for (int i = tid; i < nt * CH; i += SS_THREADS) {
      const int t = i / CH, k = i - t * CH;
      if (k >= n_ch) continue;
      const size_t r = row0 + t0 + t;
      ss_copy4(dt_s + i, dt_lin + r * inner + c0 + k);
      ss_copy4(x_s + i, x + r * inner + c0 + k);
      ss_copy4(z_s + i, zsrc + r * z_stride + z_col + c0 + k);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  issue(0, ss_smem);
  int which = 0;
  for (int t0 = 0; t0 < n_q; t0 += SS_CHUNK, which ^= 1) {
    const int nt = min(SS_CHUNK, n_q - t0);
    float* buf = ss_smem + which * buf_floats;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();     // the chunk is in; everyone is done with the other buffer
    if (t0 + SS_CHUNK < n_q) issue(t0 + SS_CHUNK, ss_smem + (which ^ 1) * buf_floats);
    float* bc_s = buf;
    float* dt_s = buf + SS_CHUNK * 2 * NP;
    const float* x_s = dt_s + SS_CHUNK * CH;
    float* z_s = dt_s + 2 * SS_CHUNK * CH;
    // step sizes and gates once per (token, channel), by all threads, ahead of the walk
    for (int i = tid; i < nt * CH; i += SS_THREADS) {
      const int k = i % CH;
      if (k < n_ch) {
        dt_s[i] = ss_softplus(dt_s[i] + dt_bias[c0 + k]);
        z_s[i] = nb_silu(z_s[i]);
      }
    }
    __syncthreads();
    // (a warp's channels beyond the last one walk along on whatever the buffer holds: the
    // shuffles below want every lane, and nothing of theirs is written)
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float dt = dt_s[t * CH + cl], xv = x_s[t * CH + cl];
      const float dx = dt * xv;
      const float4* B4 = reinterpret_cast<const float4*>(bc_s + t * 2 * NP + n0);
      const float4* C4 = B4 + NP / 4;
      float y0 = 0.0f, y1 = 0.0f;
#pragma unroll
      for (int g = 0; g < NPER / 4; ++g) {
        const float4 b = B4[g], cv = C4[g];
        S[4 * g] = fmaf(expf(dt * A[4 * g]), S[4 * g], dx * b.x);
        y0 = fmaf(S[4 * g], cv.x, y0);
        S[4 * g + 1] = fmaf(expf(dt * A[4 * g + 1]), S[4 * g + 1], dx * b.y);
        y1 = fmaf(S[4 * g + 1], cv.y, y1);
        S[4 * g + 2] = fmaf(expf(dt * A[4 * g + 2]), S[4 * g + 2], dx * b.z);
        y0 = fmaf(S[4 * g + 2], cv.z, y0);
        S[4 * g + 3] = fmaf(expf(dt * A[4 * g + 3]), S[4 * g + 3], dx * b.w);
        y1 = fmaf(S[4 * g + 3], cv.w, y1);
      }
      float y = y0 + y1;
#pragma unroll
      for (int m = LANES / 2; m > 0; m >>= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
      if (part == 0 && live) {
        y = fmaf(dsk, xv, y);
        out[(size_t)(row0 + t0 + t) * inner + c] = nb_from_f32<TOut>(y * z_s[t * CH + cl]);
      }
    }
  }
  if (live)
#pragma unroll
    for (int a = 0; a < NPER; ++a)
      if (n0 + a < N) st[n0 + a] = S[a];
}

template <int NPER, int LANES>
int launch_scan(const float* x, const float* low, int low_stride, int col_b, int col_c,
                const float* dt_lin, const float* dt_bias, const float* a_log, const float* d_skip,
                const float* z, int z_stride, int z_col, float* state, int state_stride,
                const int* cu_rows, const int* seq_slot, int inner, int N, void* out, int out_dtype,
                int n_seqs, cudaStream_t stream) {
  constexpr int CH = SS_THREADS / LANES;
  const dim3 grid((inner + CH - 1) / CH, n_seqs);
  const size_t smem = (size_t)2 * SS_CHUNK * (2 * NPER * LANES + 3 * CH) * sizeof(float);
  if (out_dtype == NB_F32) {
    auto kern = selective_scan_kernel<NPER, LANES, float>;
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch_serial(kern, grid, dim3(SS_THREADS), smem, stream, x, low, low_stride, col_b,
                             col_c, dt_lin, dt_bias, a_log, d_skip, z, z_stride, z_col, state,
                             state_stride, cu_rows, seq_slot, inner, N, (float*)out));
  } else {
    auto kern = selective_scan_kernel<NPER, LANES, __nv_bfloat16>;
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
#define NB_SS(NPER_, LANES_)                                                                      \
  rc = launch_scan<NPER_, LANES_>(x, low, low_stride, col_b, col_c, dt_lin, dt_bias, a_log,       \
                                  d_skip, z, z_stride, z_col, state, state_stride, cu_rows,       \
                                  seq_slot, inner, n_state, out, out_dtype, n_seqs, stream)
  int rc;
  if (n_state <= 4) NB_SS(4, 1);
  else if (n_state <= 8) NB_SS(4, 2);
  else if (n_state <= 16) NB_SS(4, 4);
  else if (n_state <= 32) NB_SS(4, 8);
  else if (n_state <= 64) NB_SS(4, 16);
  else if (n_state <= 128) NB_SS(4, 32);
  else NB_SS(8, 32);
#undef NB_SS
  if (rc) return rc;
  NB_CHECK_LAUNCH("selective_scan");
  return 0;
}
