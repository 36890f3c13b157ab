// A short causal convolution over time on every channel of projected rows, with the last
// taps - 1 inputs of each sequence kept in its fixed-size state row.
//
//   y_t[c] = sum_j w[c][j] * u_(t - taps + 1 + j)[c]  (+ bias[c]),   u = 0 before position 0
//
// The step's rows of a sequence are consecutive rows of the packed batch (cu_rows); inputs from
// before the step come from the state row, which holds u_(pos0 - taps + 1) .. u_(pos0 - 1) as
// [taps - 1][channels] fp32 (zeros when the sequence starts).  Everything here is fp32.
//
// Kernels:
//   nb_conv_rope_append   the attention's use: the channels are [queries | keys | values] of a
//                         fused projection; after the convolution the queries' and keys' heads
//                         are turned by position (number 2i of a head paired with number 2i+1,
//                         angle = pos * freq[i] in fp32); queries go to a buffer of their own,
//                         keys and values into two paged planes (of head sizes d and dv).
//   nb_conv_act           the recurrent branch's use: convolution, bias, activation; the result
//                         as fp32 rows and, rounded, as the next product's operand.
//   nb_conv_state_update  the state rows after the step: the step's last taps - 1 inputs (or,
//                         after fewer tokens than that, the old ones moved up).  Runs after the
//                         kernels above have read the old state; a step of one token per
//                         sequence does it inside them instead (one thread owns a channel).
#include "common.cuh"

namespace {

constexpr int CV_THREADS = 128;
constexpr int CV_MAX_TAPS = 16;
constexpr int CV_TOKENS = 8;       // tokens a CTA walks in a step of more than one token per sequence

// the convolution's result for channel c of the sequence's token t (row = row0 + t)
__device__ __forceinline__ float conv_at(const float* src, int stride, int col0, int row0, int t,
                                         int c, const float* __restrict__ W, int taps,
                                         const float* state_row, int n_channels) {
  if (taps <= 0) return src[(size_t)(row0 + t) * stride + col0 + c];
  float y = 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int tt = t - (taps - 1) + j;
    const float u = tt >= 0 ? src[(size_t)(row0 + tt) * stride + col0 + c]
                            : state_row[(size_t)(taps - 1 + tt) * n_channels + c];
    y = fmaf(W[(size_t)c * taps + j], u, y);
  }
  return y;
}

// the state row of channel c after a step of n_q tokens
__device__ __forceinline__ void state_after(const float* src, int stride, int col0, int row0,
                                            int n_q, int c, int taps, float* state_row,
                                            int n_channels) {
  float keep[CV_MAX_TAPS];
  for (int j = 0; j < taps - 1; ++j) {
    const int tt = n_q - (taps - 1) + j;
    keep[j] = tt >= 0 ? src[(size_t)(row0 + tt) * stride + col0 + c]
                      : state_row[(size_t)(taps - 1 + tt) * n_channels + c];
  }
  for (int j = 0; j < taps - 1; ++j) state_row[(size_t)j * n_channels + c] = keep[j];
}

// One token's convolution for channel c, in a step of one token per sequence: the inputs before
// it are the state row's, which moves up by one as it is read (the thread that reads a channel
// is the only one that ever touches its state numbers, so nothing has to be waited for).
__device__ __forceinline__ float conv_step(float x, int c, const float* __restrict__ W, int taps,
                                           float* state_row, int n_channels) {
  if (taps <= 0) return x;
  float y = 0.0f;
  for (int j = 0; j < taps - 1; ++j) {
    const float u = state_row[(size_t)j * n_channels + c];
    y = fmaf(W[(size_t)c * taps + j], u, y);
    if (j >= 1) state_row[(size_t)(j - 1) * n_channels + c] = u;
  }
  if (taps > 1) state_row[(size_t)(taps - 2) * n_channels + c] = x;
  return fmaf(W[(size_t)c * taps + taps - 1], x, y);
}

// A CTA takes CV_THREADS consecutive channels (blockIdx.z) of CV_TOKENS consecutive tokens
// (blockIdx.x) of a sequence (blockIdx.y); a thread keeps its channel and walks the tokens, so
// that the taps' inputs of the next token are the ones it has just read (they come from L1).
// Of a rotated pair the thread of the even number does both (it needs both convolutions
// anyway) and the other one rests: every channel is then read, and its state row written, by
// one thread only.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(CV_THREADS)
conv_rope_append_kernel(const float* src, int stride, int col0, const float* __restrict__ W,
                        int taps, float* state, int state_stride, const int* cu_rows,
                        const int* seq_slot, const int* seq_pos0, const float* __restrict__ freq,
                        int rot_dims, TQ* q_out, TC* kc, const int* k_table, int k_max_pages,
                        TC* vc, const int* v_table, int v_max_pages, int page, int n_heads,
                        int n_kv_heads, int d, int dv, int tokens_per_cta, int fused_update) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int s = blockIdx.y, t_begin = blockIdx.x * tokens_per_cta;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (t_begin >= n_q) return;
  const int t_end = min(n_q, t_begin + tokens_per_cta);
  const int slot = seq_slot[s];
  const int qw = n_heads * d, kw = n_kv_heads * d, vw = n_kv_heads * dv;
  const int C = qw + kw + vw;
  const int c = blockIdx.z * CV_THREADS + threadIdx.x;
  if (c >= C) return;
  if (slot < 0) {
    if (c < qw)
      for (int t = t_begin; t < t_end; ++t) q_out[(size_t)(row0 + t) * qw + c] = nb_from_f32<TQ>(0.0f);
    return;
  }
  float* st = state + (size_t)slot * state_stride;
  // where the channel goes: a value; or number i of a query or key head
  const bool is_v = c >= qw + kw, is_q = c < qw;
  const int e = is_v ? c - qw - kw : (is_q ? c : c - qw);
  const int hh = e / (is_v ? dv : d), i = e - hh * (is_v ? dv : d);
  const bool turned = !is_v && i < rot_dims;
  if (turned && (i & 1)) return;               // its partner does both
  const float f = turned ? freq[i >> 1] : 0.0f;
  for (int t = t_begin; t < t_end; ++t) {
    const int pos = seq_pos0[s] + t;
    float y, y2 = 0.0f;
    if (fused_update) {
      const float* row = src + (size_t)(row0 + t) * stride + col0;
      y = conv_step(row[c], c, W, taps, st, C);
      if (turned) y2 = conv_step(row[c + 1], c + 1, W, taps, st, C);
    } else {
      y = conv_at(src, stride, col0, row0, t, c, W, taps, st, C);
      if (turned) y2 = conv_at(src, stride, col0, row0, t, c + 1, W, taps, st, C);
    }
    if (is_v) {
      const size_t v_row = (size_t)v_table[(size_t)slot * v_max_pages + pos / page] * n_kv_heads * page + (pos % page);
      vc[(v_row + (size_t)hh * page) * dv + i] = nb_from_f32<TC>(y);
      continue;
    }
    if (turned) {
      float sn, cs;
      sincosf((float)pos * f, &sn, &cs);
      const float a = y * cs - y2 * sn, b = y2 * cs + y * sn;
      y = a;
      y2 = b;
    }
    if (is_q) {
      TQ* qo = q_out + (size_t)(row0 + t) * qw + e;
      qo[0] = nb_from_f32<TQ>(y);
      if (turned) qo[1] = nb_from_f32<TQ>(y2);
    } else {
      const size_t k_row = (size_t)k_table[(size_t)slot * k_max_pages + pos / page] * n_kv_heads * page + (pos % page);
      TC* ko = kc + (k_row + (size_t)hh * page) * d + i;
      ko[0] = nb_from_f32<TC>(y);
      if (turned) ko[1] = nb_from_f32<TC>(y2);
    }
  }
}

template <typename TOut>
__global__ void __launch_bounds__(CV_THREADS)
conv_act_kernel(const float* src, int stride, int col0, const float* __restrict__ W,
                const float* __restrict__ bias, int taps, int act, float* state, int state_stride,
                const int* cu_rows, const int* seq_slot, int C, float* out_f32, TOut* out_act,
                int tokens_per_cta, int fused_update) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int s = blockIdx.y, t_begin = blockIdx.x * tokens_per_cta;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (t_begin >= n_q) return;
  const int t_end = min(n_q, t_begin + tokens_per_cta);
  const int slot = seq_slot[s];
  const int c = blockIdx.z * CV_THREADS + threadIdx.x;
  if (c >= C) return;
  if (slot < 0) {
    for (int t = t_begin; t < t_end; ++t) {
      out_f32[(size_t)(row0 + t) * C + c] = 0.0f;
      if (out_act != nullptr) out_act[(size_t)(row0 + t) * C + c] = nb_from_f32<TOut>(0.0f);
    }
    return;
  }
  float* st = state + (size_t)slot * state_stride;
  const float b = bias != nullptr ? bias[c] : 0.0f;
  for (int t = t_begin; t < t_end; ++t) {
    float y = fused_update ? conv_step(src[(size_t)(row0 + t) * stride + col0 + c], c, W, taps, st, C)
                           : conv_at(src, stride, col0, row0, t, c, W, taps, st, C);
    y = nb_apply_act(y + b, act);
    out_f32[(size_t)(row0 + t) * C + c] = y;
    if (out_act != nullptr) out_act[(size_t)(row0 + t) * C + c] = nb_from_f32<TOut>(y);
  }
}

__global__ void conv_state_update_kernel(const float* src, int stride, int col0, int taps,
                                         float* state, int state_stride, const int* cu_rows,
                                         const int* seq_slot, int C) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int s = blockIdx.y;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (n_q <= 0) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  state_after(src, stride, col0, row0, n_q, c, taps, state + (size_t)slot * state_stride, C);
}

}  // namespace

typedef __nv_bfloat16 bf16;

// src: fp32 [rows][stride] with [queries n_heads*d | keys n_kv_heads*d | values n_kv_heads*dv]
// from column col0; W: fp32 [channels][taps] in that order (null with taps == 0: no
// convolution); state: fp32, a sequence's row at state + slot * state_stride holds
// [taps-1][channels]; freq: fp32 [rot_dims/2]; q_out: [rows][n_heads*d]; kc / vc: planes
// [n_pages][n_kv_heads][page][d or dv] with a block table each.  fused_update: the step has one
// token per sequence and the state is brought up to date here.
NB_EXPORT int nb_conv_rope_append(const float* src, int stride, int col0, const float* W, int taps,
                                  float* state, int state_stride, const int* cu_rows,
                                  const int* seq_slot, const int* seq_pos0, const float* freq,
                                  int rot_dims, void* q_out, int q_dtype, void* kc,
                                  const int* k_table, int k_max_pages, void* vc, const int* v_table,
                                  int v_max_pages, int cache_dtype, int page, int n_heads,
                                  int n_kv_heads, int d, int dv, int n_seqs, int max_q_len,
                                  int fused_update, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && d > 0 && dv > 0 && page > 0 && taps >= 0 &&
                 taps <= CV_MAX_TAPS && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d &&
                 (rot_dims == 0 || freq != nullptr) && (taps == 0 || W != nullptr) &&
                 (taps <= 1 || state != nullptr) && n_seqs <= 65535,
             NB_ERR_BAD_ARG, "conv_rope_append: bad sizes heads=%d/%d d=%d dv=%d taps=%d rot=%d",
             n_heads, n_kv_heads, d, dv, taps, rot_dims);
  NB_REQUIRE(!fused_update || max_q_len == 1, NB_ERR_BAD_ARG,
             "conv_rope_append: the state is updated in place only in steps of one token");
  const int channels = n_heads * d + n_kv_heads * (d + dv);
  const int per_cta = max_q_len == 1 ? 1 : CV_TOKENS;
  const dim3 grid((max_q_len + per_cta - 1) / per_cta, n_seqs, (channels + CV_THREADS - 1) / CV_THREADS);
  NB_REQUIRE(grid.z <= 65535, NB_ERR_UNSUPPORTED, "conv_rope_append: %d channels", channels);
#define NB_CRA(TQ, TC)                                                                            \
  NB_CUDA(nb_launch(conv_rope_append_kernel<TQ, TC>, grid, dim3(CV_THREADS), 0, stream, src,      \
                    stride, col0, W, taps, state, state_stride, cu_rows, seq_slot, seq_pos0, freq, \
                    rot_dims, (TQ*)q_out, (TC*)kc, k_table, k_max_pages, (TC*)vc, v_table,        \
                    v_max_pages, page, n_heads, n_kv_heads, d, dv, per_cta, fused_update))
  switch (q_dtype * 2 + cache_dtype) {
    case 0: NB_CRA(float, float); break;
    case 1: NB_CRA(float, bf16); break;
    case 2: NB_CRA(bf16, float); break;
    case 3: NB_CRA(bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "conv_rope_append: unknown dtypes %d/%d", q_dtype, cache_dtype);
  }
#undef NB_CRA
  NB_CHECK_LAUNCH("conv_rope_append");
  return 0;
}

// out_f32 [rows][C] = act(conv(src[:, col0 .. col0 + C]) + bias); out_act (optional): the same
// rounded to act_dtype.
NB_EXPORT int nb_conv_act(const float* src, int stride, int col0, const float* W, const float* bias,
                          int taps, int act, float* state, int state_stride, const int* cu_rows,
                          const int* seq_slot, int n_channels, float* out_f32, void* out_act,
                          int act_dtype, int n_seqs, int max_q_len, int fused_update,
                          cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(n_channels > 0 && taps >= 0 && taps <= CV_MAX_TAPS && (taps == 0 || W != nullptr) &&
                 (taps <= 1 || state != nullptr) && n_seqs <= 65535 && out_f32 != nullptr,
             NB_ERR_BAD_ARG, "conv_act: bad sizes channels=%d taps=%d", n_channels, taps);
  NB_REQUIRE(!fused_update || max_q_len == 1, NB_ERR_BAD_ARG,
             "conv_act: the state is updated in place only in steps of one token");
  const int per_cta = max_q_len == 1 ? 1 : CV_TOKENS;
  const dim3 grid((max_q_len + per_cta - 1) / per_cta, n_seqs, (n_channels + CV_THREADS - 1) / CV_THREADS);
  NB_REQUIRE(grid.z <= 65535, NB_ERR_UNSUPPORTED, "conv_act: %d channels", n_channels);
  if (out_act == nullptr || act_dtype == NB_F32)
    NB_CUDA(nb_launch(conv_act_kernel<float>, grid, dim3(CV_THREADS), 0, stream, src, stride, col0,
                      W, bias, taps, act, state, state_stride, cu_rows, seq_slot, n_channels,
                      out_f32, (float*)out_act, per_cta, fused_update));
  else if (act_dtype == NB_BF16)
    NB_CUDA(nb_launch(conv_act_kernel<bf16>, grid, dim3(CV_THREADS), 0, stream, src, stride, col0,
                      W, bias, taps, act, state, state_stride, cu_rows, seq_slot, n_channels,
                      out_f32, (bf16*)out_act, per_cta, fused_update));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "conv_act: unknown dtype %d", act_dtype);
  NB_CHECK_LAUNCH("conv_act");
  return 0;
}

NB_EXPORT int nb_conv_state_update(const float* src, int stride, int col0, int taps, float* state,
                                   int state_stride, const int* cu_rows, const int* seq_slot,
                                   int n_channels, int n_seqs, cudaStream_t stream) {
  if (n_seqs == 0 || taps <= 1) return 0;
  NB_REQUIRE(n_channels > 0 && taps <= CV_MAX_TAPS && state != nullptr && n_seqs <= 65535,
             NB_ERR_BAD_ARG, "conv_state_update: bad sizes channels=%d taps=%d", n_channels, taps);
  const dim3 grid((n_channels + 127) / 128, n_seqs);
  NB_CUDA(nb_launch(conv_state_update_kernel, grid, dim3(128), 0, stream, src, stride, col0, taps,
                    state, state_stride, cu_rows, seq_slot, n_channels));
  NB_CHECK_LAUNCH("conv_state_update");
  return 0;
}
