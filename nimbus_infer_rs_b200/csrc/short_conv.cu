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
constexpr int CV_TILE_W = CV_THREADS + 1;   // a staged row: the CTA's channels and the one after
constexpr int CV_TOKENS = 16;      // tokens a CTA walks in a step of more than one token per sequence

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

// A CTA first stages the inputs of its channels for its run of tokens, and the taps - 1 inputs
// before the run (from earlier rows of the step or from the state row), in shared memory: every
// thread fetches its own channel's column, all fetches in flight together (a thread that walked
// the tokens with one fetch at a time kept too few bytes in flight to use the memory's
// bandwidth).  Row r of the tile is token t_begin - (taps - 1) + r.
template <int MT>
__device__ __forceinline__ void conv_stage(float* tile, const float* src, int stride, int col0,
                                           int row0, int t_begin, int t_end, int c, int taps,
                                           const float* state_row, int n_channels,
                                           bool one_more) {
  const int before = taps > 1 ? taps - 1 : 0;
  const int rows = before + t_end - t_begin;
  if (c < n_channels) {
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
      const int tt = t_begin - before + r;
      tile[r * CV_TILE_W + threadIdx.x] =
          tt >= 0 ? src[(size_t)(row0 + tt) * stride + col0 + c]
                  : state_row[(size_t)(before + tt) * n_channels + c];
    }
  }
  // the channel after the CTA's last one: the partner of a rotated pair that starts there
  if (one_more && threadIdx.x == CV_THREADS - 1 && c + 1 < n_channels)
    for (int r = 0; r < rows; ++r) {
      const int tt = t_begin - before + r;
      tile[r * CV_TILE_W + CV_THREADS] =
          tt >= 0 ? src[(size_t)(row0 + tt) * stride + col0 + c + 1]
                  : state_row[(size_t)(before + tt) * n_channels + c + 1];
    }
}

// A channel's walk over the staged run: its weights and the taps' inputs before the next token
// stay in registers (MT slots, the newest tap in the last one, so that every index is known to
// the compiler; taps <= MT).  The products are added oldest tap first, as conv_at and conv_step
// add them: a token's number does not depend on which of the three computed it.
template <int MT>
struct ConvWalk {
  float w[MT], h[MT - 1];
  const float* col;     // the channel's column of the tile, at the run's first token
  int taps;
  __device__ __forceinline__ void start(const float* tile_col, int c, const float* __restrict__ W,
                                        int taps_) {
    taps = taps_;
    const int before = taps > 1 ? taps - 1 : 0;
    col = tile_col + before * CV_TILE_W;
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      const int j = k - (MT - taps);                       // tap j sits in slot k
      w[k] = j >= 0 ? W[(size_t)c * taps + j] : 0.0f;
      if (k < MT - 1) h[k] = j >= 0 ? tile_col[j * CV_TILE_W] : 0.0f;
    }
  }
  // the convolution at token number u of the run
  __device__ __forceinline__ float next(int u) {
    const float x = col[u * CV_TILE_W];
    if (taps <= 0) return x;
    float y = 0.0f;
#pragma unroll
    for (int k = 0; k < MT - 1; ++k) {
      if (k >= MT - taps) y = fmaf(w[k], h[k], y);
      if (k < MT - 2) h[k] = h[k + 1];
    }
    if (MT > 1) h[MT - 2] = x;
    return fmaf(w[MT - 1], x, y);
  }
};

// A CTA takes CV_THREADS consecutive channels (blockIdx.x) of CV_TOKENS consecutive tokens
// (blockIdx.z) of a sequence (blockIdx.y): the CTAs that run side by side read neighbouring
// pieces of the same rows.  A thread keeps its channel and walks the tokens with a ConvWalk (a
// step of one token per sequence reads and moves the state row instead).
template <typename TQ, typename TC, int MT>
__global__ void __launch_bounds__(CV_THREADS)
conv_rope_append_kernel(const float* src, int stride, int col0, const float* __restrict__ W,
                        int taps, float* state, int state_stride, const int* cu_rows,
                        const int* seq_slot, const int* seq_pos0, const float* __restrict__ freq,
                        int rot_dims, TQ* q_out, TC* kc, const int* k_table, int k_max_pages,
                        TC* vc, const int* v_table, int v_max_pages, int page, int n_heads,
                        int n_kv_heads, int d, int dv, int tokens_per_cta, int fused_update) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int s = blockIdx.y, t_begin = blockIdx.z * tokens_per_cta;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (t_begin >= n_q) return;
  const int t_end = min(n_q, t_begin + tokens_per_cta);
  const int slot = seq_slot[s];
  const int qw = n_heads * d, kw = n_kv_heads * d, vw = n_kv_heads * dv;
  const int C = qw + kw + vw;
  const int c = blockIdx.x * CV_THREADS + threadIdx.x;
  if (slot < 0) {
    if (c < qw)
      for (int t = t_begin; t < t_end; ++t) q_out[(size_t)(row0 + t) * qw + c] = nb_from_f32<TQ>(0.0f);
    return;
  }
  float* st = state + (size_t)slot * state_stride;
  __shared__ float tile[(CV_TOKENS + MT - 1) * CV_TILE_W];
  if (!fused_update) {
    conv_stage<MT>(tile, src, stride, col0, row0, t_begin, t_end, c, taps, st, C, rot_dims > 0);
    __syncthreads();
  }
  if (c >= C) return;
  // where the channel goes: a value; or number i of a query or key head
  const bool is_v = c >= qw + kw, is_q = c < qw;
  const int e0 = is_v ? c - qw - kw : (is_q ? c : c - qw);
  const int hh = e0 / (is_v ? dv : d), i0 = e0 - hh * (is_v ? dv : d);
  const bool turned = !is_v && i0 < rot_dims;
  // A rotated pair needs both convolutions for either number, so one thread does both numbers
  // of a token; the pair's two threads share the run's tokens, the first half to the even one
  // (all of them where the partner sits in another CTA, and in a step of one token, where a
  // channel's state row has one owner).
  const bool odd = turned && (i0 & 1);
  int u_lo = 0, u_hi = t_end - t_begin;
  if (turned) {
    const bool partner_here = odd ? threadIdx.x > 0 : threadIdx.x < CV_THREADS - 1;
    if (!partner_here || fused_update) {
      if (odd) return;
    } else {
      const int half = (u_hi + 1) / 2;
      if (odd) u_lo = half;
      else u_hi = half;
    }
  }
  if (u_lo >= u_hi) return;
  const int pc = c - (odd ? 1 : 0), ptid = (int)threadIdx.x - (odd ? 1 : 0);   // the pair's even channel
  const int e = e0 - (odd ? 1 : 0), i = i0 - (odd ? 1 : 0);
  const float f = turned ? freq[i >> 1] : 0.0f;
  ConvWalk<MT> walk, walk2;
  if (!fused_update) {
    walk.start(tile + u_lo * CV_TILE_W + ptid, pc, W, taps);
    if (turned) walk2.start(tile + u_lo * CV_TILE_W + ptid + 1, pc + 1, W, taps);
  }
  // the cache row of the token: its page from the table when the walk enters one
  const int pos_begin = seq_pos0[s] + t_begin + u_lo;
  int pg = pos_begin / page, off = pos_begin - pg * page;
  const int* table = is_v ? v_table + (size_t)slot * v_max_pages : k_table + (size_t)slot * k_max_pages;
  size_t page_row = is_q ? 0 : (size_t)table[pg] * n_kv_heads * page;
  for (int t = t_begin + u_lo; t < t_begin + u_hi; ++t, ++off) {
    const int pos = seq_pos0[s] + t;
    if (off == page) {
      off = 0;
      ++pg;
      if (!is_q) page_row = (size_t)table[pg] * n_kv_heads * page;
    }
    float y, y2 = 0.0f;
    if (fused_update) {
      const float* row = src + (size_t)(row0 + t) * stride + col0;
      y = conv_step(row[pc], pc, W, taps, st, C);
      if (turned) y2 = conv_step(row[pc + 1], pc + 1, W, taps, st, C);
    } else {
      y = walk.next(t - t_begin - u_lo);
      if (turned) y2 = walk2.next(t - t_begin - u_lo);
    }
    if (is_v) {
      vc[(page_row + off + (size_t)hh * page) * dv + i] = nb_from_f32<TC>(y);
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
      TC* ko = kc + (page_row + off + (size_t)hh * page) * d + i;
      ko[0] = nb_from_f32<TC>(y);
      if (turned) ko[1] = nb_from_f32<TC>(y2);
    }
  }
}

template <typename TOut, int MT>
__global__ void __launch_bounds__(CV_THREADS)
conv_act_kernel(const float* src, int stride, int col0, const float* __restrict__ W,
                const float* __restrict__ bias, int taps, int act, float* state, int state_stride,
                const int* cu_rows, const int* seq_slot, int C, float* out_f32, TOut* out_act,
                int tokens_per_cta, int fused_update) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int s = blockIdx.y, t_begin = blockIdx.z * tokens_per_cta;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  if (t_begin >= n_q) return;
  const int t_end = min(n_q, t_begin + tokens_per_cta);
  const int slot = seq_slot[s];
  const int c = blockIdx.x * CV_THREADS + threadIdx.x;
  if (slot < 0) {
    if (c < C)
      for (int t = t_begin; t < t_end; ++t) {
        out_f32[(size_t)(row0 + t) * C + c] = 0.0f;
        if (out_act != nullptr) out_act[(size_t)(row0 + t) * C + c] = nb_from_f32<TOut>(0.0f);
      }
    return;
  }
  float* st = state + (size_t)slot * state_stride;
  __shared__ float tile[(CV_TOKENS + MT - 1) * CV_TILE_W];
  if (!fused_update) {
    conv_stage<MT>(tile, src, stride, col0, row0, t_begin, t_end, c, taps, st, C, false);
    __syncthreads();
  }
  if (c >= C) return;
  const float b = bias != nullptr ? bias[c] : 0.0f;
  ConvWalk<MT> walk;
  if (!fused_update) walk.start(tile + threadIdx.x, c, W, taps);
  for (int t = t_begin; t < t_end; ++t) {
    float y = fused_update ? conv_step(src[(size_t)(row0 + t) * stride + col0 + c], c, W, taps, st, C)
                           : walk.next(t - t_begin);
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
  const dim3 grid((channels + CV_THREADS - 1) / CV_THREADS, n_seqs, (max_q_len + per_cta - 1) / per_cta);
  NB_REQUIRE(grid.z <= 65535, NB_ERR_UNSUPPORTED, "conv_rope_append: a step of %d tokens", max_q_len);
#define NB_CRA_MT(TQ, TC, MT)                                                                     \
  NB_CUDA(nb_launch(conv_rope_append_kernel<TQ, TC, MT>, grid, dim3(CV_THREADS), 0, stream, src,  \
                    stride, col0, W, taps, state, state_stride, cu_rows, seq_slot, seq_pos0, freq, \
                    rot_dims, (TQ*)q_out, (TC*)kc, k_table, k_max_pages, (TC*)vc, v_table,        \
                    v_max_pages, page, n_heads, n_kv_heads, d, dv, per_cta, fused_update))
#define NB_CRA(TQ, TC)                                                                            \
  do {                                                                                            \
    if (taps <= 4) NB_CRA_MT(TQ, TC, 4);                                                          \
    else NB_CRA_MT(TQ, TC, CV_MAX_TAPS);                                                          \
  } while (0)
  switch (q_dtype * 2 + cache_dtype) {
    case 0: NB_CRA(float, float); break;
    case 1: NB_CRA(float, bf16); break;
    case 2: NB_CRA(bf16, float); break;
    case 3: NB_CRA(bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "conv_rope_append: unknown dtypes %d/%d", q_dtype, cache_dtype);
  }
#undef NB_CRA
#undef NB_CRA_MT
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
  const dim3 grid((n_channels + CV_THREADS - 1) / CV_THREADS, n_seqs, (max_q_len + per_cta - 1) / per_cta);
  NB_REQUIRE(grid.z <= 65535, NB_ERR_UNSUPPORTED, "conv_act: a step of %d tokens", max_q_len);
#define NB_CA(T, MT)                                                                              \
  NB_CUDA(nb_launch(conv_act_kernel<T, MT>, grid, dim3(CV_THREADS), 0, stream, src, stride, col0, \
                    W, bias, taps, act, state, state_stride, cu_rows, seq_slot, n_channels,       \
                    out_f32, (T*)out_act, per_cta, fused_update))
  if (out_act == nullptr || act_dtype == NB_F32) {
    if (taps <= 4) NB_CA(float, 4);
    else NB_CA(float, CV_MAX_TAPS);
  } else if (act_dtype == NB_BF16) {
    if (taps <= 4) NB_CA(bf16, 4);
    else NB_CA(bf16, CV_MAX_TAPS);
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "conv_act: unknown dtype %d", act_dtype);
  }
#undef NB_CA
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
