// Row-wise kernels: token+position embedding, LayerNorm, key/value append into the paged
// cache.  One thread block per row; any width.
#include <stdarg.h>

#include "common.cuh"

// ---------------------------------------------------------------------------------
// error text of the calling thread
// ---------------------------------------------------------------------------------
static thread_local char g_error[512] = "";

void nb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

NB_EXPORT const char* nb_last_error() { return g_error; }

NB_EXPORT int nb_abi_version() { return 3; }

// ---------------------------------------------------------------------------------
// error words (see common.cuh)
// ---------------------------------------------------------------------------------
#include <mutex>
static int* g_error_words = nullptr;
int* nb_error_words() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, NB_ERRW_COUNT * sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) ==
        cudaSuccess) {
      for (int i = 0; i < NB_ERRW_COUNT; ++i) static_cast<volatile int*>(p)[i] = 0;
      g_error_words = static_cast<int*>(p);
    } else {
      (void)cudaGetLastError();
    }
  });
  return g_error_words;
}
// Bit i is set if error word i is raised.  No synchronisation: the caller has waited for the
// work it asks about.  `clear` != 0 lowers the words that were read as raised.
NB_EXPORT int nb_device_errors(int clear) {
  volatile int* w = nb_error_words();
  if (w == nullptr) return 0;
  int mask = 0;
  for (int i = 0; i < NB_ERRW_COUNT; ++i) {
    if (w[i] != 0) {
      mask |= 1 << i;
      if (clear) w[i] = 0;
    }
  }
  return mask;
}

// Whether kernels are launched so that they may overlap the tail of their predecessor.
static int g_overlap = 0;
bool nb_overlap_enabled() { return g_overlap != 0; }
NB_EXPORT void nb_set_overlap(int on) { g_overlap = on; }
NB_EXPORT int nb_get_overlap() { return g_overlap; }

// ---------------------------------------------------------------------------------
// x[r] = scale * wte[token[r]] + wpe[pos[r]]   (src/model.rs:285-295, scale 1), fp32 result.
// A negative token marks a padding row: it is written as zeros.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void embed_pos_kernel(const int* tokens, const int* pos,
                                 const T* __restrict__ wte, const T* __restrict__ wpe,
                                 float* out, int d, float scale) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  const int tok = tokens[r];
  float* o = out + (size_t)r * d;
  if (tok < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const T* e = wte + (size_t)tok * d;
  if (wpe != nullptr) {
    const T* p = wpe + (size_t)pos[r] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_to_f32(e[i]) * scale + nb_to_f32(p[i]);
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_to_f32(e[i]) * scale;
  }
}

NB_EXPORT int nb_embed_pos(const int* tokens, const int* pos, const void* wte, const void* wpe,
                           int table_dtype, float* out, int n_rows, int d, float scale,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0, NB_ERR_BAD_ARG, "embed_pos: bad sizes rows=%d d=%d", n_rows, d);
  const int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  if (table_dtype == NB_F32)
    NB_CUDA(nb_launch(embed_pos_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, tokens, pos,
                      (const float*)wte, (const float*)wpe, out, d, scale));
  else if (table_dtype == NB_BF16)
    NB_CUDA(nb_launch(embed_pos_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream,
                      tokens, pos, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, d,
                      scale));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "embed_pos: unknown table dtype %d", table_dtype);
  NB_CHECK_LAUNCH("embed_pos");
  return 0;
}

// ---------------------------------------------------------------------------------
// x[r] = scale * wte[token[r]] + pair[bucket(r)], fp32 result: a second table indexed by a hash
// of (previous token, token):  bucket = (prev * mul_prev + token * mul_cur) mod n_buckets, and
// row n_buckets (the table's last) for a sequence's first token.  The previous token of a row is
// the row before it in the step or, for the first row of a continued sequence, what the
// sequence's state row holds (`last`, one float per slot: token ids are exact there); the state
// row then takes the token of the sequence's last row in this step.
//
// The grid is one CTA per row and one more per sequence.  A sequence's first row in the step is
// left to the sequence's CTA, which reads the state row, embeds that row, and only then (behind
// a barrier of the CTA) writes the state row: no other CTA reads it.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void embed_hashed_kernel(const int* tokens, const int* pos, const int* row_slot,
                                    const int* cu_rows, int n_rows, const T* __restrict__ wte,
                                    const T* __restrict__ pair, float* last, int last_stride,
                                    float* out, int d, float scale, int mul_prev, int mul_cur,
                                    int n_buckets) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const bool of_sequence = (int)blockIdx.x >= n_rows;
  int r = blockIdx.x, last_row = -1;
  if (of_sequence) {
    const int s = blockIdx.x - n_rows;
    r = cu_rows[s];
    last_row = cu_rows[s + 1] - 1;
    if (last_row < r) return;                 // a sequence without rows
  }
  const int tok = tokens[r];
  float* o = out + (size_t)r * d;
  const int slot = row_slot[r];
  if (tok < 0 || slot < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const int p = pos[r];
  const bool first_in_step = !(r > 0 && row_slot[r - 1] == slot && pos[r - 1] == p - 1);
  if (first_in_step != of_sequence) return;   // the other kind of CTA has this row
  long long bucket = n_buckets;
  if (p > 0) {
    const int prev = of_sequence ? (int)last[(size_t)slot * last_stride] : tokens[r - 1];
    bucket = ((long long)prev * mul_prev + (long long)tok * mul_cur) % n_buckets;
    if (bucket < 0) bucket += n_buckets;
  }
  const T* e = wte + (size_t)tok * d;
  const T* b = pair + (size_t)bucket * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    o[i] = nb_to_f32(e[i]) * scale + nb_to_f32(b[i]);
  if (of_sequence) {
    __syncthreads();                          // every thread has read the state row
    if (threadIdx.x == 0 && tokens[last_row] >= 0)
      last[(size_t)slot * last_stride] = (float)tokens[last_row];
  }
}

NB_EXPORT int nb_embed_hashed(const int* tokens, const int* pos, const int* row_slot,
                              const int* cu_rows, int n_seqs, const void* wte, const void* pair,
                              int table_dtype, float* last, int last_stride, float* out, int n_rows,
                              int d, float scale, int mul_prev, int mul_cur, int n_buckets,
                              cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && n_seqs >= 0 && d > 0 && n_buckets > 0 && last != nullptr && cu_rows != nullptr,
             NB_ERR_BAD_ARG, "embed_hashed: bad sizes rows=%d d=%d buckets=%d", n_rows, d, n_buckets);
  const int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  const dim3 grid(n_rows + n_seqs);
  if (table_dtype == NB_F32)
    NB_CUDA(nb_launch(embed_hashed_kernel<float>, grid, dim3(threads), 0, stream, tokens, pos,
                      row_slot, cu_rows, n_rows, (const float*)wte, (const float*)pair, last,
                      last_stride, out, d, scale, mul_prev, mul_cur, n_buckets));
  else if (table_dtype == NB_BF16)
    NB_CUDA(nb_launch(embed_hashed_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, tokens, pos,
                      row_slot, cu_rows, n_rows, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)pair,
                      last, last_stride, out, d, scale, mul_prev, mul_cur, n_buckets));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "embed_hashed: unknown table dtype %d", table_dtype);
  NB_CHECK_LAUNCH("embed_hashed");
  return 0;
}

// ---------------------------------------------------------------------------------
// LayerNorm of fp32 rows (src/ops.rs:32-40): mean, biased variance of (x - mean), both in
// fp32 and in two passes; y = (x - mean) / sqrt(var + eps) * gamma + beta.
// `rows` (optional) selects the source row of each output row; a negative entry gives zeros.
// The row is kept in shared memory between the passes.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void layernorm_kernel(const float* x, const int* rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 TOut* out, int d, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  TOut* o = out + (size_t)r * d;
  if (src < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const float* xr = x + (size_t)src * d;
  float s = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    row[i] = v;
    s += v;
  }
  const float mean = nb_block_sum(s, red) / (float)d;
  float q = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = row[i] - mean;
    q += c * c;
  }
  const float var = nb_block_sum(q, red) / (float)d;
  const float inv = 1.0f / sqrtf(var + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float y = (row[i] - mean) * inv * gamma[i];
    if (beta) y += beta[i];
    o[i] = nb_from_f32<TOut>(y);
  }
}

// The same, one warp per row with the row held in registers (one trip to memory): widths that
// are a multiple of 4 up to 128 * VN.  EARLY: scale and shift are fetched into registers
// before the wait on the kernel in front (they are constants), which takes their trip to
// memory out of a decode step's chain (batch 64: 0.98 -> 0.93 ms a step on GPT-2 124M, 4.26
// -> 3.72 ms on XL); with thousands of rows the registers cost more CTAs per SM than the trip
// is worth (a 2,048-token prefill: 1.15 -> 1.25 ms), so those fetch them where they are used.
template <typename TOut, int VN, bool EARLY>
__global__ void __launch_bounds__(128)
layernorm_warp_kernel(const float* x, const int* rows,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      TOut* out, int n_rows, int d, float eps) {
  const int lane = threadIdx.x & 31;
  float4 gm[EARLY ? VN : 1], bt[EARLY ? VN : 1];
  if constexpr (EARLY) {
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const int k = lane * 4 + i * 128;
      gm[i] = k < d ? *reinterpret_cast<const float4*>(gamma + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      bt[i] = (beta && k < d) ? *reinterpret_cast<const float4*>(beta + k)
                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  TOut* o = out + (size_t)r * d;
  float4 v[VN];
  const float* xr = x + (size_t)(src < 0 ? 0 : src) * d;
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    const int k = lane * 4 + i * 128;
    v[i] = (src >= 0 && k < d) ? *reinterpret_cast<const float4*>(xr + k)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VN; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mean = nb_warp_sum(s) / (float)d;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    if (lane * 4 + i * 128 < d) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      q += (a * a + b * b) + (c * c + e * e);
    }
  }
  const float inv = 1.0f / sqrtf(nb_warp_sum(q) / (float)d + eps);
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    const int k = lane * 4 + i * 128;
    if (k >= d) continue;
    float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (src >= 0) {
      float4 g4, b4;
      if constexpr (EARLY) {
        g4 = gm[i];
        b4 = bt[i];
      } else {
        g4 = *reinterpret_cast<const float4*>(gamma + k);
        b4 = beta ? *reinterpret_cast<const float4*>(beta + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
      y.x = (v[i].x - mean) * inv * g4.x + b4.x;
      y.y = (v[i].y - mean) * inv * g4.y + b4.y;
      y.z = (v[i].z - mean) * inv * g4.z + b4.z;
      y.w = (v[i].w - mean) * inv * g4.w + b4.w;
    }
    if constexpr (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(o + k) = y;
    } else {
      uint2 pk;
      *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(y.x, y.y);
      *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(y.z, y.w);
      *reinterpret_cast<uint2*>(o + k) = pk;
    }
  }
}

template <typename TOut>
int launch_layernorm_warp(const float* x, const int* rows, const float* gamma, const float* beta,
                          void* out, int n_rows, int d, float eps, cudaStream_t stream) {
  const dim3 grid((n_rows + 3) / 4), block(128);
  const bool early = n_rows <= 512;   // one CTA per SM or so: registers are free
#define NB_LN(VN_)                                                                              \
  do {                                                                                          \
    if (early)                                                                                  \
      NB_CUDA(nb_launch(layernorm_warp_kernel<TOut, VN_, true>, grid, block, 0, stream, x, rows, \
                        gamma, beta, (TOut*)out, n_rows, d, eps));                              \
    else                                                                                        \
      NB_CUDA(nb_launch(layernorm_warp_kernel<TOut, VN_, false>, grid, block, 0, stream, x, rows, \
                        gamma, beta, (TOut*)out, n_rows, d, eps));                              \
  } while (0)
  if (d <= 128 * 2) NB_LN(2);
  else if (d <= 128 * 8) NB_LN(8);
  else NB_LN(16);
#undef NB_LN
  return 0;
}

NB_EXPORT int nb_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                           void* out, int out_dtype, int n_rows, int d, float eps,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0, NB_ERR_BAD_ARG, "layernorm: bad sizes rows=%d d=%d", n_rows, d);
  if (d % 4 == 0 && d <= 128 * 16 && (uintptr_t)x % 16 == 0 && (uintptr_t)gamma % 16 == 0 &&
      (uintptr_t)beta % 16 == 0 && (uintptr_t)out % 16 == 0 &&
      (out_dtype == NB_F32 || out_dtype == NB_BF16)) {
    const int rc = out_dtype == NB_F32
                       ? launch_layernorm_warp<float>(x, rows, gamma, beta, out, n_rows, d, eps, stream)
                       : launch_layernorm_warp<__nv_bfloat16>(x, rows, gamma, beta, out, n_rows, d,
                                                              eps, stream);
    if (rc) return rc;
    NB_CHECK_LAUNCH("layernorm");
    return 0;
  }
  const size_t smem = (size_t)d * sizeof(float);
  NB_REQUIRE(smem <= 200 * 1024, NB_ERR_UNSUPPORTED,
             "layernorm: width %d needs %zu bytes of shared memory (limit 204800)", d, smem);
  const int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
  if (out_dtype == NB_F32) {
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(layernorm_kernel<float>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows,
                      gamma, beta, (float*)out, d, eps));
  } else if (out_dtype == NB_BF16) {
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x,
                      rows, gamma, beta, (__nv_bfloat16*)out, d, eps));
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "layernorm: unknown output dtype %d", out_dtype);
  }
  NB_CHECK_LAUNCH("layernorm");
  return 0;
}

// ---------------------------------------------------------------------------------
// Root-mean-square norm: out[r] = x[src] / sqrt(mean(x[src]^2) + eps) * gamma, statistics and
// scaling in fp32.  The source rows are columns x_col .. x_col + d of a wider fp32 matrix of
// row stride x_stride (so that a slice of a fused projection's result can be normed in
// place of a copy); `rows` (optional) names the source row of every output row, a negative
// entry gives zeros.  `gamma` may be null (no learned scale).
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void rmsnorm_kernel(const float* x, int x_stride, int x_col, const int* rows,
                               const float* __restrict__ gamma, TOut* out, int d, float eps) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  TOut* o = out + (size_t)r * d;
  if (src < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const float* xr = x + (size_t)src * x_stride + x_col;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = nb_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    o[i] = nb_from_f32<TOut>(xr[i] * inv * (gamma ? gamma[i] : 1.0f));
}

NB_EXPORT int nb_rmsnorm(const float* x, int x_stride, int x_col, const int* rows,
                         const float* gamma, void* out, int out_dtype, int n_rows, int d, float eps,
                         cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && x_col >= 0 && x_stride >= x_col + d, NB_ERR_BAD_ARG,
             "rmsnorm: bad sizes rows=%d d=%d col=%d stride=%d", n_rows, d, x_col, x_stride);
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : (d >= 128 ? 128 : 64));
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride,
                      x_col, rows, gamma, (float*)out, d, eps));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x,
                      x_stride, x_col, rows, gamma, (__nv_bfloat16*)out, d, eps));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "rmsnorm: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------
// A sublayer's normed result added to the stream, and what the stream's next reader wants, in
// one pass over a row:  x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * gamma            (fp32)
//   out_next[r] = x[r] / sqrt(mean(x[r]^2) + next_eps) * next_gamma   if out_next  (TOut)
//   out_cast[r] = x[r]                                                if out_cast  (TOut)
// The row stays in registers between the two norms (width <= RA_MAX * threads).
// ---------------------------------------------------------------------------------
constexpr int RA_MAX = 8;

template <typename TOut, bool CENTER>
__global__ void rms_add_kernel(const float* y, const float* __restrict__ gamma, float eps, float* x,
                               const float* __restrict__ next_gamma, float next_eps,
                               TOut* out_next, TOut* out_cast, int d) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * d;
  float* xr = x + (size_t)r * d;
  float v[RA_MAX];
  float ss = 0.0f;
#pragma unroll
  for (int a = 0; a < RA_MAX; ++a) {
    const int i = threadIdx.x + a * blockDim.x;
    v[a] = i < d ? yr[i] : 0.0f;
    if (!CENTER) ss = fmaf(v[a], v[a], ss);
  }
  if (CENTER) {
    float s1 = 0.0f;
#pragma unroll
    for (int a = 0; a < RA_MAX; ++a) s1 += v[a];
    const float mean = nb_block_sum(s1, red) / (float)d;
#pragma unroll
    for (int a = 0; a < RA_MAX; ++a) {
      v[a] = threadIdx.x + a * blockDim.x < d ? v[a] - mean : 0.0f;
      ss = fmaf(v[a], v[a], ss);
    }
  }
  ss = nb_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  float s2 = 0.0f;
#pragma unroll
  for (int a = 0; a < RA_MAX; ++a) {
    const int i = threadIdx.x + a * blockDim.x;
    if (i < d) {
      v[a] = xr[i] + v[a] * inv * gamma[i];
      xr[i] = v[a];
      if (out_cast != nullptr) out_cast[(size_t)r * d + i] = nb_from_f32<TOut>(v[a]);
    } else {
      v[a] = 0.0f;
    }
    if (!CENTER) s2 = fmaf(v[a], v[a], s2);
  }
  if (out_next == nullptr) return;
  if (CENTER) {
    float s1 = 0.0f;
#pragma unroll
    for (int a = 0; a < RA_MAX; ++a) s1 += v[a];
    const float mean = nb_block_sum(s1, red) / (float)d;
#pragma unroll
    for (int a = 0; a < RA_MAX; ++a) {
      v[a] = threadIdx.x + a * blockDim.x < d ? v[a] - mean : 0.0f;
      s2 = fmaf(v[a], v[a], s2);
    }
  }
  s2 = nb_block_sum(s2, red);
  const float inv2 = 1.0f / sqrtf(s2 / (float)d + next_eps);
#pragma unroll
  for (int a = 0; a < RA_MAX; ++a) {
    const int i = threadIdx.x + a * blockDim.x;
    if (i < d) out_next[(size_t)r * d + i] = nb_from_f32<TOut>(v[a] * inv2 * next_gamma[i]);
  }
}

// The same with a warp per row and the row in registers, 16 bytes a load (width a multiple of
// 128, at most RW_MAX * 128): no barrier, the two sums by shuffles.
constexpr int RW_MAX = 16;

template <typename TOut>
__device__ __forceinline__ void nb_store4(TOut* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void nb_store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void nb_store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c,
                                                        float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TOut, int NV, bool CENTER>
__global__ void __launch_bounds__(128)
rms_add_warp_kernel(const float* y, const float* __restrict__ gamma, float eps, float* x,
                    const float* __restrict__ next_gamma, float next_eps, TOut* out_next,
                    TOut* out_cast, int d, int n_rows) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * d);
  float4* xr = reinterpret_cast<float4*>(x + (size_t)r * d);
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  float4 v[NV], xv[NV];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    v[j] = yr[j * 32 + lane];
    xv[j] = xr[j * 32 + lane];
  }
  if (CENTER) {
    float s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) s1 += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    const float mean = nb_warp_sum(s1) / (float)d;
#pragma unroll
    for (int j = 0; j < NV; ++j) { v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean; }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j)
    ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
  ss = nb_warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  float s2 = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const float4 g = g4[j * 32 + lane];
    v[j].x = xv[j].x + v[j].x * inv * g.x;
    v[j].y = xv[j].y + v[j].y * inv * g.y;
    v[j].z = xv[j].z + v[j].z * inv * g.z;
    v[j].w = xv[j].w + v[j].w * inv * g.w;
    xr[j * 32 + lane] = v[j];
    if (out_cast != nullptr)
      nb_store4<TOut>(out_cast + (size_t)r * d + (j * 32 + lane) * 4, v[j].x, v[j].y, v[j].z, v[j].w);
    if (!CENTER)
      s2 = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, s2))));
  }
  if (out_next == nullptr) return;
  if (CENTER) {
    float s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) s1 += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    const float mean = nb_warp_sum(s1) / (float)d;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
      s2 = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, s2))));
    }
  }
  s2 = nb_warp_sum(s2);
  const float inv2 = 1.0f / sqrtf(s2 / (float)d + next_eps);
  const float4* n4 = reinterpret_cast<const float4*>(next_gamma);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const float4 g = n4[j * 32 + lane];
    nb_store4<TOut>(out_next + (size_t)r * d + (j * 32 + lane) * 4, v[j].x * inv2 * g.x,
                    v[j].y * inv2 * g.y, v[j].z * inv2 * g.z, v[j].w * inv2 * g.w);
  }
}

template <typename TOut, bool CENTER>
static int rms_add_warp(int nv, cudaStream_t stream, const float* y, const float* gamma, float eps,
                        float* x, const float* next_gamma, float next_eps, void* out_next,
                        void* out_cast, int d, int n_rows) {
  const dim3 grid((n_rows + 3) / 4), block(128);
#define NB_RW(NV_)                                                                              \
  case NV_:                                                                                     \
    NB_CUDA(nb_launch(rms_add_warp_kernel<TOut, NV_, CENTER>, grid, block, 0, stream, y, gamma, eps, x, \
                      next_gamma, next_eps, (TOut*)out_next, (TOut*)out_cast, d, n_rows));      \
    break;
  switch (nv) {
    NB_RW(1) NB_RW(2) NB_RW(3) NB_RW(4) NB_RW(5) NB_RW(6) NB_RW(7) NB_RW(8) NB_RW(9) NB_RW(10)
    NB_RW(11) NB_RW(12) NB_RW(13) NB_RW(14) NB_RW(15) NB_RW(16)
    default: return NB_ERR_UNSUPPORTED;
  }
#undef NB_RW
  return 0;
}

template <bool CENTER>
static int norm_add_impl(const float* y, const float* gamma, float eps, float* x,
                         const float* next_gamma, float next_eps, void* out_next, void* out_cast,
                         int out_dtype, int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && d <= RA_MAX * 1024, NB_ERR_BAD_ARG,
             "norm_add: bad sizes rows=%d d=%d", n_rows, d);
  NB_REQUIRE(gamma != nullptr && (out_next == nullptr || next_gamma != nullptr), NB_ERR_BAD_ARG,
             "norm_add: a norm without its weight");
  NB_REQUIRE(out_dtype == NB_F32 || out_dtype == NB_BF16, NB_ERR_BAD_ARG,
             "norm_add: unknown output dtype %d", out_dtype);
  // many rows of a width that a warp holds in registers: a warp per row
  const bool aligned = (((uintptr_t)y | (uintptr_t)x | (uintptr_t)gamma | (uintptr_t)next_gamma |
                         (uintptr_t)out_next | (uintptr_t)out_cast) & 15) == 0;
  if (d % 128 == 0 && d <= RW_MAX * 128 && n_rows >= 64 && aligned) {
    const int rc = out_dtype == NB_F32
                       ? rms_add_warp<float, CENTER>(d / 128, stream, y, gamma, eps, x, next_gamma, next_eps,
                                             out_next, out_cast, d, n_rows)
                       : rms_add_warp<__nv_bfloat16, CENTER>(d / 128, stream, y, gamma, eps, x, next_gamma,
                                                     next_eps, out_next, out_cast, d, n_rows);
    if (rc != 0) return rc;
    NB_CHECK_LAUNCH("norm_add");
    return 0;
  }
  int threads = 64;
  while (threads < 1024 && threads * (d > 2048 ? RA_MAX : 4) < d) threads *= 2;
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(rms_add_kernel<float, CENTER>, dim3(n_rows), dim3(threads), 0, stream, y, gamma, eps,
                      x, next_gamma, next_eps, (float*)out_next, (float*)out_cast, d));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(rms_add_kernel<__nv_bfloat16, CENTER>, dim3(n_rows), dim3(threads), 0, stream, y,
                      gamma, eps, x, next_gamma, next_eps, (__nv_bfloat16*)out_next,
                      (__nv_bfloat16*)out_cast, d));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "norm_add: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("norm_add");
  return 0;
}

NB_EXPORT int nb_rms_add(const float* y, const float* gamma, float eps, float* x,
                         const float* next_gamma, float next_eps, void* out_next, void* out_cast,
                         int out_dtype, int n_rows, int d, cudaStream_t stream) {
  return norm_add_impl<false>(y, gamma, eps, x, next_gamma, next_eps, out_next, out_cast, out_dtype,
                              n_rows, d, stream);
}

// The same pass with both norms centred (a layer norm with a weight and no shift):
//   x[r] += (y[r] - mean) / sqrt(var + eps) * gamma;  out_next[r] = the same norm of x[r] with
//   next_gamma / next_eps;  out_cast[r] = x[r].  The variance is the mean squared deviation.
NB_EXPORT int nb_ln_add(const float* y, const float* gamma, float eps, float* x,
                        const float* next_gamma, float next_eps, void* out_next, void* out_cast,
                        int out_dtype, int n_rows, int d, cudaStream_t stream) {
  return norm_add_impl<true>(y, gamma, eps, x, next_gamma, next_eps, out_next, out_cast, out_dtype,
                             n_rows, d, stream);
}

// ---------------------------------------------------------------------------------
// out[r, i] = act(x[r, x_col + i]) for fp32 rows x: activations that a product's epilogue does
// not carry.  NB_ACT_TANH; NB_ACT_XIELU with two learned numbers p, q read from `params`:
//   z > 0:  softplus(p) z^2 + z/2;   z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float nb_softplus(float x) {
  return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x)));
}

template <typename TOut>
__global__ void act_rows_kernel(const float* x, int x_stride, int x_col, int act,
                                const float* __restrict__ params, TOut* out, int d, size_t total) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  float ap = 0.0f, an = 0.0f;
  if (act == NB_ACT_XIELU) {
    ap = nb_softplus(params[0]);
    an = 0.5f + nb_softplus(params[1]);
  }
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / d;
    const int i = (int)(e - r * d);
    const float z = x[r * x_stride + x_col + i];
    float v;
    if (act == NB_ACT_XIELU)
      v = z > 0.0f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
    else if (act == NB_ACT_TANH)
      v = tanhf(z);
    else
      v = nb_apply_act(z, act);
    out[e] = nb_from_f32<TOut>(v);
  }
}

NB_EXPORT int nb_act_rows(const float* x, int x_stride, int x_col, int act, const float* params,
                          void* out, int out_dtype, int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0 || d == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && x_col >= 0 && x_stride >= x_col + d, NB_ERR_BAD_ARG,
             "act_rows: bad sizes rows=%d d=%d col=%d stride=%d", n_rows, d, x_col, x_stride);
  NB_REQUIRE(act != NB_ACT_XIELU || params != nullptr, NB_ERR_BAD_ARG,
             "act_rows: this activation has learned numbers");
  const size_t total = (size_t)n_rows * d;
  const int blocks = (int)((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(act_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, x_stride,
                      x_col, act, params, (float*)out, d, total));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(act_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x,
                      x_stride, x_col, act, params, (__nv_bfloat16*)out, d, total));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "act_rows: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("act_rows");
  return 0;
}

// ---------------------------------------------------------------------------------
// out[r, i] = g[r, i] * table[token[r], i]: a gate times the token's row of a table (fp32 gate,
// product in fp32).  Padding rows (token < 0) give zeros.
// ---------------------------------------------------------------------------------
template <typename TT, typename TOut>
__global__ void gather_mul_kernel(const float* g, const TT* __restrict__ table, const int* tokens,
                                  TOut* out, int d, size_t total) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / d;
    const int i = (int)(e - r * d);
    const int tok = tokens[r];
    out[e] = nb_from_f32<TOut>(tok < 0 ? 0.0f : g[e] * nb_to_f32(table[(size_t)tok * d + i]));
  }
}

NB_EXPORT int nb_gather_mul(const float* g, const void* table, int table_dtype, const int* tokens,
                            void* out, int out_dtype, int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0 || d == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0, NB_ERR_BAD_ARG, "gather_mul: bad sizes rows=%d d=%d", n_rows, d);
  const size_t total = (size_t)n_rows * d;
  const int blocks = (int)((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
  typedef __nv_bfloat16 bf;
#define NB_GM(TT, TO)                                                                          \
  NB_CUDA(nb_launch(gather_mul_kernel<TT, TO>, dim3(blocks), dim3(256), 0, stream, g,          \
                    (const TT*)table, tokens, (TO*)out, d, total))
  switch (table_dtype * 2 + out_dtype) {
    case 0: NB_GM(float, float); break;
    case 1: NB_GM(float, bf); break;
    case 2: NB_GM(bf, float); break;
    case 3: NB_GM(bf, bf); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "gather_mul: unknown dtypes %d/%d", table_dtype, out_dtype);
  }
#undef NB_GM
  NB_CHECK_LAUNCH("gather_mul");
  return 0;
}

// ---------------------------------------------------------------------------------
// out[r, i] = act(x[r, gate_col + i]) * x[r, up_col + i] (nb_gate_up): the gated half of a feed-forward whose
// two first products come side by side in one fp32 row.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void glu_rows_kernel(const float* x, int x_stride, int gate_col, int up_col, int act,
                                float act_param, TOut* out, int d, size_t total) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / d;
    const int i = (int)(e - r * d);
    const float* row = x + r * x_stride;
    out[e] = nb_from_f32<TOut>(nb_gate_up<false>(row[gate_col + i], row[up_col + i], act, act_param));
  }
}

NB_EXPORT int nb_glu_rows(const float* x, int x_stride, int gate_col, int up_col, int act,
                          float act_param, void* out, int out_dtype, int n_rows, int d,
                          cudaStream_t stream) {
  if (n_rows == 0 || d == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && gate_col >= 0 && up_col >= 0 && x_stride >= gate_col + d &&
                 x_stride >= up_col + d,
             NB_ERR_BAD_ARG, "glu_rows: bad sizes rows=%d d=%d cols=%d/%d stride=%d", n_rows, d,
             gate_col, up_col, x_stride);
  const size_t total = (size_t)n_rows * d;
  const int blocks = (int)((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(glu_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, x_stride,
                      gate_col, up_col, act, act_param, (float*)out, d, total));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(glu_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x,
                      x_stride, gate_col, up_col, act, act_param, (__nv_bfloat16*)out, d, total));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "glu_rows: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("glu_rows");
  return 0;
}

// ---------------------------------------------------------------------------------
// out[r, out_col + i] = x[r, i] for fp32 rows x, into rows of stride out_stride of another type:
// the stream as the operand of a product, written beside other columns of the same operand.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void cast_cols_kernel(const float* x, TOut* out, int out_stride, int out_col, int d,
                                 size_t total) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / d;
    const int i = (int)(e - r * d);
    out[r * out_stride + out_col + i] = nb_from_f32<TOut>(x[e]);
  }
}

NB_EXPORT int nb_cast_cols(const float* x, void* out, int out_dtype, int out_stride, int out_col,
                           int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0 || d == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && out_col >= 0 && out_stride >= out_col + d, NB_ERR_BAD_ARG,
             "cast_cols: bad sizes rows=%d d=%d col=%d stride=%d", n_rows, d, out_col, out_stride);
  const size_t total = (size_t)n_rows * d;
  const int blocks = (int)((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(cast_cols_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)out,
                      out_stride, out_col, d, total));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(cast_cols_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x,
                      (__nv_bfloat16*)out, out_stride, out_col, d, total));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "cast_cols: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("cast_cols");
  return 0;
}

// ---------------------------------------------------------------------------------
// RMS norm of a whole fp32 row times a weight and a gate:
//   out[r, i] = x[r, i] / sqrt(mean(x[r]^2) + eps) * gamma[i] * sigmoid(g[r, g_col + i])
// (heads side by side normed together, then gated by a projection of the same input).
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void rmsnorm_gated_kernel(const float* x, const float* __restrict__ gamma,
                                     const float* g, int g_stride, int g_col, TOut* out, int d,
                                     float eps) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)r * d;
  const float* gr = g + (size_t)r * g_stride + g_col;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = nb_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    out[(size_t)r * d + i] = nb_from_f32<TOut>(xr[i] * inv * gamma[i] * nb_sigmoid(gr[i]));
}

NB_EXPORT int nb_rmsnorm_gated(const float* x, const float* gamma, const float* g, int g_stride,
                               int g_col, void* out, int out_dtype, int n_rows, int d, float eps,
                               cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && g_col >= 0 && g_stride >= g_col + d, NB_ERR_BAD_ARG,
             "rmsnorm_gated: bad sizes rows=%d d=%d col=%d stride=%d", n_rows, d, g_col, g_stride);
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : (d >= 128 ? 128 : 64));
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(rmsnorm_gated_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, gamma,
                      g, g_stride, g_col, (float*)out, d, eps));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(rmsnorm_gated_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream,
                      x, gamma, g, g_stride, g_col, (__nv_bfloat16*)out, d, eps));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "rmsnorm_gated: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("rmsnorm_gated");
  return 0;
}

// ---------------------------------------------------------------------------------
// Two sublayers' results, each RMS-normed over the row with a weight of its own, averaged into
// the stream, and (optionally) the norm in front of the stream's next reader in the same pass:
//   x[r] += coef * (a[r] / rms(a[r]) * gamma_a + b[r] / rms(b[r]) * gamma_b)       (fp32)
//   out_next[r] = x[r] / sqrt(mean(x[r]^2) + next_eps) * next_gamma    if out_next  (TOut)
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void rms_pair_add_kernel(const float* a, const float* __restrict__ gamma_a,
                                    const float* b, const float* __restrict__ gamma_b, float eps,
                                    float coef, float* x, const float* __restrict__ next_gamma,
                                    float next_eps, TOut* out_next, int d) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* ar = a + (size_t)r * d;
  const float* br = b + (size_t)r * d;
  float* xr = x + (size_t)r * d;
  float sa = 0.0f, sb = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    sa = fmaf(ar[i], ar[i], sa);
    sb = fmaf(br[i], br[i], sb);
  }
  sa = nb_block_sum(sa, red);
  sb = nb_block_sum(sb, red);
  const float ia = 1.0f / sqrtf(sa / (float)d + eps), ib = 1.0f / sqrtf(sb / (float)d + eps);
  float sx = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i] + coef * (ar[i] * ia * gamma_a[i] + br[i] * ib * gamma_b[i]);
    xr[i] = v;
    sx = fmaf(v, v, sx);
  }
  if (out_next == nullptr) return;
  sx = nb_block_sum(sx, red);
  const float ix = 1.0f / sqrtf(sx / (float)d + next_eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    out_next[(size_t)r * d + i] = nb_from_f32<TOut>(xr[i] * ix * next_gamma[i]);
}

NB_EXPORT int nb_rms_pair_add(const float* a, const float* gamma_a, const float* b,
                              const float* gamma_b, float eps, float coef, float* x,
                              const float* next_gamma, float next_eps, void* out_next,
                              int out_dtype, int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0 && (out_next == nullptr || next_gamma != nullptr), NB_ERR_BAD_ARG,
             "rms_pair_add: bad sizes rows=%d d=%d", n_rows, d);
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : (d >= 128 ? 128 : 64));
  if (out_next == nullptr || out_dtype == NB_F32)
    NB_CUDA(nb_launch(rms_pair_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, a,
                      gamma_a, b, gamma_b, eps, coef, x, next_gamma, next_eps, (float*)out_next, d));
  else if (out_dtype == NB_BF16)
    NB_CUDA(nb_launch(rms_pair_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, a,
                      gamma_a, b, gamma_b, eps, coef, x, next_gamma, next_eps,
                      (__nv_bfloat16*)out_next, d));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "rms_pair_add: unknown output dtype %d", out_dtype);
  NB_CHECK_LAUNCH("rms_pair_add");
  return 0;
}

// ---------------------------------------------------------------------------------
// Append this step's keys and values to the paged cache (src/cache.rs:44-57 writes rows
// P..P+T of every head).  Row r of `src` holds [.. | K: n_kv_heads*head_dim | V: same ..]
// starting at column k_col / v_col; it goes to token `pos[r]` of sequence slot `slot[r]`.
// Rows with a negative slot are padding and are skipped.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ src, int src_stride, int k_col, int v_col,
                                 const int* row_slot, const int* row_pos,
                                 NbPagedKV kv) {
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const int page_id = kv.block_table[(size_t)slot * kv.max_pages + pos / kv.page];
  const int in_page = pos % kv.page;
  const int width = kv.n_kv_heads * kv.head_dim;
  const T* srow = src + (size_t)r * src_stride;
  T* kdst = (T*)kv.k;
  T* vdst = (T*)kv.v;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int h = i / kv.head_dim, c = i - h * kv.head_dim;
    const size_t o =
        (((size_t)page_id * kv.n_kv_heads + h) * kv.page + in_page) * kv.head_dim + c;
    kdst[o] = srow[k_col + i];
    vdst[o] = srow[v_col + i];
  }
}

// The same in 16-byte pieces (head size, columns and pitch multiples of 16 bytes): a warp takes
// a row at a time, the lanes its pieces; a block of 8 warps walks over rows.
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_vec_kernel(const T* __restrict__ src, int src_stride, int k_col, int v_col,
                     const int* row_slot, const int* row_pos,
                     NbPagedKV kv, int n_rows) {
  constexpr int E = 16 / sizeof(T);              // elements per piece
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pieces_per_head = kv.head_dim / E;
  const int pieces = kv.n_kv_heads * pieces_per_head;   // of K, and as many of V
  for (int r = blockIdx.x * 8 + warp; r < n_rows; r += gridDim.x * 8) {
    const int slot = row_slot[r];
    if (slot < 0) continue;
    const int pos = row_pos[r];
    const int page_id = kv.block_table[(size_t)slot * kv.max_pages + pos / kv.page];
    const int in_page = pos % kv.page;
    const T* srow = src + (size_t)r * src_stride;
    for (int i = lane; i < 2 * pieces; i += 32) {
      const bool is_v = i >= pieces;
      const int p = is_v ? i - pieces : i;
      const int h = p / pieces_per_head, c = (p - h * pieces_per_head) * E;
      const size_t o = (((size_t)page_id * kv.n_kv_heads + h) * kv.page + in_page) * kv.head_dim + c;
      const uint4 val = *reinterpret_cast<const uint4*>(srow + (is_v ? v_col : k_col) + p * E);
      *reinterpret_cast<uint4*>((is_v ? (T*)kv.v : (T*)kv.k) + o) = val;
    }
  }
}

NB_EXPORT int nb_kv_append(const void* src, int dtype, int src_stride, int k_col, int v_col,
                           const int* row_slot, const int* row_pos, void* k_cache, void* v_cache,
                           const int* block_table, int max_pages, int page, int n_kv_heads,
                           int head_dim, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NbPagedKV kv{k_cache, v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  const int width = n_kv_heads * head_dim;
  const int threads = width >= 256 ? 256 : (width >= 128 ? 128 : 64);
  const int esize = dtype == NB_F32 ? 4 : 2, e16 = 16 / esize;
  const bool vec = (dtype == NB_F32 || dtype == NB_BF16) && head_dim % e16 == 0 &&
                   src_stride % e16 == 0 && k_col % e16 == 0 && v_col % e16 == 0 &&
                   (uintptr_t)src % 16 == 0 && (uintptr_t)k_cache % 16 == 0 &&
                   (uintptr_t)v_cache % 16 == 0;
  if (vec) {
    const int blocks = (n_rows + 7) / 8 < 148 * 8 ? (n_rows + 7) / 8 : 148 * 8;
    if (dtype == NB_F32)
      kv_append_vec_kernel<float><<<blocks, 256, 0, stream>>>(
          (const float*)src, src_stride, k_col, v_col, row_slot, row_pos, kv, n_rows);
    else
      kv_append_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
          (const __nv_bfloat16*)src, src_stride, k_col, v_col, row_slot, row_pos, kv, n_rows);
    NB_CHECK_LAUNCH("kv_append");
    return 0;
  }
  if (dtype == NB_F32)
    kv_append_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)src, src_stride, k_col,
                                                            v_col, row_slot, row_pos, kv);
  else if (dtype == NB_BF16)
    kv_append_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        (const __nv_bfloat16*)src, src_stride, k_col, v_col, row_slot, row_pos, kv);
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "kv_append: unknown dtype %d", dtype);
  NB_CHECK_LAUNCH("kv_append");
  return 0;
}

// ---------------------------------------------------------------------------------
// Between two decode steps on the device: the sampled token becomes the next input and the
// position of every live row moves on by one.  Rows with a negative slot are padding.
// ---------------------------------------------------------------------------------
__global__ void advance_decode_kernel(int* tokens, const int* next,
                                      int* row_pos, const int* row_slot,
                                      int n) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (row_slot[i] >= 0) {
    tokens[i] = next[i];
    row_pos[i] += 1;
  } else {
    tokens[i] = -1;
  }
}

NB_EXPORT int nb_advance_decode(int* tokens, const int* next, int* row_pos, const int* row_slot,
                                int n, cudaStream_t stream) {
  if (n == 0) return 0;
  NB_CUDA(nb_launch(advance_decode_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, next,
                    row_pos, row_slot, n));
  NB_CHECK_LAUNCH("advance_decode");
  return 0;
}
