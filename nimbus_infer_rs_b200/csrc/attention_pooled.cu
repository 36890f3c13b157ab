// Sliding-window attention that also sees pooled blocks of what has left the window, with
// values that are the keys and a sink in the softmax.  fp32 arithmetic on the CUDA cores, any
// sizes, bf16 or fp32 storage.
//
// Three kernels:
//   nb_qk_norm_rope_append  per (row, head): RMS norm of the projected query or key over the
//                           head (fp32, weight shared by the heads), rotation of the first
//                           rot_dims numbers by the row's position (dimension i paired with
//                           i + rot_dims/2, angle = pos * freq[i] in fp32, cos and sin times an
//                           amplitude); queries go to a buffer of their own, keys into the K
//                           plane of the paged store, and the key AS PROJECTED (no norm, no
//                           rotation) into the V plane: the values are the keys.
//   nb_qkv_norm_rope_append the same with values from columns of their own (any head size, a
//                           plane and block table of their own) and the norm optional: what any
//                           attention with rotated, optionally normed queries and keys needs.
//   nb_pool_blocks          for every row that completes a block of `pool` tokens: the mean of
//                           the block's keys as the store holds them, and of its values, into
//                           entry pos / pool of a second paged store.
//   nb_attention_pooled     per (row, head): position i sees tokens j with 0 <= i - j < window
//                           and the blocks b with b*pool + pool - 1 <= i - window, in one
//                           softmax whose denominator has one more term exp(sink_h).
#include "common.cuh"

namespace {

constexpr int QK_THREADS = 128;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(QK_THREADS)
qk_norm_rope_append_kernel(const float* src, int stride, int q_col, int k_col, int v_col,
                           const float* __restrict__ q_gamma, const float* __restrict__ k_gamma,
                           float eps, const float* __restrict__ freq, int rot_dims, float amplitude,
                           const int* row_slot, const int* row_pos, TQ* q_out, TC* kc, TC* vc,
                           const int* block_table, int max_pages, const int* v_table,
                           int v_max_pages, int page, int n_heads, int n_kv_heads, int d, int dv,
                           int write) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = row_slot[r];
  TQ* qo = q_out + (size_t)r * n_heads * d;
  if (slot < 0) {
    for (int i = threadIdx.x; i < n_heads * d; i += QK_THREADS) qo[i] = nb_from_f32<TQ>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int half = rot_dims / 2;
  const float* row = src + (size_t)r * stride;
  size_t cache_row = 0, v_row = 0;
  if (write) {
    const int page_id = block_table[(size_t)slot * max_pages + pos / page];
    cache_row = (size_t)page_id * n_kv_heads * page + (pos % page);   // + g * page, then * d
    const int v_page = v_table[(size_t)slot * v_max_pages + pos / page];
    v_row = (size_t)v_page * n_kv_heads * page + (pos % page);
  }
  for (int hh = warp; hh < n_heads + (write ? n_kv_heads : 0); hh += QK_THREADS / 32) {
    const bool is_q = hh < n_heads;
    const int g = hh - n_heads;
    const float* x = row + (is_q ? q_col + hh * d : k_col + g * d);
    const float* gamma = is_q ? q_gamma : k_gamma;
    float inv = 1.0f;
    if (gamma != nullptr) {
      float ss = 0.0f;
      for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
      ss = nb_warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)d + eps);
    }
    TC* kd = is_q ? nullptr : kc + (cache_row + (size_t)g * page) * d;
    TQ* qd = qo + (size_t)hh * d;
    for (int i = lane; i < half; i += 32) {
      float a = x[i], b = x[i + half];
      if (gamma != nullptr) {
        a = a * inv * gamma[i];
        b = b * inv * gamma[i + half];
      }
      float s, c;
      sincosf((float)pos * freq[i], &s, &c);
      s *= amplitude;
      c *= amplitude;
      const float a2 = a * c - b * s, b2 = b * c + a * s;
      if (is_q) {
        qd[i] = nb_from_f32<TQ>(a2);
        qd[i + half] = nb_from_f32<TQ>(b2);
      } else {
        kd[i] = nb_from_f32<TC>(a2);
        kd[i + half] = nb_from_f32<TC>(b2);
      }
    }
    for (int i = rot_dims + lane; i < d; i += 32) {
      const float a = gamma != nullptr ? x[i] * inv * gamma[i] : x[i];
      if (is_q) qd[i] = nb_from_f32<TQ>(a);
      else kd[i] = nb_from_f32<TC>(a);
    }
    if (!is_q) {
      // the value: the key as projected, or columns of its own
      const float* xv = v_col < 0 ? x : row + v_col + g * dv;
      TC* vd = vc + (v_row + (size_t)g * page) * dv;
      for (int i = lane; i < dv; i += 32) vd[i] = nb_from_f32<TC>(xv[i]);
    }
  }
}

template <typename TC>
__global__ void pool_blocks_kernel(const int* row_slot, const int* row_pos, const TC* kc,
                                   const TC* vc, const int* block_table, int max_pages, TC* bk,
                                   TC* bv, const int* b_table, int b_max_pages, int page,
                                   int n_kv_heads, int d, int pool) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  if ((pos + 1) % pool != 0) return;
  const int b = pos / pool;
  const int* pages = block_table + (size_t)slot * max_pages;
  const int b_page = b_table[(size_t)slot * b_max_pages + b / page];
  const float inv = 1.0f / (float)pool;
  const int width = n_kv_heads * d;
  for (int e = threadIdx.x; e < width; e += blockDim.x) {
    const int g = e / d, i = e - g * d;
    float sk = 0.0f, sv = 0.0f;
    for (int j = pos + 1 - pool; j <= pos; ++j) {
      const size_t o = (((size_t)pages[j / page] * n_kv_heads + g) * page + (j % page)) * d + i;
      sk += nb_to_f32(kc[o]);
      sv += nb_to_f32(vc[o]);
    }
    const size_t o = (((size_t)b_page * n_kv_heads + g) * page + (b % page)) * d + i;
    bk[o] = nb_from_f32<TC>(sk * inv);
    bv[o] = nb_from_f32<TC>(sv * inv);
  }
}

constexpr int AT_THREADS = 128;
constexpr int AT_WARPS = AT_THREADS / 32;
constexpr int AT_CHUNK = 1024;   // scores held in shared memory at a time
constexpr int AT_MAXD = 256;     // largest head
constexpr int AT_DPL = AT_MAXD / 32;

// The entries a row sees, numbered 0 .. n_blocks + n_tokens - 1: blocks first, then tokens.
template <typename TC>
struct Seen {
  const TC* k;
  const TC* v;
  const TC* bk;
  const TC* bv;
  const int* pages;
  const int* b_pages;
  int page, n_kv_heads, g, d, n_blocks, j_begin;
  __device__ __forceinline__ size_t offset(int e, bool& block) const {
    block = e < n_blocks;
    const int idx = block ? e : j_begin + (e - n_blocks);
    const int pg = block ? b_pages[idx / page] : pages[idx / page];
    return (((size_t)pg * n_kv_heads + g) * page + (idx % page)) * d;
  }
};

template <typename TQ, typename TC, typename TOut>
__global__ void __launch_bounds__(AT_THREADS)
attention_pooled_kernel(const TQ* q, const int* row_slot, const int* row_pos, const TC* kc,
                        const TC* vc, const int* block_table, int max_pages, const TC* bk,
                        const TC* bv, const int* b_table, int b_max_pages, int page, int n_heads,
                        int n_kv_heads, int d, const float* sink, TOut* out, float scale,
                        int window, int pool) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float q_s[AT_MAXD];
  __shared__ float scores[AT_CHUNK];
  __shared__ float part[AT_WARPS][AT_MAXD];
  __shared__ float red[32];
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  TOut* o = out + ((size_t)r * n_heads + h) * d;
  const int slot = row_slot[r];
  if (slot < 0) {
    for (int i = tid; i < d; i += AT_THREADS) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  Seen<TC> seen;
  seen.k = kc; seen.v = vc; seen.bk = bk; seen.bv = bv;
  seen.pages = block_table + (size_t)slot * max_pages;
  seen.b_pages = bk != nullptr ? b_table + (size_t)slot * b_max_pages : nullptr;
  seen.page = page; seen.n_kv_heads = n_kv_heads; seen.g = h / (n_heads / n_kv_heads); seen.d = d;
  seen.j_begin = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  seen.n_blocks = (bk != nullptr && window > 0 && pool > 0 && pos + 1 >= window)
                      ? (pos + 1 - window) / pool : 0;
  const int n_seen = seen.n_blocks + (pos + 1 - seen.j_begin);

  const TQ* qr = q + ((size_t)r * n_heads + h) * d;
  for (int i = tid; i < d; i += AT_THREADS) q_s[i] = nb_to_f32(qr[i]);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[AT_DPL];
#pragma unroll
  for (int a = 0; a < AT_DPL; ++a) acc[a] = 0.0f;

  for (int c0 = 0; c0 < n_seen; c0 += AT_CHUNK) {
    const int c1 = min(c0 + AT_CHUNK, n_seen);
    float cmax = -INFINITY;
    for (int e = c0 + warp; e < c1; e += AT_WARPS) {
      bool blk;
      const size_t off = seen.offset(e, blk);
      const TC* kr = (blk ? seen.bk : seen.k) + off;
      float dot = 0.0f;
      for (int i = lane; i < d; i += 32) dot = fmaf(q_s[i], nb_to_f32(kr[i]), dot);
      dot = nb_warp_sum(dot) * scale;
      if (lane == 0) scores[e - c0] = dot;
      cmax = fmaxf(cmax, dot);
    }
    cmax = nb_block_max(cmax, red);
    const float m_new = fmaxf(m_run, cmax);
    float csum = 0.0f;
    for (int e = c0 + tid; e < c1; e += AT_THREADS) {
      const float p = expf(scores[e - c0] - m_new);
      scores[e - c0] = p;
      csum += p;
    }
    csum = nb_block_sum(csum, red);   // also orders the writes of `scores` before the reads below
    const float rescale = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * rescale + csum;
#pragma unroll
    for (int a = 0; a < AT_DPL; ++a) acc[a] *= rescale;
    // the weighted sum: warps over entries, lanes over the head's dims
    for (int e = c0 + warp; e < c1; e += AT_WARPS) {
      bool blk;
      const size_t off = seen.offset(e, blk);
      const TC* vr = (blk ? seen.bv : seen.v) + off;
      const float p = scores[e - c0];
#pragma unroll
      for (int a = 0; a < AT_DPL; ++a) {
        const int i = lane + 32 * a;
        if (i < d) acc[a] = fmaf(p, nb_to_f32(vr[i]), acc[a]);
      }
    }
    m_run = m_new;
    __syncthreads();   // `scores` is rewritten by the next chunk
  }
  // every warp holds the sum over its entries; warp 0 adds them up in a fixed order
#pragma unroll
  for (int a = 0; a < AT_DPL; ++a) {
    const int i = lane + 32 * a;
    if (i < d) part[warp][i] = acc[a];
  }
  __syncthreads();
  if (warp != 0) return;
  float denom = l_run, fix = 1.0f;
  if (sink != nullptr) {
    // one more term of the denominator, with no key and no value
    const float s = sink[h];
    const float m_f = fmaxf(m_run, s);
    fix = expf(m_run - m_f);
    denom = l_run * fix + expf(s - m_f);
  }
  const float inv = denom > 0.0f ? fix / denom : 0.0f;
  for (int i = lane; i < d; i += 32) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < AT_WARPS; ++w) v += part[w][i];
    o[i] = nb_from_f32<TOut>(v * inv);
  }
}

}  // namespace

typedef __nv_bfloat16 bf16;

// src: fp32 [n_rows][stride], the queries' heads at columns q_col .., the keys' at k_col ..;
// q_out: [n_rows][n_heads*d]; kc, vc: planes [n_pages][n_kv_heads][page][d]; freq: fp32
// [rot_dims/2] (null when rot_dims is 0).  write == 0: queries only (a reader of another
// layer's store).
// The general form.  q_gamma / k_gamma: null for no norm.  v_col < 0: the values are the keys as
// projected (dv = d, into `vc` by the keys' block table); else the values are columns v_col ..
// of `src` (n_kv_heads heads of dv), written to the plane `vc`, whose pages `v_table` lists (the
// keys' table again when keys and values share a store of two planes).
NB_EXPORT int nb_qkv_norm_rope_append(const float* src, int stride, int q_col, int k_col, int v_col,
                                      const float* q_gamma, const float* k_gamma, float eps,
                                      const float* freq, int rot_dims, float amplitude,
                                      const int* row_slot, const int* row_pos, void* q_out,
                                      int q_dtype, void* kc, void* vc, int cache_dtype,
                                      const int* block_table, int max_pages, const int* v_table,
                                      int v_max_pages, int page, int n_heads, int n_kv_heads, int d,
                                      int dv, int write, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && d > 0 && dv > 0 && page > 0 && rot_dims >= 0 &&
                 rot_dims % 2 == 0 && rot_dims <= d && (rot_dims == 0 || freq != nullptr) &&
                 (v_col >= 0 || dv == d) && (q_gamma == nullptr) == (k_gamma == nullptr),
             NB_ERR_BAD_ARG, "qkv_norm_rope_append: bad sizes heads=%d/%d d=%d/%d rot=%d", n_heads,
             n_kv_heads, d, dv, rot_dims);
  if (v_table == nullptr) { v_table = block_table; v_max_pages = max_pages; }
#define NB_QK(TQ, TC)                                                                             \
  NB_CUDA(nb_launch(qk_norm_rope_append_kernel<TQ, TC>, dim3(n_rows), dim3(QK_THREADS), 0, stream, \
                    src, stride, q_col, k_col, v_col, q_gamma, k_gamma, eps, freq, rot_dims,      \
                    amplitude, row_slot, row_pos, (TQ*)q_out, (TC*)kc, (TC*)vc, block_table,      \
                    max_pages, v_table, v_max_pages, page, n_heads, n_kv_heads, d, dv, write))
  switch (q_dtype * 2 + cache_dtype) {
    case 0: NB_QK(float, float); break;
    case 1: NB_QK(float, bf16); break;
    case 2: NB_QK(bf16, float); break;
    case 3: NB_QK(bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "qkv_norm_rope_append: unknown dtypes %d/%d", q_dtype, cache_dtype);
  }
#undef NB_QK
  NB_CHECK_LAUNCH("qkv_norm_rope_append");
  return 0;
}

NB_EXPORT int nb_qk_norm_rope_append(const float* src, int stride, int q_col, int k_col,
                                     const float* q_gamma, const float* k_gamma, float eps,
                                     const float* freq, int rot_dims, float amplitude,
                                     const int* row_slot, const int* row_pos, void* q_out,
                                     int q_dtype, void* kc, void* vc, int cache_dtype,
                                     const int* block_table, int max_pages, int page, int n_heads,
                                     int n_kv_heads, int d, int write, int n_rows,
                                     cudaStream_t stream) {
  NB_REQUIRE(q_gamma != nullptr && k_gamma != nullptr, NB_ERR_BAD_ARG,
             "qk_norm_rope_append: a norm without its weight");
  return nb_qkv_norm_rope_append(src, stride, q_col, k_col, -1, q_gamma, k_gamma, eps, freq, rot_dims,
                                 amplitude, row_slot, row_pos, q_out, q_dtype, kc, vc, cache_dtype,
                                 block_table, max_pages, block_table, max_pages, page, n_heads,
                                 n_kv_heads, d, d, write, n_rows, stream);
}

NB_EXPORT int nb_pool_blocks(const int* row_slot, const int* row_pos, const void* kc, const void* vc,
                             const int* block_table, int max_pages, void* bk, void* bv,
                             const int* b_table, int b_max_pages, int cache_dtype, int page,
                             int n_kv_heads, int d, int pool, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(pool > 0 && page > 0 && n_kv_heads > 0 && d > 0, NB_ERR_BAD_ARG,
             "pool_blocks: bad sizes pool=%d page=%d heads=%d d=%d", pool, page, n_kv_heads, d);
  const int threads = n_kv_heads * d >= 256 ? 256 : 128;
  if (cache_dtype == NB_F32)
    NB_CUDA(nb_launch(pool_blocks_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, row_slot,
                      row_pos, (const float*)kc, (const float*)vc, block_table, max_pages,
                      (float*)bk, (float*)bv, b_table, b_max_pages, page, n_kv_heads, d, pool));
  else if (cache_dtype == NB_BF16)
    NB_CUDA(nb_launch(pool_blocks_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, row_slot,
                      row_pos, (const bf16*)kc, (const bf16*)vc, block_table, max_pages, (bf16*)bk,
                      (bf16*)bv, b_table, b_max_pages, page, n_kv_heads, d, pool));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "pool_blocks: unknown cache dtype %d", cache_dtype);
  NB_CHECK_LAUNCH("pool_blocks");
  return 0;
}

// q: [n_rows][n_heads*d]; kc, vc and (optional) bk, bv: paged planes with their block tables;
// sink: fp32 [n_heads] or null; out: [n_rows][n_heads*d].
NB_EXPORT int nb_attention_pooled(const void* q, int q_dtype, const int* row_slot,
                                  const int* row_pos, const void* kc, const void* vc,
                                  const int* block_table, int max_pages, const void* bk,
                                  const void* bv, const int* b_table, int b_max_pages,
                                  int cache_dtype, int page, int n_heads, int n_kv_heads, int d,
                                  const float* sink, void* out, int out_dtype, float scale,
                                  int window, int pool, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(d >= 1 && d <= AT_MAXD, NB_ERR_UNSUPPORTED,
             "attention_pooled: heads of %d are outside 1..%d", d, AT_MAXD);
  NB_REQUIRE(n_heads >= 1 && n_heads <= 65535 && n_kv_heads >= 1 && n_heads % n_kv_heads == 0 &&
                 page > 0 && window >= 0 && pool >= 0,
             NB_ERR_BAD_ARG, "attention_pooled: bad sizes heads=%d/%d page=%d window=%d pool=%d",
             n_heads, n_kv_heads, page, window, pool);
  const dim3 grid(n_rows, n_heads);
#define NB_AP(TQ, TC, TO)                                                                        \
  NB_CUDA(nb_launch(attention_pooled_kernel<TQ, TC, TO>, grid, dim3(AT_THREADS), 0, stream,      \
                    (const TQ*)q, row_slot, row_pos, (const TC*)kc, (const TC*)vc, block_table,  \
                    max_pages, (const TC*)bk, (const TC*)bv, b_table, b_max_pages, page, n_heads, \
                    n_kv_heads, d, sink, (TO*)out, scale, window, pool))
  switch (q_dtype * 4 + cache_dtype * 2 + out_dtype) {
    case 0: NB_AP(float, float, float); break;
    case 3: NB_AP(float, bf16, bf16); break;
    case 7: NB_AP(bf16, bf16, bf16); break;
    case 6: NB_AP(bf16, bf16, float); break;
    default:
      NB_REQUIRE(false, NB_ERR_UNSUPPORTED, "attention_pooled: dtypes %d/%d/%d are not built",
                 q_dtype, cache_dtype, out_dtype);
  }
#undef NB_AP
  NB_CHECK_LAUNCH("attention_pooled");
  return 0;
}
