// Causal attention over two paged planes (keys of head size d, values of head size dv, a block
// table each) with a cap on the scores and a sink in the softmax:
//
//   score = scale * q . k;   with softcap > 0:  score = softcap * tanh(score / softcap)
//   weights = softmax over the seen keys, the denominator holding one more term exp(sink_h)
//             (no key, no value; neither scaled nor capped)
//
// What a position sees (nb_attention_masked; nb_attention_capped sees every j <= i):
//   window > 0:  j <= i with i - j < window, and also every j < keep_first (the first tokens
//                stay visible, at their true positions)
//   chunk > 0:   j <= i with floor(i / chunk) == floor(j / chunk), chunks counted from position 0
// With `gate` (fp32 rows, one logit per head at columns gate_col ..) head h's result is
// multiplied by sigmoid(gate[r][gate_col + h]).
//
// fp32 arithmetic on the CUDA cores, any sizes, bf16 or fp32 storage: the 32-bit path, and the
// path of shapes the tensor-core kernel leaves out.  A CTA per (row, head); the scores of up to
// 1024 keys at a time in shared memory; warps over keys, lanes over the head's numbers; every
// row is reduced in the same order whatever the step's cut or the batch.
#include "common.cuh"

namespace {

constexpr int AC_THREADS = 128;
constexpr int AC_WARPS = AC_THREADS / 32;
constexpr int AC_CHUNK = 1024;
constexpr int AC_MAXD = 256;
constexpr int AC_DPL = AC_MAXD / 32;

template <typename TQ, typename TC, typename TOut>
__global__ void __launch_bounds__(AC_THREADS)
attention_capped_kernel(const TQ* q, const int* row_slot, const int* row_pos, const TC* kc,
                        const int* k_table, int k_max_pages, const TC* vc, const int* v_table,
                        int v_max_pages, int page, int n_heads, int n_kv_heads, int d, int dv,
                        const float* __restrict__ sink, TOut* out, float scale, float softcap,
                        int window, int keep_first, int chunk, const float* gate, int gate_stride,
                        int gate_col) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float scores[AC_CHUNK];
  __shared__ float q_s[AC_MAXD];
  __shared__ float part[AC_WARPS][AC_MAXD];
  __shared__ float red[32];
  const int r = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  TOut* o = out + ((size_t)r * n_heads + h) * dv;
  const int slot = row_slot[r];
  if (slot < 0) {
    for (int i = tid; i < dv; i += AC_THREADS) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int g = h / (n_heads / n_kv_heads);
  const int* kt = k_table + (size_t)slot * k_max_pages;
  const int* vt = v_table + (size_t)slot * v_max_pages;
  const TQ* qr = q + ((size_t)r * n_heads + h) * d;
  for (int i = tid; i < d; i += AC_THREADS) q_s[i] = nb_to_f32(qr[i]);
  __syncthreads();
  // the seen keys: [0, n_head) and [lo, pos]; index t of the walk is key t below n_head, else
  // key lo + (t - n_head)
  int lo = 0;
  if (chunk > 0) lo = (pos / chunk) * chunk;
  if (window > 0) lo = max(lo, pos - window + 1);
  const int n_head = window > 0 ? min(keep_first, lo) : 0;
  const int shift = lo - n_head;
  const int n_seen = n_head + pos + 1 - lo;
  float m_run = -INFINITY, l_run = 0.0f;
  float acc[AC_DPL];
#pragma unroll
  for (int a = 0; a < AC_DPL; ++a) acc[a] = 0.0f;
  const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;

  for (int c0 = 0; c0 < n_seen; c0 += AC_CHUNK) {
    const int c1 = min(c0 + AC_CHUNK, n_seen);
    float cmax = -INFINITY;
    for (int t = c0 + warp; t < c1; t += AC_WARPS) {
      const int e = t < n_head ? t : t + shift;
      const TC* kr = kc + (((size_t)kt[e / page] * n_kv_heads + g) * page + (e % page)) * d;
      float dot = 0.0f;
      for (int i = lane; i < d; i += 32) dot = fmaf(q_s[i], nb_to_f32(kr[i]), dot);
      dot = nb_warp_sum(dot) * scale;
      if (softcap > 0.0f) dot = softcap * tanhf(dot * inv_cap);
      if (lane == 0) scores[t - c0] = dot;
      cmax = fmaxf(cmax, dot);
    }
    cmax = nb_block_max(cmax, red);
    const float m_new = fmaxf(m_run, cmax);
    float csum = 0.0f;
    for (int e = c0 + tid; e < c1; e += AC_THREADS) {
      const float p = expf(scores[e - c0] - m_new);
      scores[e - c0] = p;
      csum += p;
    }
    csum = nb_block_sum(csum, red);   // also orders the writes of `scores` before the reads below
    const float rescale = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * rescale + csum;
#pragma unroll
    for (int a = 0; a < AC_DPL; ++a) acc[a] *= rescale;
    for (int t = c0 + warp; t < c1; t += AC_WARPS) {
      const int e = t < n_head ? t : t + shift;
      const TC* vr = vc + (((size_t)vt[e / page] * n_kv_heads + g) * page + (e % page)) * dv;
      const float p = scores[t - c0];
#pragma unroll
      for (int a = 0; a < AC_DPL; ++a) {
        const int i = lane + 32 * a;
        if (i < dv) acc[a] = fmaf(p, nb_to_f32(vr[i]), acc[a]);
      }
    }
    m_run = m_new;
    __syncthreads();   // `scores` is rewritten by the next chunk
  }
#pragma unroll
  for (int a = 0; a < AC_DPL; ++a) {
    const int i = lane + 32 * a;
    if (i < dv) part[warp][i] = acc[a];
  }
  __syncthreads();
  if (warp != 0) return;
  float denom = l_run, fix = 1.0f;
  if (sink != nullptr) {
    const float s = sink[h];
    const float m_f = fmaxf(m_run, s);
    fix = expf(m_run - m_f);
    denom = l_run * fix + expf(s - m_f);
  }
  float inv = denom > 0.0f ? fix / denom : 0.0f;
  if (gate != nullptr) inv *= nb_sigmoid(gate[(size_t)r * gate_stride + gate_col + h]);
  for (int i = lane; i < dv; i += 32) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < AC_WARPS; ++w) v += part[w][i];
    o[i] = nb_from_f32<TOut>(v * inv);
  }
}

}  // namespace

typedef __nv_bfloat16 bf16;

// q: [n_rows][n_heads*d]; kc: [n_pages][n_kv_heads][page][d]; vc: [n_pages][n_kv_heads][page][dv];
// sink: fp32 [n_heads] or null; softcap: 0 for none; window / keep_first / chunk: 0 for none;
// gate: fp32 [n_rows][gate_stride] or null; out: [n_rows][n_heads*dv].
NB_EXPORT int nb_attention_masked(const void* q, int q_dtype, const int* row_slot, const int* row_pos,
                                  const void* kc, const int* k_table, int k_max_pages,
                                  const void* vc, const int* v_table, int v_max_pages,
                                  int cache_dtype, int page, int n_heads, int n_kv_heads, int d,
                                  int dv, const float* sink, void* out, int out_dtype, float scale,
                                  float softcap, int window, int keep_first, int chunk,
                                  const float* gate, int gate_stride, int gate_col, int n_rows,
                                  cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(d >= 1 && d <= AC_MAXD && dv >= 1 && dv <= AC_MAXD, NB_ERR_UNSUPPORTED,
             "attention_masked: heads of %d / %d are outside 1..%d", d, dv, AC_MAXD);
  NB_REQUIRE(n_heads >= 1 && n_heads <= 65535 && n_kv_heads >= 1 && n_heads % n_kv_heads == 0 &&
                 page > 0 && softcap >= 0.0f && window >= 0 && keep_first >= 0 && chunk >= 0 &&
                 (gate == nullptr || gate_stride >= gate_col + n_heads),
             NB_ERR_BAD_ARG, "attention_masked: bad sizes heads=%d/%d page=%d mask=%d/%d/%d",
             n_heads, n_kv_heads, page, window, keep_first, chunk);
  const dim3 grid(n_rows, n_heads);
#define NB_AC(TQ, TC, TO)                                                                        \
  NB_CUDA(nb_launch(attention_capped_kernel<TQ, TC, TO>, grid, dim3(AC_THREADS), 0, stream,      \
                    (const TQ*)q, row_slot, row_pos, (const TC*)kc, k_table, k_max_pages,        \
                    (const TC*)vc, v_table, v_max_pages, page, n_heads, n_kv_heads, d, dv, sink, \
                    (TO*)out, scale, softcap, window, keep_first, chunk, gate, gate_stride,      \
                    gate_col))
  switch (q_dtype * 4 + cache_dtype * 2 + out_dtype) {
    case 0: NB_AC(float, float, float); break;
    case 7: NB_AC(bf16, bf16, bf16); break;
    case 6: NB_AC(bf16, bf16, float); break;
    default:
      NB_REQUIRE(false, NB_ERR_UNSUPPORTED, "attention_masked: dtypes %d/%d/%d are not built",
                 q_dtype, cache_dtype, out_dtype);
  }
#undef NB_AC
  NB_CHECK_LAUNCH("attention_masked");
  return 0;
}

NB_EXPORT int nb_attention_capped(const void* q, int q_dtype, const int* row_slot, const int* row_pos,
                                  const void* kc, const int* k_table, int k_max_pages,
                                  const void* vc, const int* v_table, int v_max_pages,
                                  int cache_dtype, int page, int n_heads, int n_kv_heads, int d,
                                  int dv, const float* sink, void* out, int out_dtype, float scale,
                                  float softcap, int n_rows, cudaStream_t stream) {
  return nb_attention_masked(q, q_dtype, row_slot, row_pos, kc, k_table, k_max_pages, vc, v_table,
                             v_max_pages, cache_dtype, page, n_heads, n_kv_heads, d, dv, sink, out,
                             out_dtype, scale, softcap, 0, 0, 0, nullptr, 0, 0, n_rows, stream);
}
