// Prefill attention: many query rows per sequence over the paged key/value cache, bf16 on the
// tensor cores with fp32 softmax (running maximum and sum per row, probabilities rounded to
// bf16 only as the operand of the value product).
//
// One CTA takes 64 consecutive query rows of one sequence and one head; each of its four warps
// owns 16 rows.  Key/value pages (64 tokens x head_dim, contiguous in the cache) are streamed
// into shared memory with cp.async, two pages in flight; scores are mma.sync m16n8k16 products
// of the query fragments (held in registers) with the page's keys, the causal limit (and the
// window) is applied to the fp32 scores, and the probabilities, re-used in place as the next
// product's A operand, multiply the page's values.  Rows of a sequence sit anywhere in the
// packed batch (cu_rows) and start at any cached length (seq_pos0), so chunks that continue a
// sequence work like whole prompts.
//
// This kernel uses the legacy mma.sync tensor-core path, not tcgen05.
//
// Reference: src/model.rs:401-422 (scores = dot(q,k)*scale for keys 0..P+i, softmax with the
// maximum subtracted, weighted values).
#include "attention_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int THREADS = 128;
constexpr int BLOCK_Q = 64;
constexpr int PAGE_TOKENS = 64;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// EXTRA: the kernel also takes a second paged store of pooled blocks (entry b = the mean key
// and mean value of tokens b*pool .. b*pool+pool-1; row i sees it once b*pool + pool - 1 <=
// i - window) whose pages are walked before the window's, and a sink per head: one more term
// exp(sink_h) of the softmax's denominator, without a key, a value or the score scale.  Or, in
// place of the blocks, the options of NbAttnOpts: a window that keeps the sequence's first tokens
// (their pages, where they lie before the window's, are the units walked first), a mask by blocks
// of positions, a gate per head; and with softcap > 0 scores bent by softcap * tanh(score /
// softcap).
template <int HD, typename TOut, bool EXTRA>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, int q_col,
                         const int* __restrict__ cu_rows, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_pos0, NbPagedKV kv, int group,
                         TOut* __restrict__ out, int out_stride, float scale, int window,
                         NbPagedKV blocks, int pool, const float* __restrict__ sink,
                         NbAttnOpts opt, float softcap) {
  constexpr int ROW = HD + 8;              // padded row (elements): ldmatrix without conflicts
  constexpr int KS = HD / 16;              // k-steps of the score product
  constexpr int NT = HD / 8;               // n-tiles of the value product
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);          // [64][ROW]
  bf16* kv_s = q_s + BLOCK_Q * ROW;                        // [2 stages][K | V][64][ROW]

  const int tile = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  const int q0 = tile * BLOCK_Q;
  if (q0 >= n_q) return;
  const int slot = seq_slot[s];
  if (slot < 0) {
    // a sequence that has ended (a decode session keeps its row): zeros, not what the buffer held
    if (EXTRA)
      for (int i = threadIdx.x; i < min(BLOCK_Q, n_q - q0) * HD; i += THREADS)
        out[(size_t)(row0 + q0 + i / HD) * out_stride + h * HD + i % HD] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos0 = seq_pos0[s];
  const int kvh = h / group;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(BLOCK_Q, n_q - q0);
  const int last_pos = pos0 + q0 + rows_here - 1;                    // newest key any row sees
  const int first_key = EXTRA ? opt.first_key(pos0 + q0)
                              : ((window > 0) ? max(0, pos0 + q0 + 1 - window) : 0);
  const int p_begin = first_key / PAGE_TOKENS, p_end = last_pos / PAGE_TOKENS + 1;
  const int* table = kv.block_table + (size_t)slot * kv.max_pages;
  // blocks the tile's last row sees, and their pages: walked first, as units 0 .. n_bpages - 1
  const int nb_tile = (EXTRA && pool > 0 && window > 0 && blocks.k != nullptr)
                          ? max(0, (last_pos + 1 - window) / pool) : 0;
  // or the pages of kept first tokens that lie before the window's first page
  const int keep_first = (EXTRA && opt.keeps() && nb_tile == 0) ? opt.keep_first : 0;
  const int n_hpages = min((keep_first + PAGE_TOKENS - 1) / PAGE_TOKENS, p_begin);
  const int n_bpages = n_hpages > 0 ? n_hpages : (nb_tile + PAGE_TOKENS - 1) / PAGE_TOKENS;
  const int* btable = (EXTRA && n_bpages > 0 && n_hpages == 0)
                          ? blocks.block_table + (size_t)slot * blocks.max_pages : nullptr;
  const int n_units = n_bpages + (p_end - p_begin);

  auto issue = [&](int unit, int stage) {
    const bool blk = EXTRA && unit < n_bpages && n_hpages == 0;
    const int page_id = blk ? btable[unit] : table[unit < n_bpages ? unit : p_begin + unit - n_bpages];
    const bf16* ksrc = (const bf16*)(blk ? blocks.k : kv.k) + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    const bf16* vsrc = (const bf16*)(blk ? blocks.v : kv.v) + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    bf16* kdst = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW;
    bf16* vdst = kdst + PAGE_TOKENS * ROW;
    constexpr int CPR = HD / 8;   // 16-byte chunks per row
    for (int i = tid; i < PAGE_TOKENS * CPR; i += THREADS) {
      const int r = i / CPR, c = i - r * CPR;
      cp_async16(kdst + r * ROW + c * 8, ksrc + r * HD + c * 8);
      cp_async16(vdst + r * ROW + c * 8, vsrc + r * HD + c * 8);
    }
    cp_async_commit();
  };
  issue(0, 0);

  // the query tile: rows beyond the sequence are zero
  {
    constexpr int CPR = HD / 8;
    for (int i = tid; i < BLOCK_Q * CPR; i += THREADS) {
      const int r = i / CPR, c = i - r * CPR;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows_here)
        v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + q0 + r) * q_stride + q_col +
                                            (size_t)h * HD + c * 8);
      *reinterpret_cast<uint4*>(q_s + r * ROW + c * 8) = v;
    }
  }
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldmatrix_x4(qf[ks], q_s + (warp * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8);

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const bool capped = EXTRA && softcap > 0.0f;
  // scores in units of log2(e); with a cap, first softcap * tanh(scale * score / softcap)
  const float sl2 = (capped ? 1.0f : scale) * 1.4426950408889634f;
  const float cap_in = capped ? scale / softcap : 0.0f;
  auto bent = [&](float raw) { return capped ? nb_softcap(raw, cap_in, softcap) * sl2 : raw * sl2; };
  const int qpos_a = pos0 + q0 + warp * 16 + g;     // absolute position of row g
  const int qpos_b = qpos_a + 8;                    // ... and of row g + 8
  // blocks each of the two rows sees
  const int nb_a = (EXTRA && nb_tile > 0 && qpos_a + 1 >= window) ? (qpos_a + 1 - window) / pool : 0;
  const int nb_b = (EXTRA && nb_tile > 0 && qpos_b + 1 >= window) ? (qpos_b + 1 - window) / pool : 0;

  for (int u = 0; u < n_units; ++u) {
    const int stage = u & 1;
    const bool head = EXTRA && u < n_hpages;        // a page of kept first tokens
    const bool blk = EXTRA && u < n_bpages && !head;
    const int p = head ? u : p_begin + u - n_bpages;   // the page of tokens (when not blocks)
    if (u + 1 < n_units) {
      issue(u + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kt = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW;
    bf16* vt = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW + PAGE_TOKENS * ROW;
    // Rows of the last page after the newest key hold whatever an earlier owner of the page
    // left there.  Their probabilities are zero, but zero times a non-finite value is not: the
    // value rows are cleared in the staged copy (masked scores are replaced, not multiplied).
    const int tail_row = blk ? nb_tile - u * PAGE_TOKENS : last_pos + 1 - p * PAGE_TOKENS;   // (a head page is full)
    if (tail_row < PAGE_TOKENS) {   // uniform over the CTA
      constexpr int CPR = HD / 8;
      for (int i = tid; i < (PAGE_TOKENS - tail_row) * CPR; i += THREADS) {
        const int r = tail_row + i / CPR, c = (i % CPR) * 8;
        *reinterpret_cast<uint4*>(vt + r * ROW + c) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }

    // scores of 16 rows x 64 keys
    float sc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[n][j] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {   // two key tiles of 8 per ldmatrix.x4
        uint32_t kb[4];
        ldmatrix_x4(kb, kt + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + ks * 16 +
                            ((lane >> 3) & 1) * 8);
        mma_bf16(sc[2 * n2], qf[ks], kb[0], kb[1]);
        mma_bf16(sc[2 * n2 + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // causal limit, window, scale; running maximum.  A page that lies wholly before the first
    // row of this warp (and needs no window) is visible to all of its rows: no comparisons.
    const int j0 = p * PAGE_TOKENS;
    float mx[2] = {-INFINITY, -INFINITY};
    if (blk) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int b = u * PAGE_TOKENS + n * 8 + t * 2 + (j & 1);
          const bool ok = b < ((j < 2) ? nb_a : nb_b);
          const float v = ok ? bent(sc[n][j]) : -INFINITY;
          sc[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
    } else if (window <= 0 && (!EXTRA || opt.block <= 0) &&
               j0 + PAGE_TOKENS - 1 <= pos0 + q0 + warp * 16) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = EXTRA ? bent(sc[n][j]) : sc[n][j] * sl2;
          sc[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = j0 + n * 8 + t * 2 + (j & 1);
          const int qp = (j < 2) ? qpos_a : qpos_b;
          const bool ok = EXTRA ? (key <= qp && (key >= opt.first_key(qp) || key < keep_first))
                                : (key <= qp && (window <= 0 || key > qp - window));
          const float v = ok ? (EXTRA ? bent(sc[n][j]) : sc[n][j] * sl2) : -INFINITY;
          sc[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
    }
    float m_use[2], resc[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.0f : m_new;
      resc[r] = (m_run[r] == -INFINITY) ? 0.0f : nb_exp2(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= resc[r];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= resc[0]; o[n][1] *= resc[0];
      o[n][2] *= resc[1]; o[n][3] *= resc[1];
    }
    // probabilities (fp32), their row sums, and their bf16 form as the next A operand
    uint32_t pf[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = nb_exp2(sc[n][0] - m_use[0]), p1 = nb_exp2(sc[n][1] - m_use[0]);
      const float p2 = nb_exp2(sc[n][2] - m_use[1]), p3 = nb_exp2(sc[n][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // o += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {       // 16 keys per step
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {   // two value tiles of 8 columns per ldmatrix.x4
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + n2 * 16 +
                                  (lane >> 4) * 8);
        mma_bf16(o[2 * n2], pf[kk], vb[0], vb[1]);
        mma_bf16(o[2 * n2 + 1], pf[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();   // the stage may be refilled
  }

  // row sums across the four lanes of a row, then the result
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (EXTRA && sink != nullptr) {
    const float s2 = sink[h] * 1.4426950408889634f;   // like the scores, in units of log2(e)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float m_f = fmaxf(m_run[r], s2);
      const float fix = (m_run[r] == -INFINITY) ? 0.0f : nb_exp2(m_run[r] - m_f);
      l_run[r] = l_run[r] * fix + nb_exp2(s2 - m_f);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][2 * r] *= fix;
        o[n][2 * r + 1] *= fix;
      }
    }
  }
  const float inv_a = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f;
  const float inv_b = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
  const int ra = warp * 16 + g, rb = ra + 8;
  // the gate of this head, where the row's sum divides its result
  const float gi_a = (EXTRA && ra < rows_here) ? inv_a * opt.gate_of(row0 + q0 + ra, h) : inv_a;
  const float gi_b = (EXTRA && rb < rows_here) ? inv_b * opt.gate_of(row0 + q0 + rb, h) : inv_b;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int col = h * HD + n * 8 + t * 2;
    if (ra < rows_here) {
      TOut* dst = out + (size_t)(row0 + q0 + ra) * out_stride + col;
      dst[0] = nb_from_f32<TOut>(o[n][0] * gi_a);
      dst[1] = nb_from_f32<TOut>(o[n][1] * gi_a);
    }
    if (rb < rows_here) {
      TOut* dst = out + (size_t)(row0 + q0 + rb) * out_stride + col;
      dst[0] = nb_from_f32<TOut>(o[n][2] * gi_b);
      dst[1] = nb_from_f32<TOut>(o[n][3] * gi_b);
    }
  }
}

template <int HD, typename TOut, bool EXTRA = false>
int launch(const void* q, int q_stride, int q_col, const int* cu_rows, const int* seq_slot,
           const int* seq_pos0, const NbPagedKV& kv, int n_heads, void* out, int out_stride,
           float scale, int window, int n_seqs, int max_q_len, cudaStream_t stream,
           const NbPagedKV& blocks = NbPagedKV{}, int pool = 0, const float* sink = nullptr,
           const NbAttnOpts* options = nullptr, float softcap = 0.0f) {
  const NbAttnOpts opt = options ? *options : NbAttnOpts{window, 0, 0, nullptr, 0, 0};
  constexpr int ROW = HD + 8;
  const size_t smem = (size_t)(BLOCK_Q + 4 * PAGE_TOKENS) * ROW * sizeof(bf16);
  auto kern = attention_prefill_kernel<HD, TOut, EXTRA>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((max_q_len + BLOCK_Q - 1) / BLOCK_Q, n_heads, n_seqs);
  kern<<<grid, THREADS, smem, stream>>>((const bf16*)q, q_stride, q_col, cu_rows, seq_slot,
                                        seq_pos0, kv, n_heads / kv.n_kv_heads, (TOut*)out,
                                        out_stride, scale, window, blocks, pool, sink, opt, softcap);
  return 0;
}

}  // namespace

NB_EXPORT int nb_attention_prefill_supported(int dtype, int head_dim, int n_heads, int n_kv_heads,
                                             int page, int q_stride, int q_col) {
  if (dtype != NB_BF16 || page != PAGE_TOKENS) return 0;
  if (n_kv_heads < 1 || n_heads % n_kv_heads != 0) return 0;
  if (q_stride % 8 != 0 || q_col % 8 != 0) return 0;   // 16-byte query loads
  return head_dim == 16 || head_dim == 32 || head_dim == 48 || head_dim == 64 ||
         head_dim == 96 || head_dim == 128;
}

// Rows of sequence s are cu_rows[s]..cu_rows[s+1] of the packed batch, at positions
// seq_pos0[s].. of slot seq_slot[s]; their keys and values are already in the cache.
NB_EXPORT int nb_attention_prefill(const void* q, int dtype, int q_stride, int q_col,
                                   const int* cu_rows, const int* seq_slot, const int* seq_pos0,
                                   const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_pages, int page, int n_heads,
                                   int n_kv_heads, int head_dim, void* out, int out_dtype,
                                   int out_stride, float scale, int window, int n_seqs,
                                   int max_q_len, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_supported(dtype, head_dim, n_heads, n_kv_heads, page, q_stride, q_col),
             NB_ERR_UNSUPPORTED,
             "attention_prefill: unsupported shape (head size %d, %d/%d heads, row pitch %d)",
             head_dim, n_heads, n_kv_heads, q_stride);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, NB_ERR_UNSUPPORTED,
             "attention_prefill: grid too large");
  NB_REQUIRE((uintptr_t)q % 16 == 0, NB_ERR_UNSUPPORTED, "attention_prefill: unaligned queries");
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  int rc = NB_ERR_UNSUPPORTED;
#define NB_HD(HD_)                                                                             \
  case HD_:                                                                                    \
    rc = out_dtype == NB_F32                                                                   \
             ? launch<HD_, float>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream) \
             : launch<HD_, bf16>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream); \
    break;
  switch (head_dim) {
    NB_HD(16) NB_HD(32) NB_HD(48) NB_HD(64) NB_HD(96) NB_HD(128)
  }
#undef NB_HD
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_prefill");
  return 0;
}

// The same walk with pooled blocks before the window and a sink (see EXTRA above).  bk, bv,
// b_table: the paged store of blocks (null: none); sink: fp32 [n_heads] or null.  Steps of one
// row per sequence run it too (a tile with one row).
NB_EXPORT int nb_attention_pooled_mma(const void* q, int q_stride, int q_col, const int* cu_rows,
                                      const int* seq_slot, const int* seq_pos0, const void* k_cache,
                                      const void* v_cache, const int* block_table, int max_pages,
                                      const void* bk, const void* bv, const int* b_table,
                                      int b_max_pages, int page, int n_heads, int n_kv_heads,
                                      int head_dim, const float* sink, void* out, int out_dtype,
                                      int out_stride, float scale, int window, int pool, int n_seqs,
                                      int max_q_len, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_supported(NB_BF16, head_dim, n_heads, n_kv_heads, page, q_stride, q_col),
             NB_ERR_UNSUPPORTED,
             "attention_pooled_mma: unsupported shape (head size %d, %d/%d heads, row pitch %d)",
             head_dim, n_heads, n_kv_heads, q_stride);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, NB_ERR_UNSUPPORTED,
             "attention_pooled_mma: grid too large");
  NB_REQUIRE((uintptr_t)q % 16 == 0 && window >= 0 && pool >= 0, NB_ERR_UNSUPPORTED,
             "attention_pooled_mma: unaligned queries or a negative window");
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  NbPagedKV blocks{(void*)bk, (void*)bv, b_table, b_max_pages, page, n_kv_heads, head_dim};
  int rc = NB_ERR_UNSUPPORTED;
#define NB_HD(HD_)                                                                             \
  case HD_:                                                                                    \
    rc = out_dtype == NB_F32                                                                   \
             ? launch<HD_, float, true>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream, blocks, pool, sink) \
             : launch<HD_, bf16, true>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream, blocks, pool, sink); \
    break;
  switch (head_dim) {
    NB_HD(16) NB_HD(32) NB_HD(48) NB_HD(64) NB_HD(96) NB_HD(128)
  }
#undef NB_HD
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_pooled_mma");
  return 0;
}

// The same walk under the options of NbAttnOpts (window + kept first tokens, or blocks of
// positions; a gate per head: fp32 rows with a logit per head at columns gate_col ..), capped
// scores (softcap > 0) and a sink (fp32 [n_heads] or null): bfloat16 prompts whose heads the
// tcgen05 kernel does not take.
NB_EXPORT int nb_attention_prefill_masked(const void* q, int q_stride, int q_col, const int* cu_rows,
                                          const int* seq_slot, const int* seq_pos0, const void* kc,
                                          const void* vc, const int* block_table, int max_pages,
                                          int page, int n_heads, int n_kv_heads, int head_dim,
                                          const float* sink, void* out, int out_dtype, int out_stride,
                                          float scale, float softcap, int window, int keep_first,
                                          int mask_block, const float* gate, int gate_stride,
                                          int gate_col, int n_seqs, int max_q_len,
                                          cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_supported(NB_BF16, head_dim, n_heads, n_kv_heads, page, q_stride, q_col),
             NB_ERR_UNSUPPORTED,
             "attention_prefill_masked: unsupported shape (head size %d, %d/%d heads, row pitch %d)",
             head_dim, n_heads, n_kv_heads, q_stride);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, NB_ERR_UNSUPPORTED,
             "attention_prefill_masked: grid too large");
  NB_REQUIRE((uintptr_t)q % 16 == 0 && window >= 0 && keep_first >= 0 && mask_block >= 0 &&
                 !(window > 0 && mask_block > 0) && softcap >= 0.0f,
             NB_ERR_BAD_ARG, "attention_prefill_masked: unaligned queries or a bad mask");
  NbPagedKV kv{(void*)kc, (void*)vc, block_table, max_pages, page, n_kv_heads, head_dim};
  const NbAttnOpts opt{window, keep_first, mask_block, gate, gate_stride, gate_col};
  int rc = NB_ERR_UNSUPPORTED;
#define NB_CASE(HD_)                                                                                   \
  case HD_:                                                                                            \
    rc = out_dtype == NB_F32                                                                           \
             ? launch<HD_, float, true>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream, NbPagedKV{}, 0, sink, &opt, softcap) \
             : launch<HD_, bf16, true>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream, NbPagedKV{}, 0, sink, &opt, softcap); \
    break;
  switch (head_dim) {
    NB_CASE(16) NB_CASE(32) NB_CASE(48) NB_CASE(64) NB_CASE(96) NB_CASE(128)
    default: break;
  }
#undef NB_CASE
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_prefill_masked");
  return 0;
}
