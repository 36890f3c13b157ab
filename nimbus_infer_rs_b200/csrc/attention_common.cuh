// Small helpers shared by the attention kernels: 16-byte asynchronous copies into shared
// memory and the 16 bytes a lane reads, widened to floats.
#pragma once

#include "common.cuh"

namespace {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// 2^x by the hardware unit (one instruction; relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float nb_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// softcap * tanh(raw * cap_in), with tanh(t) = 1 - 2 / (1 + e^(2t)) on the hardware's exponential
// and reciprocal: the absolute error is about 2e-7 * softcap for every t (the ends give -1 and 1).
__device__ __forceinline__ float nb_softcap(float raw, float cap_in, float softcap) {
  const float e = nb_exp2(raw * cap_in * 2.8853900817779268f);
  return softcap * (1.0f - __fdividef(2.0f, 1.0f + e));
}

// The softmax's last step when its denominator has one more term exp(sink) without key or
// value: sum `l` and weighted values `a` are in units of exp(m) (base 2 when `base2`); returns
// the factor for `a` after adding the term to `l`.
__device__ __forceinline__ float nb_sink_fix(float& l, float m, float sink_logit, bool base2) {
  const float sk = base2 ? sink_logit * 1.4426950408889634f : sink_logit;
  const float m_f = fmaxf(m, sk);
  const float fix = (m == -INFINITY) ? 0.0f : (base2 ? nb_exp2(m - m_f) : expf(m - m_f));
  l = fmaf(l, fix, base2 ? nb_exp2(sk - m_f) : expf(sk - m_f));
  return fix;
}

// Options of the masked attention kernels.  What a query at position `pos` sees among the keys
// j <= pos:
//   window > 0:     j > pos - window, and besides those every j < keep_first (the sequence's
//                   first tokens stay visible)
//   block > 0:      j >= floor(pos / block) * block (only its own block of positions)
//   neither:        every j
//
// gate (or null): fp32 rows with one logit per head at columns gate_col ..; head h's result of row
// r is multiplied by sigmoid(gate[r * gate_stride + gate_col + h]) where the row's sum divides it.
struct NbAttnOpts {
  int window;
  int keep_first;
  int block;
  const float* gate;
  int gate_stride;
  int gate_col;
  // the first key of the contiguous run that ends at `pos`
  __host__ __device__ __forceinline__ int first_key(int pos) const {
    if (block > 0) return (pos / block) * block;
    return (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  }
  // whether the kept first tokens are a range of their own
  __host__ __device__ __forceinline__ bool keeps() const { return window > 0 && keep_first > 0; }
  // the factor of head `head` of row `r`
  __device__ __forceinline__ float gate_of(int r, int head) const {
    return gate == nullptr ? 1.0f
                           : 1.0f / (1.0f + expf(-gate[(size_t)r * gate_stride + gate_col + head]));
  }
};

template <typename T>
struct Lane16;   // the 16 bytes a lane reads, as floats
template <>
struct Lane16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  }
  __device__ static void unpack(const uint4& u, float (&v)[4]) {
    v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y);
    v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
  }
};
template <>
struct Lane16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    unpack(*reinterpret_cast<const uint4*>(p), v);
  }
  __device__ static void unpack(const uint4& u, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __bfloat162float(h[i].x);
      v[2 * i + 1] = __bfloat162float(h[i].y);
    }
  }
};


}  // namespace
