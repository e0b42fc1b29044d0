// Per-element Adam/AdamW arithmetic and the four parameter-precision schemes.
//
// The formulas restate what the reference optimizer's four step kernels compute
// (reference: src/offload_adam/kernels/stochastic_rounding.py:56-79,
// fp32_master.py:40-59, fp31_master.py:26-54, fp32_master_custom_rounding.py:33-54):
//
//   decoupled:  p -= (lr*wd) * p          else:  g += wd * p
//   m += (1-b1h) * (g - m)
//   v += (1-b2h) * (g*g - v)
//   p -= (lr*m) / (sqrt(v) + eps)
//
// where b1h/b2h are the bias-correction-folded EMA coefficients computed on the
// host.  Every operation is an explicitly rounded fp32 op (no FMA contraction).
#pragma once
#include "adam_step.h"
#include "common.cuh"

namespace oab {

struct AdamScalars {
  float lr;
  float wd;
  float lr_wd;      // fp32(lr) * fp32(wd)
  float one_m_b1h;  // 1 - beta1_hat (fp32)
  float one_m_b2h;  // 1 - beta2_hat (fp32)
  float eps;
};

template <bool DECOUPLED>
__device__ __forceinline__ void adam_math(float& p, float g, float& m, float& v,
                                          const AdamScalars& s) {
  if (DECOUPLED) {
    p = __fsub_rn(p, __fmul_rn(s.lr_wd, p));
  } else {
    g = __fadd_rn(g, __fmul_rn(s.wd, p));
  }
  m = __fadd_rn(m, __fmul_rn(s.one_m_b1h, __fsub_rn(g, m)));
  v = __fadd_rn(v, __fmul_rn(s.one_m_b2h, __fsub_rn(__fmul_rn(g, g), v)));
  float denom = __fadd_rn(__fsqrt_rn(v), s.eps);
  p = __fsub_rn(p, __fdiv_rn(__fmul_rn(s.lr, m), denom));
}

// --- fp31: drop the fp32 LSB with round-half-to-even, split into bf16 + int16 ---
__device__ __forceinline__ uint32_t round_to_fp31_bits(uint32_t x) {
  uint32_t up = (x & 1u) & ((x >> 1) & 1u);
  return (x & ~1u) + (up << 1);
}
__device__ __forceinline__ float fp31_reconstruct(uint32_t p_bf16, int16_t err) {
  uint32_t xq = p_bf16 << 16;
  return __uint_as_float(xq + ((uint32_t)(int32_t)err << 1));
}
__device__ __forceinline__ void fp31_decompose(float x, uint32_t& p_bf16, int16_t& err) {
  uint32_t xb = round_to_fp31_bits(__float_as_uint(x));
  p_bf16 = f32_to_bf16_rne_bits(__uint_as_float(xb));
  int32_t e = (int32_t)(xb - (p_bf16 << 16));
  err = (int16_t)(e >> 1);
}

// --- custom rounding: bf16 = (bits + 0x8000) >> 16, error fits int16 exactly ---
__device__ __forceinline__ float custom_reconstruct(uint32_t p_bf16, int16_t err) {
  return __uint_as_float((p_bf16 << 16) + (uint32_t)(int32_t)err);
}
__device__ __forceinline__ void custom_decompose(float x, uint32_t& p_bf16, int16_t& err) {
  uint32_t xb = __float_as_uint(x);
  p_bf16 = ((xb + 0x8000u) >> 16) & 0xffffu;
  err = (int16_t)(xb - (p_bf16 << 16));
}

// 16-bit random word for global element index G (see Philox note in common.cuh)
__device__ __forceinline__ uint32_t philox_word16(const Philox4& r, int j) {
  uint32_t w = (j < 2) ? r.x : (j < 4) ? r.y : (j < 6) ? r.z : r.w;
  return (w >> (16 * (j & 1))) & 0xffffu;
}

}  // namespace oab
