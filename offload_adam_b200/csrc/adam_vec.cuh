// Vector building blocks of the fused Adam step kernels: operand pointers, the
// 16-element load / update / store helpers and the scalar tail path.  Shared by the
// plain step kernel (adam_step.cu) and the kernels that re-quantize the updated
// fp32 master in the same pass (adam_quant.cu).
//
// A thread owns groups of 16 consecutive elements.  Every operand moves with
// Blackwell's 256-bit global loads/stores (one 32-byte request per bf16 stream, two
// for the fp32 master), all issued before the first use.
#pragma once
#include "adam_math.cuh"
#include "adam_step.h"

namespace oab {
namespace vec {

constexpr int kThreads = 256;
constexpr int kVec = 16;  // elements per thread per iteration (one 32-byte bf16 vector)

struct Ptrs {
  uint16_t* p;
  const uint16_t* g;
  const uint16_t* g2;
  uint16_t* m;
  uint16_t* v;
  void* extra;
  void* extra_copy;  // fp32_master only: optional second destination of the updated master
};

// Peer-mapped replicas for the fused reduce-scatter / all-gather variant.
struct Peers {
  const uint16_t* g[kMaxPeers];
  uint16_t* p[kMaxPeers];
  int n_g;
  int n_p;
  float g_scale;
};

// bf16(scale * (a + b + ...)) of two packed bf16 pairs, fp32 accumulation
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// 16 gradient values = average of the same 16 values on every rank
__device__ __forceinline__ V8 pull_reduce_vec(const Peers& pr, int64_t e) {
  V8 in[kMaxPeers];
#pragma unroll
  for (int j = 0; j < kMaxPeers; ++j)
    if (j < pr.n_g) in[j] = ld32_peer(pr.g[j] + e);
  V8 out;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPeers; ++j)
      if (j < pr.n_g) {
        float2 f = unpack2(in[j].w[w]);
        lo = __fadd_rn(lo, f.x);
        hi = __fadd_rn(hi, f.y);
      }
    out.w[w] = f32_to_bf16_rne_bits(__fmul_rn(lo, pr.g_scale)) |
               (f32_to_bf16_rne_bits(__fmul_rn(hi, pr.g_scale)) << 16);
  }
  return out;
}
__device__ __forceinline__ uint32_t pull_reduce_one(const Peers& pr, int64_t i) {
  float s = 0.f;
  for (int j = 0; j < pr.n_g; ++j) s = __fadd_rn(s, bf16_bits_to_f32(pr.g[j][i]));
  return f32_to_bf16_rne_bits(__fmul_rn(s, pr.g_scale));
}

template <int MODE>
struct VecRegs {
  V8 p, g, g2, m, v, e0, e1;
};

template <int MODE, bool HAS_G2, bool PEERS>
__device__ __forceinline__ void load_vec(VecRegs<MODE>& r, const Ptrs& t, const Peers& pr, int64_t vec) {
  const int64_t e = vec * kVec;
  if (MODE != kModeFP32Master) r.p = ld32(t.p + e);  // params stay cacheable (forward re-reads)
  if (PEERS && pr.n_g > 0) r.g = pull_reduce_vec(pr, e);  // gradient pulled from all replicas
  else r.g = ld32_stream(t.g + e);
  if (HAS_G2 && !PEERS) r.g2 = ld32_stream(t.g2 + e);
  r.m = ld32_stream(t.m + e);
  r.v = ld32_stream(t.v + e);
  if (MODE == kModeFP32Master) {
    const float* mp = reinterpret_cast<const float*>(t.extra) + e;
    r.e0 = ld32_stream(mp);
    r.e1 = ld32_stream(mp + 8);
  } else if (MODE == kModeFP31 || MODE == kModeCustom) {
    r.e0 = ld32_stream(reinterpret_cast<const int16_t*>(t.extra) + e);
  }
}

// One element: `p` is the full-precision parameter on entry and on exit, m and v the
// moments (fp32 values of their bf16 storage on entry, unrounded on exit).
template <bool DECOUPLED>
__device__ __forceinline__ void element_math(float& p, uint32_t g16, bool has_g2, uint32_t g2_16,
                                             float& m, float& v, float clip, const AdamScalars& s) {
  float g = bf16_bits_to_f32(g16);
  if (has_g2) {
    g = bf16_bits_to_f32(f32_to_bf16_rne_bits(__fadd_rn(g, bf16_bits_to_f32(g2_16))));
  }
  g = __fmul_rn(g, clip);
  adam_math<DECOUPLED>(p, g, m, v, s);
}

// One element from and to its stored form (scalar tail path and multi-tensor kernel).
template <int MODE, bool DECOUPLED>
__device__ __forceinline__ float element_step(uint32_t& p16, uint32_t g16, bool has_g2,
                                              uint32_t g2_16, uint32_t& m16, uint32_t& v16,
                                              float& master, int16_t& err, float clip,
                                              const AdamScalars& s, uint32_t rand16) {
  float m = bf16_bits_to_f32(m16);
  float v = bf16_bits_to_f32(v16);
  float p;
  if (MODE == kModeSR) p = bf16_bits_to_f32(p16);
  else if (MODE == kModeFP32Master) p = master;
  else if (MODE == kModeFP31) p = fp31_reconstruct(p16, err);
  else p = custom_reconstruct(p16, err);

  element_math<DECOUPLED>(p, g16, has_g2, g2_16, m, v, clip, s);

  m16 = f32_to_bf16_rne_bits(m);
  v16 = f32_to_bf16_rne_bits(v);
  if (MODE == kModeSR) {
    p16 = f32_to_bf16_sr_bits(p, rand16);
  } else if (MODE == kModeFP32Master) {
    master = p;
    p16 = f32_to_bf16_rne_bits(p);
  } else if (MODE == kModeFP31) {
    fp31_decompose(p, p16, err);
  } else {
    custom_decompose(p, p16, err);
  }
  return p;
}

// Updates the 16 elements held in `r` in place: r.p receives the new bf16 parameter
// (for fp32_master: bf16(master)), r.m / r.v the new moments, r.e0 / r.e1 the new
// master (fp32_master) or rounding error.  Returns max |updated fp32 value| when AMAX.
// Elements are handled in pairs, one 32-bit word of each bf16 stream at a time, so that
// the roundings to bf16 are one hardware convert per pair and no half-word is masked in.
template <int MODE, bool DECOUPLED, bool HAS_G2, bool AMAX>
__device__ __forceinline__ float compute_vec(VecRegs<MODE>& r, int64_t vec, float clip,
                                             const AdamScalars& s, uint64_t seed, int64_t elem_offset) {
  const int64_t e = vec * kVec;
  Philox4 rnd;
  float amax = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    // one Philox block serves eight elements; it is drawn when its first element comes
    // up, so that only one block is alive at a time
    if (MODE == kModeSR && (w & 3) == 0) rnd = philox4x32_10((uint64_t)((elem_offset + e) >> 3) + (w >> 2), seed);
    const uint32_t gw = r.g.w[w], g2w = HAS_G2 ? r.g2.w[w] : 0u;
    const uint32_t pw = (MODE != kModeFP32Master) ? r.p.w[w] : 0u;
    float m[2] = {__uint_as_float(r.m.w[w] << 16), __uint_as_float(r.m.w[w] & 0xffff0000u)};
    float v[2] = {__uint_as_float(r.v.w[w] << 16), __uint_as_float(r.v.w[w] & 0xffff0000u)};
    float p[2];
    uint32_t p16[2];
    int16_t err[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 2 * w + h;
      const uint32_t pin = (pw >> (16 * h)) & 0xffffu;
      if (MODE == kModeFP31 || MODE == kModeCustom) err[h] = (int16_t)half_of(r.e0, j);
      if (MODE == kModeSR) p[h] = bf16_bits_to_f32(pin);
      else if (MODE == kModeFP32Master) p[h] = __uint_as_float(j < 8 ? r.e0.w[j & 7] : r.e1.w[j & 7]);
      else if (MODE == kModeFP31) p[h] = fp31_reconstruct(pin, err[h]);
      else p[h] = custom_reconstruct(pin, err[h]);
      element_math<DECOUPLED>(p[h], (gw >> (16 * h)) & 0xffffu, HAS_G2, (g2w >> (16 * h)) & 0xffffu,
                              m[h], v[h], clip, s);
      if (AMAX) amax = fmaxf(amax, fabsf(p[h]));
      if (MODE == kModeSR) {
        p16[h] = f32_to_bf16_sr_bits(p[h], philox_word16(rnd, j & 7));
      } else if (MODE == kModeFP32Master) {
        if (j < 8) r.e0.w[j & 7] = __float_as_uint(p[h]); else r.e1.w[j & 7] = __float_as_uint(p[h]);
      } else if (MODE == kModeFP31) {
        fp31_decompose(p[h], p16[h], err[h]);
      } else {
        custom_decompose(p[h], p16[h], err[h]);
      }
    }
    r.m.w[w] = f32x2_to_bf16x2_rne(m[0], m[1]);
    r.v.w[w] = f32x2_to_bf16x2_rne(v[0], v[1]);
    if (MODE == kModeFP32Master) r.p.w[w] = f32x2_to_bf16x2_rne(p[0], p[1]);
    else r.p.w[w] = (p16[0] & 0xffffu) | (p16[1] << 16);
    if (MODE == kModeFP31 || MODE == kModeCustom)
      r.e0.w[w] = (uint32_t)(uint16_t)err[0] | ((uint32_t)(uint16_t)err[1] << 16);
  }
  return amax;
}

// Stores what compute_vec left in `r`.  WRITE_P = false skips the bf16 parameter (the
// caller re-quantizes the master instead).
template <int MODE, bool PEERS, bool WRITE_P = true>
__device__ __forceinline__ void store_vec(const VecRegs<MODE>& r, const Ptrs& t, const Peers& pr, int64_t vec) {
  const int64_t e = vec * kVec;
  if (WRITE_P) {
    if (PEERS && pr.n_p > 0) {
      // push the new rows into every replica (all-gather folded into the update)
#pragma unroll
      for (int j = 0; j < kMaxPeers; ++j)
        if (j < pr.n_p) st32(pr.p[j] + e, r.p);
    } else if (t.p != nullptr) {
      st32(t.p + e, r.p);
    }
  }
  st32_stream(t.m + e, r.m);
  st32_stream(t.v + e, r.v);
  if (MODE == kModeFP32Master) {
    float* mp = reinterpret_cast<float*>(t.extra) + e;
    st32_stream(mp, r.e0);
    st32_stream(mp + 8, r.e1);
    if (t.extra_copy != nullptr) {  // second home of the updated master (kept on the device)
      float* cp = reinterpret_cast<float*>(t.extra_copy) + e;
      st32(cp, r.e0);
      st32(cp + 8, r.e1);
    }
  } else if (MODE == kModeFP31 || MODE == kModeCustom) {
    st32_stream(reinterpret_cast<int16_t*>(t.extra) + e, r.e0);
  }
}

// Scalar path: tails and tensors whose pointers are not 32-byte aligned.
template <int MODE, bool DECOUPLED, bool PEERS = false>
__device__ __forceinline__ float scalar_element(const Ptrs& t, int64_t i, bool has_g2, float clip,
                                                const AdamScalars& s, uint64_t seed,
                                                int64_t elem_offset, const Peers* pr = nullptr) {
  uint32_t p16 = (MODE != kModeFP32Master) ? t.p[i] : 0u;
  uint32_t m16 = t.m[i], v16 = t.v[i];
  float master = 0.f;
  int16_t err = 0;
  if (MODE == kModeFP32Master) master = reinterpret_cast<float*>(t.extra)[i];
  if (MODE == kModeFP31 || MODE == kModeCustom) err = reinterpret_cast<int16_t*>(t.extra)[i];
  uint32_t rand16 = 0;
  if (MODE == kModeSR) {
    int64_t G = elem_offset + i;
    Philox4 rnd = philox4x32_10((uint64_t)(G >> 3), seed);
    rand16 = philox_word16(rnd, (int)(G & 7));
  }
  const uint32_t g16 = (PEERS && pr->n_g > 0) ? pull_reduce_one(*pr, i) : (uint32_t)t.g[i];
  float pf = element_step<MODE, DECOUPLED>(p16, g16, has_g2 && !PEERS, (has_g2 && !PEERS) ? t.g2[i] : 0u,
                                           m16, v16, master, err, clip, s, rand16);
  if (PEERS && pr->n_p > 0) {
    for (int j = 0; j < pr->n_p; ++j) pr->p[j][i] = (uint16_t)p16;
  } else if (t.p != nullptr) {
    t.p[i] = (uint16_t)p16;
  }
  t.m[i] = (uint16_t)m16;
  t.v[i] = (uint16_t)v16;
  if (MODE == kModeFP32Master) {
    reinterpret_cast<float*>(t.extra)[i] = master;
    if (t.extra_copy != nullptr) reinterpret_cast<float*>(t.extra_copy)[i] = master;
  }
  if (MODE == kModeFP31 || MODE == kModeCustom) reinterpret_cast<int16_t*>(t.extra)[i] = err;
  return fabsf(pf);
}

}  // namespace vec
}  // namespace oab
