// Device helpers shared by the weight-only quantization kernels (quant.cu) and the
// optimizer kernels that re-quantize the updated fp32 master in the same pass
// (adam_quant.cu): typed 16-element loads/stores, block statistics, the E2M1 / e4m3
// conversions and, per format, "16 fp32 values -> packed words" and back.
//
// Rounding rules (pinned by the checkpoint formats): every reciprocal is correctly
// rounded (rcp.rn) and then multiplied, integers round half to even, NF4 picks the
// nearest codebook entry with the lowest index winning ties, E2M1 rounds to nearest
// even and saturates, -0 keeps its sign bit.
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace oab {
namespace qm {

constexpr float kEps = 1e-12f;

// ------------------------------------------------------------------ element I/O
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ void load16(const float* p, float (&x)[16]) {
    V8 a = ld32_stream(p), b = ld32_stream(p + 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) { x[i] = __uint_as_float(a.w[i]); x[8 + i] = __uint_as_float(b.w[i]); }
  }
  static __device__ __forceinline__ void store16(float* p, const float (&x)[16]) {
    V8 a, b;
#pragma unroll
    for (int i = 0; i < 8; ++i) { a.w[i] = __float_as_uint(x[i]); b.w[i] = __float_as_uint(x[8 + i]); }
    st32_stream(p, a); st32_stream(p + 8, b);
  }
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&x)[16]) {
    V8 a = ld32_stream(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) { x[2 * i] = __uint_as_float(a.w[i] << 16); x[2 * i + 1] = __uint_as_float(a.w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&x)[16]) {
    V8 a;
#pragma unroll
    for (int i = 0; i < 8; ++i) a.w[i] = f32x2_to_bf16x2_rne(x[2 * i], x[2 * i + 1]);
    st32_stream(p, a);
  }
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ void load16(const __half* p, float (&x)[16]) {
    V8 a = ld32_stream(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __half2 h = *reinterpret_cast<__half2*>(&a.w[i]);
      float2 f = __half22float2(h);
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store16(__half* p, const float (&x)[16]) {
    V8 a;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __half2 h = __halves2half2(__float2half_rn(x[2 * i]), __float2half_rn(x[2 * i + 1]));
      a.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st32_stream(p, a);
  }
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ float amax16(const float (&x)[16]) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(x[i]));
  return m;
}
// max over groups of `lanes` consecutive lanes (power of two)
__device__ __forceinline__ float group_max(float v, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float rcp_rn(float x) { return __frcp_rn(x); }

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
// two fp32 -> one byte of E2M1 codes (lo in the low nibble), RNE, saturating
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n cvt.u32.u8 %0, t;\n}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// one byte of E2M1 codes -> two fp32 (low nibble first)
__device__ __forceinline__ float2 e2m1x2_to_f32(uint32_t byte) {
  uint32_t r;
  asm("{\n .reg .b8 t;\n cvt.u8.u32 t, %1;\n cvt.rn.f16x2.e2m1x2 %0, t;\n}" : "=r"(r) : "r"(byte));
  __half2 h = *reinterpret_cast<__half2*>(&r);
  return __half22float2(h);
}

// ------------------------------------------------------------------------- NF4
static __constant__ float kNF4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// Index of the nearest codebook entry; among equal distances the lowest index wins (the
// rule of a sequential scan over the 16 entries with a strict '<' on
// |fl(x - entry)|).  For neighbouring entries i, i + 1 the outcome "i + 1 is strictly
// closer" is monotone in x, so it is decided by one threshold: kNF4Threshold[i] is the
// smallest fp32 x for which |fl(x - entry[i+1])| < |fl(x - entry[i])|, found by bisection
// over the fp32 values between the two entries (tests/test_qweight_formats.py recomputes
// the table from the codebook).  The index is the number of thresholds <= x: a four-step
// binary search over constants, no table look-ups.
#define OAB_NF4_THRESHOLD_BITS                                                                      \
  0xbf591cd8u, 0xbf1c5270u, 0xbeeb847fu, 0xbeadea76u, 0xbe703cecu, 0xbe0d38bbu, 0xbd3a7870u,        \
  0x3d22fb00u, 0x3df64863u, 0x3e5067e1u, 0x3e9582d5u, 0x3ec753fau, 0x3f006d04u, 0x3f248db0u, 0x3f5c89dau
__device__ __forceinline__ int nf4_nearest(float x, const float* /*lut*/) {
  constexpr uint32_t B[15] = {OAB_NF4_THRESHOLD_BITS};
#define OAB_T(i) __uint_as_float(B[i])
  const bool c3 = x >= OAB_T(7);
  const bool c2 = x >= (c3 ? OAB_T(11) : OAB_T(3));
  const float t1 = c3 ? (c2 ? OAB_T(13) : OAB_T(9)) : (c2 ? OAB_T(5) : OAB_T(1));
  const bool c1 = x >= t1;
  const float t0 = c3 ? (c2 ? (c1 ? OAB_T(14) : OAB_T(12)) : (c1 ? OAB_T(10) : OAB_T(8)))
                      : (c2 ? (c1 ? OAB_T(6) : OAB_T(4)) : (c1 ? OAB_T(2) : OAB_T(0)));
  const bool c0 = x >= t0;
#undef OAB_T
  return (c3 ? 8 : 0) | (c2 ? 4 : 0) | (c1 ? 2 : 0) | (c0 ? 1 : 0);
}

// ---------------------------------------------------------------- 16-value packers
// NVFP4: e4m3 block scale + two words of E2M1 codes (even element in the low nibble).
__device__ __forceinline__ void nvfp4_pack16(const float (&e)[16], float global, float inv_global,
                                             uint8_t& s8, uint32_t& w0, uint32_t& w1) {
  const float bamax = fmaxf(amax16(e), kEps);
  s8 = f32_to_e4m3(__fmul_rn(__fdiv_rn(bamax, 6.0f), inv_global));
  const float eff = __fmul_rn(e4m3_to_f32(s8), global);
  const float inv_eff = rcp_rn(fmaxf(eff, kEps));
  w0 = 0; w1 = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w0 |= e2m1x2(__fmul_rn(e[2 * i], inv_eff), __fmul_rn(e[2 * i + 1], inv_eff)) << (8 * i);
    w1 |= e2m1x2(__fmul_rn(e[8 + 2 * i], inv_eff), __fmul_rn(e[9 + 2 * i], inv_eff)) << (8 * i);
  }
}
__device__ __forceinline__ void nvfp4_unpack16(uint32_t w0, uint32_t w1, float eff, float (&e)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a = e2m1x2_to_f32((w0 >> (8 * i)) & 0xffu);
    float2 c = e2m1x2_to_f32((w1 >> (8 * i)) & 0xffu);
    e[2 * i] = __fmul_rn(a.x, eff); e[2 * i + 1] = __fmul_rn(a.y, eff);
    e[8 + 2 * i] = __fmul_rn(c.x, eff); e[9 + 2 * i] = __fmul_rn(c.y, eff);
  }
}
// NVFP4 tensor scale from max|x| of the whole weight
__device__ __forceinline__ void nvfp4_global(float tensor_amax, float& global, float& inv_global) {
  global = __fdiv_rn(fmaxf(tensor_amax, kEps), 448.0f * 6.0f);
  inv_global = rcp_rn(fmaxf(global, kEps));
}

// NF4: two words of codebook indices (even element in the HIGH nibble)
__device__ __forceinline__ void nf4_pack16(const float (&e)[16], float inv, const float* lut,
                                           uint32_t& w0, uint32_t& w1) {
  w0 = 0; w1 = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t b0 = (nf4_nearest(__fmul_rn(e[2 * i], inv), lut) << 4) | nf4_nearest(__fmul_rn(e[2 * i + 1], inv), lut);
    uint32_t b1 = (nf4_nearest(__fmul_rn(e[8 + 2 * i], inv), lut) << 4) | nf4_nearest(__fmul_rn(e[9 + 2 * i], inv), lut);
    w0 |= b0 << (8 * i);
    w1 |= b1 << (8 * i);
  }
}
__device__ __forceinline__ void nf4_unpack16(uint32_t w0, uint32_t w1, float am, const float* lut, float (&e)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t b0 = (w0 >> (8 * i)) & 0xffu, b1 = (w1 >> (8 * i)) & 0xffu;
    e[2 * i] = __fmul_rn(lut[b0 >> 4], am); e[2 * i + 1] = __fmul_rn(lut[b0 & 15], am);
    e[8 + 2 * i] = __fmul_rn(lut[b1 >> 4], am); e[9 + 2 * i] = __fmul_rn(lut[b1 & 15], am);
  }
}

// Round-half-even of a clamped value to an integer, and small integers back to fp32,
// with plain fp32 additions instead of the conversion instructions (which issue at a
// quarter of the rate): adding 1.5 * 2^23 leaves the rounded integer in the low mantissa
// bits (two's complement for negatives), and 2^23 | k is the float 2^23 + k.  Clamping to
// integer bounds before or after the rounding gives the same result.
__device__ __forceinline__ int round_clamped(float x, float lo, float hi) {
  const float t = __fadd_rn(fminf(fmaxf(x, lo), hi), 12582912.0f);
  return (int)(__float_as_uint(t) - 0x4B400000u);
}
// fp32 value of k - bias for 0 <= k < 2^22
__device__ __forceinline__ float small_int_to_f32(uint32_t k, float bias_plus_2p23) {
  return __fsub_rn(__uint_as_float(0x4B000000u | k), bias_plus_2p23);
}

// int8: 16 values -> four words of bytes.  The magic constant carries the +128 bias, so the
// low byte of the sum is q + 128; flipping bit 7 of every byte gives two's complement q.
__device__ __forceinline__ int int8_round(float x, float inv) {
  return round_clamped(__fmul_rn(x, inv), -128.f, 127.f);
}
__device__ __forceinline__ uint32_t int8_biased(float x, float inv) {
  const float t = __fadd_rn(fminf(fmaxf(__fmul_rn(x, inv), -128.f), 127.f), 12583040.0f);  // 1.5 * 2^23 + 128
  return __float_as_uint(t) & 0xffu;
}
__device__ __forceinline__ uint4 int8_pack16(const float (&e)[16], float inv) {
  uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i >> 2] |= int8_biased(e[i], inv) << (8 * (i & 3));
  return make_uint4(w[0] ^ 0x80808080u, w[1] ^ 0x80808080u, w[2] ^ 0x80808080u, w[3] ^ 0x80808080u);
}

// GPTQ int4: 16 values -> two words of eight (v + 8) nibbles, first value in the low nibble.
// Here the magic constant carries the +8, so the low nibble of the sum is the stored code.
__device__ __forceinline__ int int4_round(float x, float inv) {
  return round_clamped(__fmul_rn(x, inv), -8.f, 7.f);
}
__device__ __forceinline__ uint32_t int4_code(float x, float inv) {
  const float t = __fadd_rn(fminf(fmaxf(__fmul_rn(x, inv), -8.f), 7.f), 12582920.0f);  // 1.5 * 2^23 + 8
  return __float_as_uint(t) & 0xfu;
}
__device__ __forceinline__ void int4_pack16(const float (&e)[16], float inv, uint32_t& w0, uint32_t& w1) {
  w0 = 0; w1 = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w0 |= int4_code(e[i], inv) << (4 * i);
    w1 |= int4_code(e[8 + i], inv) << (4 * i);
  }
}
// scale of a symmetric int group from its absolute maximum: the stored scale is the fp32
// value rounded to S; quantization divides by the unrounded fp32 scale
template <typename S>
__device__ __forceinline__ float stored_scale(float scale) { return Elem<S>::to_f32(Elem<S>::from_f32(scale)); }


// ---- GPTQ int4 tile: 32 output rows x 128 input columns, 256 threads.  Thread t owns
// row (t >> 3) and the 16 columns starting at (t & 7) * 16, so the eight lanes of a row
// are consecutive and a quantization group (32, 64 or 128 columns) is 2, 4 or 8 lanes.
// Packed words pass through shared memory so that the transposed (in_f / 8, out_f)
// layout is written in 128-byte runs along out_f.
struct Int4Tile {
  int32_t words[16][33];
  float scale[4][33];
};
// Quantizes the caller's 16 values into the tile (call from all 256 threads; rows that
// do not exist pass zeros).  Follow with __syncthreads() before int4_tile_store.
__device__ __forceinline__ void int4_tile_quantize(const float (&e)[16], int group, Int4Tile& sm) {
  const int lr = threadIdx.x >> 3, seg = threadIdx.x & 7;
  const int lanes = group >> 4;
  const float scale = __fmul_rn(group_max(amax16(e), lanes), 0.125f);
  uint32_t w0, w1;
  int4_pack16(e, rcp_rn(fmaxf(scale, kEps)), w0, w1);
  sm.words[seg * 2][lr] = (int32_t)w0;
  sm.words[seg * 2 + 1][lr] = (int32_t)w1;
  if ((seg % lanes) == 0) sm.scale[seg / lanes][lr] = scale;
}
// Writes the tile into one payload: global rows [grow0, grow0 + rows_valid) of a weight
// with out_f rows, input columns [col0, col0 + 128).
template <typename S>
__device__ __forceinline__ void int4_tile_store(const Int4Tile& sm, int64_t out_f, int64_t grow0, int rows_valid,
                                                int64_t col0, int group, int32_t* qweight, S* scales) {
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) {
    const int k = i >> 5, lr = i & 31;
    if (lr < rows_valid) qweight[(col0 / 8 + k) * out_f + grow0 + lr] = sm.words[k][lr];
  }
  const int groups_per_tile = 128 / group;
  for (int i = threadIdx.x; i < groups_per_tile * 32; i += blockDim.x) {
    const int gi = i >> 5, lr = i & 31;
    if (lr < rows_valid) scales[(col0 / group + gi) * out_f + grow0 + lr] = Elem<S>::from_f32(sm.scale[gi][lr]);
  }
}
// The same tile into `n` replicas of the payload (own and peer GPUs'): every word is read
// from shared memory once and its address computed once.
template <typename S, int MAXR>
__device__ __forceinline__ void int4_tile_store_multi(const Int4Tile& sm, int64_t out_f, int64_t grow0, int rows_valid,
                                                      int64_t col0, int group, uint8_t* const (&p0)[MAXR],
                                                      uint8_t* const (&p1)[MAXR], int n) {
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) {
    const int k = i >> 5, lr = i & 31;
    if (lr < rows_valid) {
      const int64_t at = (col0 / 8 + k) * out_f + grow0 + lr;
      const int32_t w = sm.words[k][lr];
#pragma unroll
      for (int j = 0; j < MAXR; ++j)
        if (j < n) reinterpret_cast<int32_t*>(p0[j])[at] = w;
    }
  }
  const int groups_per_tile = 128 / group;
  for (int i = threadIdx.x; i < groups_per_tile * 32; i += blockDim.x) {
    const int gi = i >> 5, lr = i & 31;
    if (lr < rows_valid) {
      const int64_t at = (col0 / group + gi) * out_f + grow0 + lr;
      const S v = Elem<S>::from_f32(sm.scale[gi][lr]);
#pragma unroll
      for (int j = 0; j < MAXR; ++j)
        if (j < n) reinterpret_cast<S*>(p1[j])[at] = v;
    }
  }
}
// Loads a tile of a payload into shared memory (rows beyond rows_valid read as zero).
template <typename S>
__device__ __forceinline__ void int4_tile_load(Int4Tile& sm, int64_t out_f, int64_t grow0, int rows_valid,
                                               int64_t col0, int group, const int32_t* qweight, const S* scales) {
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) {
    const int k = i >> 5, lr = i & 31;
    sm.words[k][lr] = (lr < rows_valid) ? qweight[(col0 / 8 + k) * out_f + grow0 + lr] : 0;
  }
  const int groups_per_tile = 128 / group;
  for (int i = threadIdx.x; i < groups_per_tile * 32; i += blockDim.x) {
    const int gi = i >> 5, lr = i & 31;
    sm.scale[gi][lr] = (lr < rows_valid) ? Elem<S>::to_f32(scales[(col0 / group + gi) * out_f + grow0 + lr]) : 0.f;
  }
}
// value of nibble i of the pair (w0, w1) times scale, for the caller's 16 columns
__device__ __forceinline__ void int4_unpack16(uint32_t w0, uint32_t w1, float s, float (&e)[16]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    e[i] = __fmul_rn(small_int_to_f32((w0 >> (4 * i)) & 0xfu, 8388616.0f), s);
    e[8 + i] = __fmul_rn(small_int_to_f32((w1 >> (4 * i)) & 0xfu, 8388616.0f), s);
  }
}

// 16 elements with or without the 32-byte alignment that the vector path needs
template <typename T>
__device__ __forceinline__ void load16_any(const T* p, float (&x)[16], bool aligned) {
  if (aligned) { Elem<T>::load16(p, x); return; }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = Elem<T>::to_f32(p[i]);
}
template <typename T>
__device__ __forceinline__ void store16_any(T* p, const float (&x)[16], bool aligned) {
  if (aligned) { Elem<T>::store16(p, x); return; }
#pragma unroll
  for (int i = 0; i < 16; ++i) p[i] = Elem<T>::from_f32(x[i]);
}
// The integer formats de-quantize in the scale dtype S (the product is rounded to S),
// except when fp32 output is asked for; the result is then cast to the output dtype T.
template <typename T, typename S>
__device__ __forceinline__ float round_like_dequant(float prod) {
  return (sizeof(T) == 4) ? prod : Elem<S>::to_f32(Elem<S>::from_f32(prod));
}

}  // namespace qm
}  // namespace oab
