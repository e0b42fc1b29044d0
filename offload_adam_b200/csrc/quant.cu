// Weight-only quantize / dequantize kernels for sm_100a: NVFP4, NF4, GPTQ int4, int8.
//
// Storage formats and rounding rules follow the reference's four formats
// (reference: src/offload_adam/qweight/nvfp4.py:133-191, nf4.py:102-152,
// int4.py:30-92, int8.py:29-57) so that packed tensors are interchangeable:
//   NVFP4  two E2M1 codes per byte (even column -> low nibble), one e4m3 scale per
//          16 elements, one fp32 tensor scale = amax / (448 * 6);
//   NF4    two codebook indices per byte (even column -> HIGH nibble), fp32 absmax
//          per block, nearest codebook entry with the lowest index winning ties;
//   int4   (in_f/8, out_f) int32, eight (v + 8) nibbles LSB first along in_f,
//          scales (groups, out_f) = absmax / 8, round-half-even, clamp [-8, 7];
//   int8   (out_f, in_f) int8, per-row scale = absmax / 127, round-half-even.
// All reciprocals are correctly rounded (rcp.rn) and then multiplied, never a
// division of the element, matching the reference quantizers bit for bit.
//
// Each thread owns 16 consecutive elements of a row and moves them with 256-bit
// loads/stores; block statistics are combined with warp shuffles.  The E2M1
// conversions use the Blackwell cvt instructions (cvt.rn.satfinite.e2m1x2.f32,
// cvt.rn.f16x2.e2m1x2).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "quant.h"

namespace oab {
namespace {

constexpr int kThreads = 256;
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
    for (int i = 0; i < 8; ++i) a.w[i] = f32_to_bf16_rne_bits(x[2 * i]) | (f32_to_bf16_rne_bits(x[2 * i + 1]) << 16);
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

// ------------------------------------------------------------------------ amax
template <typename T>
__global__ void __launch_bounds__(kThreads) absmax_kernel(const T* x, int64_t n, float* out) {
  __shared__ float red[kThreads / 32];
  float m = 0.f;
  const int64_t nvec = n >> 4;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * kThreads) {
    float e[16];
    Elem<T>::load16(x + v * 16, e);
    m = fmaxf(m, amax16(e));
  }
  for (int64_t i = (nvec << 4) + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
    m = fmaxf(m, fabsf(Elem<T>::to_f32(x[i])));
  float bm = block_max<kThreads>(m, red);
  if (threadIdx.x == 0 && bm > 0.f) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(bm));
}

// ----------------------------------------------------------------------- NVFP4
// one thread per 16-element block; global_scale[0] is written by thread 0
template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T* x, int64_t nblocks, const float* amax, uint8_t* packed, uint8_t* scales,
                      float* global_scale_out) {
  const float tensor_amax = fmaxf(*amax, kEps);
  const float global = __fdiv_rn(tensor_amax, 448.0f * 6.0f);
  const float inv_global = rcp_rn(fmaxf(global, kEps));
  if (blockIdx.x == 0 && threadIdx.x == 0) *global_scale_out = global;
  for (int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * kThreads) {
    float e[16];
    Elem<T>::load16(x + b * 16, e);
    const float bamax = fmaxf(amax16(e), kEps);
    const uint8_t s8 = f32_to_e4m3(__fmul_rn(__fdiv_rn(bamax, 6.0f), inv_global));
    scales[b] = s8;
    const float eff = __fmul_rn(e4m3_to_f32(s8), global);
    const float inv_eff = rcp_rn(fmaxf(eff, kEps));
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w0 |= e2m1x2(__fmul_rn(e[2 * i], inv_eff), __fmul_rn(e[2 * i + 1], inv_eff)) << (8 * i);
      w1 |= e2m1x2(__fmul_rn(e[8 + 2 * i], inv_eff), __fmul_rn(e[9 + 2 * i], inv_eff)) << (8 * i);
    }
    *reinterpret_cast<uint2*>(packed + b * 8) = make_uint2(w0, w1);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t* packed, const uint8_t* scales, const float* global_scale,
                        int64_t nblocks, T* out) {
  const float global = *global_scale;
  for (int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * kThreads) {
    const uint2 w = *reinterpret_cast<const uint2*>(packed + b * 8);
    const float eff = __fmul_rn(e4m3_to_f32(scales[b]), global);
    float e[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = e2m1x2_to_f32((w.x >> (8 * i)) & 0xffu);
      float2 c = e2m1x2_to_f32((w.y >> (8 * i)) & 0xffu);
      e[2 * i] = __fmul_rn(a.x, eff); e[2 * i + 1] = __fmul_rn(a.y, eff);
      e[8 + 2 * i] = __fmul_rn(c.x, eff); e[9 + 2 * i] = __fmul_rn(c.y, eff);
    }
    Elem<T>::store16(out + b * 16, e);
  }
}

// ------------------------------------------------------------------------- NF4
__constant__ float kNF4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// index of the nearest codebook entry; among equal distances the lowest index wins
// (the rule of a sequential scan with a strict '<').  A 4-step bisection on the
// midpoints finds a candidate, its two neighbours settle rounding and ties.
__device__ __forceinline__ int nf4_nearest(float x, const float* lut) {
  int lo = 0;
#pragma unroll
  for (int step = 8; step > 0; step >>= 1) {
    int mid = lo + step;  // compare against the midpoint between mid-1 and mid
    float mp = 0.5f * (lut[mid - 1] + lut[mid]);
    lo = (x > mp) ? mid : lo;
  }
  int best = lo > 0 ? lo - 1 : lo;
  float bd = fabsf(__fsub_rn(x, lut[best]));
  int hi = lo < 15 ? lo + 1 : lo;
  for (int c = best + 1; c <= hi; ++c) {
    float d = fabsf(__fsub_rn(x, lut[c]));
    if (d < bd) { bd = d; best = c; }
  }
  return best;
}

// one thread per 16 elements; lanes_per_block = blocksize / 16 (power of two <= 32)
template <typename T>
__global__ void __launch_bounds__(kThreads)
nf4_quantize_kernel(const T* x, int64_t nchunks, int lanes_per_block, uint8_t* packed, float* absmax) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNF4[threadIdx.x];
  __syncthreads();
  // grid covers whole warps so every shuffle has its partners
  const int64_t total = (nchunks + 31) / 32 * 32;
  for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < total; c += (int64_t)gridDim.x * kThreads) {
    float e[16];
    const bool live = c < nchunks;
    if (live) Elem<T>::load16(x + c * 16, e);
    else {
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = 0.f;
    }
    const float am = group_max(amax16(e), lanes_per_block);
    if (!live) continue;
    if ((c % lanes_per_block) == 0) absmax[c / lanes_per_block] = am;
    const float inv = rcp_rn(fmaxf(am, kEps));
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b0 = (nf4_nearest(__fmul_rn(e[2 * i], inv), lut) << 4) | nf4_nearest(__fmul_rn(e[2 * i + 1], inv), lut);
      uint32_t b1 = (nf4_nearest(__fmul_rn(e[8 + 2 * i], inv), lut) << 4) | nf4_nearest(__fmul_rn(e[9 + 2 * i], inv), lut);
      w0 |= b0 << (8 * i);
      w1 |= b1 << (8 * i);
    }
    *reinterpret_cast<uint2*>(packed + c * 8) = make_uint2(w0, w1);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nf4_dequantize_kernel(const uint8_t* packed, const float* absmax, int64_t nchunks, int lanes_per_block, T* out) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNF4[threadIdx.x];
  __syncthreads();
  for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < nchunks; c += (int64_t)gridDim.x * kThreads) {
    const uint2 w = *reinterpret_cast<const uint2*>(packed + c * 8);
    const float am = absmax[c / lanes_per_block];
    float e[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b0 = (w.x >> (8 * i)) & 0xffu, b1 = (w.y >> (8 * i)) & 0xffu;
      e[2 * i] = __fmul_rn(lut[b0 >> 4], am); e[2 * i + 1] = __fmul_rn(lut[b0 & 15], am);
      e[8 + 2 * i] = __fmul_rn(lut[b1 >> 4], am); e[9 + 2 * i] = __fmul_rn(lut[b1 & 15], am);
    }
    Elem<T>::store16(out + c * 16, e);
  }
}

// ------------------------------------------------------------------------ int8
// one block per row; the second pass re-reads the row, which the first pass left in L2
template <typename T, typename S>
__global__ void __launch_bounds__(kThreads)
int8_quantize_kernel(const T* x, int64_t in_f, int8_t* q, S* scales) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_inv;
  const int64_t row = blockIdx.x;
  const T* xr = x + row * in_f;
  float m = 0.f;
  const bool vec = (in_f % 16 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 31u) == 0);
  if (vec) {
    for (int64_t v = threadIdx.x; v < (in_f >> 4); v += kThreads) {
      float e[16];
      Elem<T>::load16(xr + v * 16, e);
      m = fmaxf(m, amax16(e));
    }
  } else {
    for (int64_t i = threadIdx.x; i < in_f; i += kThreads) m = fmaxf(m, fabsf(Elem<T>::to_f32(xr[i])));
  }
  float bm = block_max<kThreads>(m, red);
  if (threadIdx.x == 0) {
    const float scale = __fdiv_rn(bm, 127.0f);
    scales[row] = Elem<S>::from_f32(scale);
    s_inv = rcp_rn(fmaxf(scale, kEps));
  }
  __syncthreads();
  const float inv = s_inv;
  int8_t* qr = q + row * in_f;
  if (vec && ((reinterpret_cast<uintptr_t>(qr) & 15u) == 0)) {
    for (int64_t v = threadIdx.x; v < (in_f >> 4); v += kThreads) {
      float e[16];
      Elem<T>::load16(xr + v * 16, e);
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float r = fminf(fmaxf(rintf(__fmul_rn(e[i], inv)), -128.f), 127.f);
        w[i >> 2] |= ((uint32_t)(uint8_t)(int8_t)(int)r) << (8 * (i & 3));
      }
      *reinterpret_cast<uint4*>(qr + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int64_t i = threadIdx.x; i < in_f; i += kThreads) {
      float r = fminf(fmaxf(rintf(__fmul_rn(Elem<T>::to_f32(xr[i]), inv)), -128.f), 127.f);
      qr[i] = (int8_t)(int)r;
    }
  }
}

// out = S(q) * scale, computed and rounded in S
template <typename S>
__global__ void __launch_bounds__(kThreads)
int8_dequantize_kernel(const int8_t* q, const S* scales, int64_t out_f, int64_t in_f, S* out) {
  const int64_t n = out_f * in_f;
  const bool vec = (in_f % 16 == 0) && ((reinterpret_cast<uintptr_t>(q) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 31u) == 0);
  if (vec) {
    const int64_t nvec = n >> 4;
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * kThreads) {
      const float s = Elem<S>::to_f32(scales[(v * 16) / in_f]);
      const uint4 w4 = *reinterpret_cast<const uint4*>(q + v * 16);
      const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
      float e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = __fmul_rn((float)(int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xffu), s);
      Elem<S>::store16(out + v * 16, e);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
      out[i] = Elem<S>::from_f32(__fmul_rn((float)q[i], Elem<S>::to_f32(scales[i / in_f])));
  }
}

// ------------------------------------------------------------------------ int4
// Tile = 32 rows x 128 columns.  A warp quantizes 4 rows; each lane owns 4 columns.
// Packed words go through shared memory so that the (in_f/8, out_f) layout is
// written with 128-byte rows-contiguous stores.
template <typename T, typename S>
__global__ void __launch_bounds__(kThreads)
int4_quantize_kernel(const T* x, int64_t out_f, int64_t in_f, int group, int32_t* qweight, S* scales) {
  __shared__ int32_t tile[16][33];
  __shared__ float tscale[4][33];
  const int64_t row0 = (int64_t)blockIdx.x * 32;
  const int64_t col0 = (int64_t)blockIdx.y * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lanes_per_group = group / 4;
  const int groups_per_tile = 128 / group;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int lr = warp * 4 + r;
    const int64_t row = row0 + lr;
    float e[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < out_f) {
      const T* src = x + row * in_f + col0 + lane * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) e[i] = Elem<T>::to_f32(src[i]);
    }
    float am = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
    am = group_max(am, lanes_per_group);
    const float scale = __fmul_rn(am, 0.125f);
    const float inv = rcp_rn(fmaxf(scale, kEps));
    uint32_t nib = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = fminf(fmaxf(rintf(__fmul_rn(e[i], inv)), -8.f), 7.f);
      nib |= ((uint32_t)((int)q + 8) & 0xfu) << (4 * i);
    }
    const uint32_t other = __shfl_down_sync(0xffffffffu, nib, 1);
    if ((lane & 1) == 0) tile[lane >> 1][lr] = (int32_t)(nib | (other << 16));
    if ((lane % lanes_per_group) == 0) tscale[lane / lanes_per_group][lr] = scale;
  }
  __syncthreads();
  // 16 packed rows x 32 output rows
  for (int i = threadIdx.x; i < 16 * 32; i += kThreads) {
    const int k = i >> 5, lr = i & 31;
    if (row0 + lr < out_f) qweight[(col0 / 8 + k) * out_f + row0 + lr] = tile[k][lr];
  }
  for (int i = threadIdx.x; i < groups_per_tile * 32; i += kThreads) {
    const int gi = i >> 5, lr = i & 31;
    if (row0 + lr < out_f) scales[(col0 / group + gi) * out_f + row0 + lr] = Elem<S>::from_f32(tscale[gi][lr]);
  }
}

template <typename S>
__global__ void __launch_bounds__(kThreads)
int4_dequantize_kernel(const int32_t* qweight, const S* scales, int64_t out_f, int64_t in_f, int group, S* out) {
  __shared__ int32_t tile[16][33];
  __shared__ float tscale[4][33];
  const int64_t row0 = (int64_t)blockIdx.x * 32;
  const int64_t col0 = (int64_t)blockIdx.y * 128;
  const int groups_per_tile = 128 / group;
  for (int i = threadIdx.x; i < 16 * 32; i += kThreads) {
    const int k = i >> 5, lr = i & 31;
    tile[k][lr] = (row0 + lr < out_f) ? qweight[(col0 / 8 + k) * out_f + row0 + lr] : 0;
  }
  for (int i = threadIdx.x; i < groups_per_tile * 32; i += kThreads) {
    const int gi = i >> 5, lr = i & 31;
    tscale[gi][lr] = (row0 + lr < out_f) ? Elem<S>::to_f32(scales[(col0 / group + gi) * out_f + row0 + lr]) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int lr = warp * 4 + r;
    const int64_t row = row0 + lr;
    if (row >= out_f) continue;
    const uint32_t w = (uint32_t)tile[lane >> 1][lr] >> (16 * (lane & 1));
    const float s = tscale[(lane * 4) / group][lr];
    S* dst = out + row * in_f + col0 + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = Elem<S>::from_f32(__fmul_rn((float)((int)((w >> (4 * i)) & 0xfu) - 8), s));
  }
}

int grid_for(int64_t work_items) {
  int64_t want = (work_items + kThreads - 1) / kThreads;
  int cap = kNumSMs * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

#define OAB_DISPATCH_IN(dt, ...)                                             \
  switch (dt) {                                                              \
    case kF32: { using T = float; __VA_ARGS__; break; }                      \
    case kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case kF16: { using T = __half; __VA_ARGS__; break; }                     \
    default: return cudaErrorInvalidValue;                                   \
  }
#define OAB_DISPATCH_SCALE(dt, ...)                                          \
  switch (dt) {                                                              \
    case kF32: { using S = float; __VA_ARGS__; break; }                      \
    case kBF16: { using S = __nv_bfloat16; __VA_ARGS__; break; }             \
    case kF16: { using S = __half; __VA_ARGS__; break; }                     \
    default: return cudaErrorInvalidValue;                                   \
  }

cudaError_t launch_absmax(const void* x, int dtype, int64_t n, float* out, cudaStream_t st) {
  count_launch();
  OAB_DISPATCH_IN(dtype, absmax_kernel<T><<<grid_for((n + 15) / 16), kThreads, 0, st>>>((const T*)x, n, out));
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_quantize(const void* x, int dtype, int64_t numel, const float* amax,
                                  uint8_t* packed, uint8_t* scales, float* global_scale, cudaStream_t st) {
  const int64_t nb = numel / 16;
  count_launch();
  OAB_DISPATCH_IN(dtype, nvfp4_quantize_kernel<T><<<grid_for(nb), kThreads, 0, st>>>((const T*)x, nb, amax, packed, scales, global_scale));
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* global_scale,
                                    int64_t numel, void* out, int dtype, cudaStream_t st) {
  const int64_t nb = numel / 16;
  count_launch();
  OAB_DISPATCH_IN(dtype, nvfp4_dequantize_kernel<T><<<grid_for(nb), kThreads, 0, st>>>(packed, scales, global_scale, nb, (T*)out));
  return cudaGetLastError();
}

cudaError_t launch_nf4_quantize(const void* x, int dtype, int64_t numel, int blocksize, uint8_t* packed,
                                float* absmax, cudaStream_t st) {
  const int64_t nc = numel / 16;
  count_launch();
  OAB_DISPATCH_IN(dtype, nf4_quantize_kernel<T><<<grid_for(nc), kThreads, 0, st>>>((const T*)x, nc, blocksize / 16, packed, absmax));
  return cudaGetLastError();
}

cudaError_t launch_nf4_dequantize(const uint8_t* packed, const float* absmax, int64_t numel, int blocksize,
                                  void* out, int dtype, cudaStream_t st) {
  const int64_t nc = numel / 16;
  count_launch();
  OAB_DISPATCH_IN(dtype, nf4_dequantize_kernel<T><<<grid_for(nc), kThreads, 0, st>>>(packed, absmax, nc, blocksize / 16, (T*)out));
  return cudaGetLastError();
}

cudaError_t launch_int8_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int8_t* q,
                                 void* scales, int scale_dtype, cudaStream_t st) {
  if (out_f <= 0) return cudaSuccess;
  count_launch();
  OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
      int8_quantize_kernel<T, S><<<(unsigned)out_f, kThreads, 0, st>>>((const T*)x, in_f, q, (S*)scales)));
  return cudaGetLastError();
}

cudaError_t launch_int8_dequantize(const int8_t* q, const void* scales, int scale_dtype, int64_t out_f,
                                   int64_t in_f, void* out, cudaStream_t st) {
  count_launch();
  OAB_DISPATCH_SCALE(scale_dtype, int8_dequantize_kernel<S><<<grid_for((out_f * in_f + 15) / 16), kThreads, 0, st>>>(q, (const S*)scales, out_f, in_f, (S*)out));
  return cudaGetLastError();
}

cudaError_t launch_int4_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int group,
                                 int32_t* qweight, void* scales, int scale_dtype, cudaStream_t st) {
  dim3 grid((unsigned)((out_f + 31) / 32), (unsigned)(in_f / 128));
  count_launch();
  OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
      int4_quantize_kernel<T, S><<<grid, kThreads, 0, st>>>((const T*)x, out_f, in_f, group, qweight, (S*)scales)));
  return cudaGetLastError();
}

cudaError_t launch_int4_dequantize(const int32_t* qweight, const void* scales, int scale_dtype, int64_t out_f,
                                   int64_t in_f, int group, void* out, cudaStream_t st) {
  dim3 grid((unsigned)((out_f + 31) / 32), (unsigned)(in_f / 128));
  count_launch();
  OAB_DISPATCH_SCALE(scale_dtype, int4_dequantize_kernel<S><<<grid, kThreads, 0, st>>>(qweight, (const S*)scales, out_f, in_f, group, (S*)out));
  return cudaGetLastError();
}

}  // namespace oab
