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
#include "quant.h"
#include "quant_math.cuh"

namespace oab {
namespace {

constexpr int kThreads = 256;
using namespace qm;

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
// One thread per 16-element block.  The four scale bytes of four neighbouring blocks
// are combined with shuffles and leave as one 32-bit store; global_scale[0] is written
// by thread 0.  FAKE: instead of the payload, write the de-quantized values to `out`.
template <typename T, bool FAKE>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T* x, int64_t nblocks, const float* amax, uint8_t* packed, uint8_t* scales,
                      float* global_scale_out, int scale_words_ok, T* out) {
  float global, inv_global;
  nvfp4_global(*amax, global, inv_global);
  if (!FAKE && blockIdx.x == 0 && threadIdx.x == 0) *global_scale_out = global;
  const int lane = threadIdx.x & 31;
  // whole warps iterate together so that every shuffle has its partners
  for (int64_t base = (int64_t)blockIdx.x * kThreads + (threadIdx.x & ~31); base < nblocks;
       base += (int64_t)gridDim.x * kThreads) {
    const int64_t b = base + lane;
    const bool live = b < nblocks;
    float e[16];
    uint8_t s8 = 0;
    uint32_t w0 = 0, w1 = 0;
    if (live) {
      Elem<T>::load16(x + b * 16, e);
      nvfp4_pack16(e, global, inv_global, s8, w0, w1);
    }
    if (FAKE) {
      if (live) {
        nvfp4_unpack16(w0, w1, __fmul_rn(e4m3_to_f32(s8), global), e);
        Elem<T>::store16(out + b * 16, e);
      }
      continue;
    }
    uint32_t s32 = s8;
    s32 |= __shfl_down_sync(0xffffffffu, (uint32_t)s8, 1) << 8;
    s32 |= __shfl_down_sync(0xffffffffu, s32, 2) << 16;
    if (!live) continue;
    *reinterpret_cast<uint2*>(packed + b * 8) = make_uint2(w0, w1);
    if (scale_words_ok && b + 3 < nblocks) {
      if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(scales + b) = s32;
    } else {
      scales[b] = s8;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t* packed, const uint8_t* scales, const float* global_scale,
                        int64_t nblocks, T* out) {
  const float global = *global_scale;
  for (int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * kThreads) {
    const uint2 w = *reinterpret_cast<const uint2*>(packed + b * 8);
    float e[16];
    nvfp4_unpack16(w.x, w.y, __fmul_rn(e4m3_to_f32(scales[b]), global), e);
    Elem<T>::store16(out + b * 16, e);
  }
}

// ------------------------------------------------------------------------- NF4
// one thread per 16 elements; lanes_per_block = blocksize / 16 (power of two <= 32).
// FAKE: write the de-quantized values to `out` instead of the payload.
template <typename T, bool FAKE>
__global__ void __launch_bounds__(kThreads)
nf4_quantize_kernel(const T* x, int64_t nchunks, int lanes_per_block, uint8_t* packed, float* absmax, T* out) {
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
    uint32_t w0, w1;
    nf4_pack16(e, rcp_rn(fmaxf(am, kEps)), lut, w0, w1);
    if (FAKE) {
      nf4_unpack16(w0, w1, am, lut, e);
      Elem<T>::store16(out + c * 16, e);
      continue;
    }
    if ((c % lanes_per_block) == 0) absmax[c / lanes_per_block] = am;
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
    float e[16];
    nf4_unpack16(w.x, w.y, absmax[c / lanes_per_block], lut, e);
    Elem<T>::store16(out + c * 16, e);
  }
}

// ------------------------------------------------------------------------ int8
// one block per row; the second pass re-reads the row, which the first pass left in L2.
// FAKE: write the de-quantized row to `out` (dtype T) instead of the payload.
template <typename T, typename S, bool FAKE>
__global__ void __launch_bounds__(kThreads)
int8_quantize_kernel(const T* x, int64_t out_f, int64_t in_f, int8_t* q, S* scales, T* out) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_inv, s_scale;
  for (int64_t row = blockIdx.x; row < out_f; row += gridDim.x) {
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
      if (!FAKE) scales[row] = Elem<S>::from_f32(scale);
      s_scale = stored_scale<S>(scale);
      s_inv = rcp_rn(fmaxf(scale, kEps));
    }
    __syncthreads();
    const float inv = s_inv, sc = s_scale;
    if (FAKE) {
      T* orow = out + row * in_f;
      const bool ovec = vec && ((reinterpret_cast<uintptr_t>(orow) & 31u) == 0);
      for (int64_t v = threadIdx.x; v < ((in_f + 15) >> 4); v += kThreads) {
        const int64_t left = in_f - v * 16;
        if (ovec) {
          float e[16];
          Elem<T>::load16(xr + v * 16, e);
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = round_like_dequant<T, S>(__fmul_rn((float)int8_round(e[i], inv), sc));
          Elem<T>::store16(orow + v * 16, e);
        } else {
          for (int i = 0; i < 16 && i < left; ++i) {
            const float xv = Elem<T>::to_f32(xr[v * 16 + i]);
            orow[v * 16 + i] = Elem<T>::from_f32(round_like_dequant<T, S>(__fmul_rn((float)int8_round(xv, inv), sc)));
          }
        }
      }
    } else {
      int8_t* qr = q + row * in_f;
      if (vec && ((reinterpret_cast<uintptr_t>(qr) & 15u) == 0)) {
        for (int64_t v = threadIdx.x; v < (in_f >> 4); v += kThreads) {
          float e[16];
          Elem<T>::load16(xr + v * 16, e);
          *reinterpret_cast<uint4*>(qr + v * 16) = int8_pack16(e, inv);
        }
      } else {
        for (int64_t i = threadIdx.x; i < in_f; i += kThreads) qr[i] = (int8_t)int8_round(Elem<T>::to_f32(xr[i]), inv);
      }
    }
    __syncthreads();  // s_inv / s_scale are rewritten for the next row
  }
}

// Same result, for rows of at most kThreads * VPT * 16 columns that start 32-byte aligned:
// every thread keeps its VPT vectors of the row in registers between the maximum and the
// rounding, so the row is read once.
template <typename T, typename S, bool FAKE, int VPT>
__global__ void __launch_bounds__(kThreads)
int8_quantize_cached_kernel(const T* x, int64_t out_f, int64_t in_f, int8_t* q, S* scales, T* out) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_inv, s_scale;
  const int nvec = (int)(in_f >> 4);
  for (int64_t row = blockIdx.x; row < out_f; row += gridDim.x) {
    const T* xr = x + row * in_f;
    float e[VPT][16];
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * kThreads;
      if (v < nvec) {
        Elem<T>::load16(xr + (int64_t)v * 16, e[k]);
        m = fmaxf(m, amax16(e[k]));
      }
    }
    const float bm = block_max<kThreads>(m, red);
    if (threadIdx.x == 0) {
      const float scale = __fdiv_rn(bm, 127.0f);
      if (!FAKE) scales[row] = Elem<S>::from_f32(scale);
      s_scale = stored_scale<S>(scale);
      s_inv = rcp_rn(fmaxf(scale, kEps));
    }
    __syncthreads();
    const float inv = s_inv, sc = s_scale;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * kThreads;
      if (v < nvec) {
        if (FAKE) {
#pragma unroll
          for (int i = 0; i < 16; ++i) e[k][i] = round_like_dequant<T, S>(__fmul_rn((float)int8_round(e[k][i], inv), sc));
          Elem<T>::store16(out + row * in_f + (int64_t)v * 16, e[k]);
        } else {
          *reinterpret_cast<uint4*>(q + row * in_f + (int64_t)v * 16) = int8_pack16(e[k], inv);
        }
      }
    }
    __syncthreads();  // s_inv / s_scale are rewritten for the next row
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
      // 32-bit division when the row index fits (it always does for weights)
      const int64_t row = (n < (int64_t(1) << 31)) ? (int64_t)((uint32_t)(v * 16) / (uint32_t)in_f) : (v * 16) / in_f;
      const float s = Elem<S>::to_f32(scales[row]);
      const uint4 w4 = *reinterpret_cast<const uint4*>(q + v * 16);
      const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
      float e[16];
#pragma unroll
      // (byte ^ 0x80) - 128 is the signed value; see small_int_to_f32
      for (int i = 0; i < 16; ++i) e[i] = __fmul_rn(small_int_to_f32(((w[i >> 2] >> (8 * (i & 3))) & 0xffu) ^ 0x80u, 8388736.0f), s);
      Elem<S>::store16(out + v * 16, e);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
      out[i] = Elem<S>::from_f32(__fmul_rn((float)q[i], Elem<S>::to_f32(scales[i / in_f])));
  }
}

// ------------------------------------------------------------------------ int4
// Tile = 32 rows x 128 columns (see Int4Tile): every thread moves 16 consecutive
// elements of a row with one (bf16/fp16) or two (fp32) 256-bit accesses; the packed
// words are transposed through shared memory.
// A CTA can work on several neighbouring tiles of one 32-row band, all of their loads issued
// before the first use; measured on B200, quantization is fastest with one.
constexpr int kInt4QuantTiles = 1;

template <typename T, typename S, int kInt4Tiles>
__global__ void __launch_bounds__(kThreads)
int4_quantize_kernel(const T* x, int64_t out_f, int64_t in_f, int group, int32_t* qweight, S* scales, int aligned) {
  __shared__ Int4Tile sm[kInt4Tiles];
  const int64_t row0 = (int64_t)blockIdx.x * 32;
  const int64_t tile0 = (int64_t)blockIdx.y * kInt4Tiles, ntiles = in_f >> 7;
  const int lr = threadIdx.x >> 3, seg = threadIdx.x & 7;
  const bool row_ok = row0 + lr < out_f;
  float e[kInt4Tiles][16];
#pragma unroll
  for (int t = 0; t < kInt4Tiles; ++t) {
    if (row_ok && tile0 + t < ntiles) load16_any(x + (row0 + lr) * in_f + ((tile0 + t) << 7) + seg * 16, e[t], aligned != 0);
    else {
#pragma unroll
      for (int i = 0; i < 16; ++i) e[t][i] = 0.f;
    }
  }
#pragma unroll
  for (int t = 0; t < kInt4Tiles; ++t) int4_tile_quantize(e[t], group, sm[t]);
  __syncthreads();
  const int64_t left = out_f - row0;
  const int valid = left < 32 ? (int)left : 32;
#pragma unroll
  for (int t = 0; t < kInt4Tiles; ++t)
    if (tile0 + t < ntiles) int4_tile_store<S>(sm[t], out_f, row0, valid, (tile0 + t) << 7, group, qweight, scales);
}

// De-quantization without shared memory: a warp takes 32 consecutive output rows, one per
// lane.  Word k of the transposed payload is then a coalesced 128-byte read across the
// lanes, and a lane that has read eight consecutive words owns 64 consecutive outputs of
// its row: a whole 128-byte line, written with four 256-bit stores.  Nothing is exchanged
// between threads, so there is no barrier and eight loads per lane are in flight at once.
// The warps of a CTA share the band and split its columns.
template <typename S>
__global__ void __launch_bounds__(kThreads)
int4_dequantize_kernel(const int32_t* qweight, const S* scales, int64_t out_f, int64_t in_f, int group, S* out, int aligned) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * 32 + lane;
  if (row >= out_f) return;
  const int64_t spans = in_f >> 6;  // 64 columns = 8 words per step
  for (int64_t sp = (int64_t)blockIdx.y * (kThreads / 32) + warp; sp < spans; sp += (int64_t)gridDim.y * (kThreads / 32)) {
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = (uint32_t)qweight[(sp * 8 + k) * out_f + row];
    const int64_t col = sp << 6;
    S* dst = out + row * in_f + col;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      // 16 columns never straddle a group (groups are 32, 64 or 128 columns wide)
      const float s = Elem<S>::to_f32(scales[((col + h * 16) / group) * out_f + row]);
      float e[16];
      int4_unpack16(w[2 * h], w[2 * h + 1], s, e);
      store16_any(dst + h * 16, e, aligned != 0);
    }
  }
}

// dq(q(x)) for int4 needs no transposition: one thread per 16 elements of a row, a
// group is 2, 4 or 8 consecutive lanes
template <typename T, typename S>
__global__ void __launch_bounds__(kThreads)
int4_fake_quant_kernel(const T* x, int64_t nchunks, int lanes_per_group, T* out) {
  const int64_t total = (nchunks + 31) / 32 * 32;
  for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < total; c += (int64_t)gridDim.x * kThreads) {
    float e[16];
    const bool live = c < nchunks;
    if (live) Elem<T>::load16(x + c * 16, e);
    else {
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = 0.f;
    }
    const float scale = __fmul_rn(group_max(amax16(e), lanes_per_group), 0.125f);
    if (!live) continue;
    const float inv = rcp_rn(fmaxf(scale, kEps)), sc = stored_scale<S>(scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] = round_like_dequant<T, S>(__fmul_rn((float)int4_round(e[i], inv), sc));
    Elem<T>::store16(out + c * 16, e);
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

namespace {
bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }
}  // namespace

cudaError_t launch_nvfp4_quantize(const void* x, int dtype, int64_t numel, const float* amax,
                                  uint8_t* packed, uint8_t* scales, float* global_scale, cudaStream_t st) {
  const int64_t nb = numel / 16;
  if (nb <= 0) return cudaSuccess;
  if (!aligned32(x) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return cudaErrorInvalidValue;
  const int words_ok = (reinterpret_cast<uintptr_t>(scales) & 3u) == 0;
  count_launch();
  OAB_DISPATCH_IN(dtype, nvfp4_quantize_kernel<T, false><<<grid_for(nb), kThreads, 0, st>>>(
      (const T*)x, nb, amax, packed, scales, global_scale, words_ok, nullptr));
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* global_scale,
                                    int64_t numel, void* out, int dtype, cudaStream_t st) {
  const int64_t nb = numel / 16;
  if (nb <= 0) return cudaSuccess;
  if (!aligned32(out) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return cudaErrorInvalidValue;
  count_launch();
  OAB_DISPATCH_IN(dtype, nvfp4_dequantize_kernel<T><<<grid_for(nb), kThreads, 0, st>>>(packed, scales, global_scale, nb, (T*)out));
  return cudaGetLastError();
}

cudaError_t launch_nf4_quantize(const void* x, int dtype, int64_t numel, int blocksize, uint8_t* packed,
                                float* absmax, cudaStream_t st) {
  const int64_t nc = numel / 16;
  if (nc <= 0) return cudaSuccess;
  if (!aligned32(x) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return cudaErrorInvalidValue;
  count_launch();
  OAB_DISPATCH_IN(dtype, nf4_quantize_kernel<T, false><<<grid_for(nc), kThreads, 0, st>>>(
      (const T*)x, nc, blocksize / 16, packed, absmax, nullptr));
  return cudaGetLastError();
}

cudaError_t launch_nf4_dequantize(const uint8_t* packed, const float* absmax, int64_t numel, int blocksize,
                                  void* out, int dtype, cudaStream_t st) {
  const int64_t nc = numel / 16;
  if (nc <= 0) return cudaSuccess;
  if (!aligned32(out) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return cudaErrorInvalidValue;
  count_launch();
  OAB_DISPATCH_IN(dtype, nf4_dequantize_kernel<T><<<grid_for(nc), kThreads, 0, st>>>(packed, absmax, nc, blocksize / 16, (T*)out));
  return cudaGetLastError();
}

// rows that fit the register-cached kernel (aligned, whole vectors) take it
#define OAB_INT8_LAUNCH(FAKE, Q, SC, OUT)                                                              \
  do {                                                                                                 \
    const bool fits = in_f % 16 == 0 && aligned32(x) && (FAKE ? aligned32(OUT) : ((reinterpret_cast<uintptr_t>(Q) & 15u) == 0)); \
    if (fits && in_f <= kThreads * 16)                                                                 \
      int8_quantize_cached_kernel<T, S, FAKE, 1><<<grid, kThreads, 0, st>>>((const T*)x, out_f, in_f, Q, SC, OUT); \
    else if (fits && in_f <= kThreads * 16 * 4)                                                        \
      int8_quantize_cached_kernel<T, S, FAKE, 4><<<grid, kThreads, 0, st>>>((const T*)x, out_f, in_f, Q, SC, OUT); \
    else                                                                                               \
      int8_quantize_kernel<T, S, FAKE><<<grid, kThreads, 0, st>>>((const T*)x, out_f, in_f, Q, SC, OUT); \
  } while (0)

cudaError_t launch_int8_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int8_t* q,
                                 void* scales, int scale_dtype, cudaStream_t st) {
  if (out_f <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)(out_f < (int64_t)kNumSMs * 16 ? out_f : (int64_t)kNumSMs * 16);
  count_launch();
  OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
      OAB_INT8_LAUNCH(false, q, (S*)scales, nullptr)));
  return cudaGetLastError();
}

cudaError_t launch_int8_dequantize(const int8_t* q, const void* scales, int scale_dtype, int64_t out_f,
                                   int64_t in_f, void* out, cudaStream_t st) {
  if (out_f <= 0) return cudaSuccess;
  count_launch();
  OAB_DISPATCH_SCALE(scale_dtype, int8_dequantize_kernel<S><<<grid_for((out_f * in_f + 15) / 16), kThreads, 0, st>>>(q, (const S*)scales, out_f, in_f, (S*)out));
  return cudaGetLastError();
}

cudaError_t launch_int4_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int group,
                                 int32_t* qweight, void* scales, int scale_dtype, cudaStream_t st) {
  if (out_f <= 0) return cudaSuccess;
  if (in_f % 128 != 0 || (group != 32 && group != 64 && group != 128)) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((out_f + 31) / 32), (unsigned)((in_f / 128 + kInt4QuantTiles - 1) / kInt4QuantTiles));
  count_launch();
  OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
      int4_quantize_kernel<T, S, kInt4QuantTiles><<<grid, kThreads, 0, st>>>((const T*)x, out_f, in_f, group, qweight, (S*)scales, aligned32(x) ? 1 : 0)));
  return cudaGetLastError();
}

cudaError_t launch_int4_dequantize(const int32_t* qweight, const void* scales, int scale_dtype, int64_t out_f,
                                   int64_t in_f, int group, void* out, cudaStream_t st) {
  if (out_f <= 0) return cudaSuccess;
  if (in_f % 128 != 0 || (group != 32 && group != 64 && group != 128)) return cudaErrorInvalidValue;
  // one CTA per band of 32 rows unless there are few bands: then the columns are split over grid.y
  const int64_t bands = (out_f + 31) / 32, spans = in_f / 64;
  int64_t gy = (kNumSMs * 4 + bands - 1) / bands;
  if (gy > (spans + 7) / 8) gy = (spans + 7) / 8;
  if (gy < 1) gy = 1;
  dim3 grid((unsigned)bands, (unsigned)gy);
  count_launch();
  OAB_DISPATCH_SCALE(scale_dtype, int4_dequantize_kernel<S><<<grid, kThreads, 0, st>>>(qweight, (const S*)scales, out_f, in_f, group, (S*)out, aligned32(out) ? 1 : 0));
  return cudaGetLastError();
}

// ------------------------------------------------------------------ fake quantization
cudaError_t launch_fake_quant(int format, const void* x, void* out, int dtype, int64_t out_f, int64_t in_f,
                              int group, int scale_dtype, const float* tensor_amax, cudaStream_t st) {
  const int64_t numel = out_f * in_f;
  if (numel <= 0) return cudaSuccess;
  count_launch();
  switch (format) {
    case kQNVFP4: {
      if (in_f % 16 != 0 || tensor_amax == nullptr || !aligned32(x) || !aligned32(out)) return cudaErrorInvalidValue;
      const int64_t nb = numel / 16;
      OAB_DISPATCH_IN(dtype, nvfp4_quantize_kernel<T, true><<<grid_for(nb), kThreads, 0, st>>>(
          (const T*)x, nb, tensor_amax, nullptr, nullptr, nullptr, 0, (T*)out));
      break;
    }
    case kQNF4: {
      if (group < 16 || group > 512 || (group & (group - 1)) || in_f % group != 0 || !aligned32(x) || !aligned32(out))
        return cudaErrorInvalidValue;
      const int64_t nc = numel / 16;
      OAB_DISPATCH_IN(dtype, nf4_quantize_kernel<T, true><<<grid_for(nc), kThreads, 0, st>>>(
          (const T*)x, nc, group / 16, nullptr, nullptr, (T*)out));
      break;
    }
    case kQInt4: {
      if ((group != 32 && group != 64 && group != 128) || in_f % group != 0 || !aligned32(x) || !aligned32(out))
        return cudaErrorInvalidValue;
      const int64_t nc = numel / 16;
      OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
          int4_fake_quant_kernel<T, S><<<grid_for(nc), kThreads, 0, st>>>((const T*)x, nc, group / 16, (T*)out)));
      break;
    }
    case kQInt8: {
      const unsigned grid = (unsigned)(out_f < (int64_t)kNumSMs * 16 ? out_f : (int64_t)kNumSMs * 16);
      OAB_DISPATCH_IN(dtype, OAB_DISPATCH_SCALE(scale_dtype,
          OAB_INT8_LAUNCH(true, nullptr, (S*)nullptr, (T*)out)));
      break;
    }
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace oab
