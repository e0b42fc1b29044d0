// Step of a quantized weight in one pass (sm_100a): Adam on the fp32 master, weight-only
// re-quantization of the updated rows, and the store of the packed rows into every
// replica of the weight, the local one and, through NVLink peer mappings, the other
// ranks'.
//
// The reference steps the master, all-gathers the fp32 master of every rank
// (4 bytes per element on the wire) and lets every rank re-quantize the whole weight
// (reference: src/offload_adam/distributed_offload_adam.py:250-262; on one GPU
// src/offload_adam/offload_adam.py:421-444 runs the step kernel and then a separate
// quantize kernel over a master that has to be resident as a whole).  Here the owner of
// a row range quantizes its rows while they are still in registers (or in shared
// memory, for the formats whose statistics span more than a thread) and only packed
// bytes and scales cross NVLink: 0.5 to 1 byte per element.  With one replica the same
// kernels serve a single GPU, chunk by chunk through the staging buffer.
//
// Formats and their statistics:
//   NF4    block of 16..512 columns  -> 1..32 lanes of a warp, shuffle reduction
//   int4   group of 32/64/128 columns, transposed GPTQ payload -> 32 x 128 tile in
//          shared memory, 128-byte stores along out_f
//   int8   whole row -> one CTA per row, the updated row parked in shared memory
//   NVFP4  whole tensor (and across ranks) -> cannot be fused with the update; the
//          step kernel leaves max|master| and a device copy of the master, and
//          nvfp4_quantize_push_kernel runs once the maximum is known
#include "adam_quant.h"
#include "adam_vec.cuh"
#include "quant_math.cuh"

namespace oab {
namespace {

using namespace vec;
using namespace qm;

constexpr int M = kModeFP32Master;

struct Replicas {
  uint8_t* p0[kMaxPeers];
  uint8_t* p1[kMaxPeers];
  int n;
  int group;
  int64_t out_f, in_f, row0;
};

__device__ __forceinline__ void master_of(const VecRegs<M>& r, float (&e)[16]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { e[i] = __uint_as_float(r.e0.w[i]); e[8 + i] = __uint_as_float(r.e1.w[i]); }
}
__device__ __forceinline__ void zero16(float (&e)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) e[i] = 0.f;
}

// Adam on 16 elements; leaves the new moments and master in memory and the master in e.
template <bool DECOUPLED, bool HAS_G2, bool PULL>
__device__ __forceinline__ void step16(const Ptrs& t, const Peers& pr, int64_t vec, float clip,
                                       const AdamScalars& s, float (&e)[16]) {
  VecRegs<M> r;
  load_vec<M, HAS_G2, PULL>(r, t, pr, vec);
  compute_vec<M, DECOUPLED, HAS_G2 && !PULL, false>(r, vec, clip, s, 0, 0);
  store_vec<M, false, false>(r, t, pr, vec);
  master_of(r, e);
}

// ------------------------------------------------------------------------- NF4
template <bool DECOUPLED, bool HAS_G2, bool PULL>
__global__ void __launch_bounds__(kThreads, 2)
adam_nf4_push_kernel(Ptrs t, Peers pr, int64_t n, AdamScalars s, const float* __restrict__ clip_ptr,
                     const int* abort_flag, Replicas q) {
  __shared__ float lut[16];
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  if (threadIdx.x < 16) lut[threadIdx.x] = kNF4[threadIdx.x];
  __syncthreads();
  const float clip = clip_ptr ? *clip_ptr : 1.0f;
  const int lanes = q.group >> 4;
  const int64_t nvec = n >> 4;
  const int64_t total = (nvec + 31) / 32 * 32;  // whole warps: every shuffle has its partners
  const int64_t g0 = q.row0 * q.in_f;           // element index of this launch's first element
  for (int64_t vec = (int64_t)blockIdx.x * kThreads + threadIdx.x; vec < total; vec += (int64_t)gridDim.x * kThreads) {
    float e[16];
    const bool live = vec < nvec;
    if (live) step16<DECOUPLED, HAS_G2, PULL>(t, pr, vec, clip, s, e);
    else zero16(e);
    const float am = group_max(amax16(e), lanes);
    if (!live) continue;
    uint32_t w0, w1;
    nf4_pack16(e, rcp_rn(fmaxf(am, kEps)), lut, w0, w1);
    const int64_t g = g0 + vec * 16;
    const bool first = (vec % lanes) == 0;
#pragma unroll
    for (int j = 0; j < kMaxPeers; ++j)
      if (j < q.n) {
        *reinterpret_cast<uint2*>(q.p0[j] + (g >> 1)) = make_uint2(w0, w1);
        if (first) reinterpret_cast<float*>(q.p1[j])[g / q.group] = am;
      }
  }
}

// ------------------------------------------------------------------------ int8
// One CTA per row.  The updated row waits in shared memory (element k of vector v at
// k * nvec + v: consecutive threads touch consecutive words) until its maximum is known.
template <typename S, bool DECOUPLED, bool HAS_G2, bool PULL>
__global__ void __launch_bounds__(kThreads, 2)
adam_int8_push_kernel(Ptrs t, Peers pr, int64_t rows, AdamScalars s, const float* __restrict__ clip_ptr,
                      const int* abort_flag, Replicas q) {
  extern __shared__ float rowbuf[];
  __shared__ float red[kThreads / 32];
  __shared__ float s_inv;
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  const float clip = clip_ptr ? *clip_ptr : 1.0f;
  const int nvec = (int)(q.in_f >> 4);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float m = 0.f;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float e[16];
      step16<DECOUPLED, HAS_G2, PULL>(t, pr, row * nvec + v, clip, s, e);
#pragma unroll
      for (int k = 0; k < 16; ++k) rowbuf[k * nvec + v] = e[k];
      m = fmaxf(m, amax16(e));
    }
    const float bm = block_max<kThreads>(m, red);
    const int64_t grow = q.row0 + row;
    if (threadIdx.x == 0) {
      const float scale = __fdiv_rn(bm, 127.0f);
      s_inv = rcp_rn(fmaxf(scale, kEps));
      for (int j = 0; j < q.n; ++j) reinterpret_cast<S*>(q.p1[j])[grow] = Elem<S>::from_f32(scale);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float e[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) e[k] = rowbuf[k * nvec + v];
      const uint4 w = int8_pack16(e, inv);
#pragma unroll
      for (int j = 0; j < kMaxPeers; ++j)
        if (j < q.n) *reinterpret_cast<uint4*>(q.p0[j] + grow * q.in_f + (int64_t)v * 16) = w;
    }
    __syncthreads();  // rowbuf and s_inv are rewritten for the next row
  }
}

// ------------------------------------------------------------------------ int4
// One CTA per 32 x 128 tile of the rows of this launch (see Int4Tile).
template <typename S, bool DECOUPLED, bool HAS_G2, bool PULL>
__global__ void __launch_bounds__(kThreads, 2)
adam_int4_push_kernel(Ptrs t, Peers pr, int64_t rows, AdamScalars s, const float* __restrict__ clip_ptr,
                      const int* abort_flag, Replicas q) {
  __shared__ Int4Tile sm;
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  const float clip = clip_ptr ? *clip_ptr : 1.0f;
  const int64_t tiles_per_band = q.in_f >> 7;
  const int64_t ntiles = ((rows + 31) >> 5) * tiles_per_band;
  const int lr = threadIdx.x >> 3, seg = threadIdx.x & 7;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t band = tile / tiles_per_band, col0 = (tile % tiles_per_band) << 7;
    const int64_t row = band * 32 + lr;
    float e[16];
    if (row < rows) step16<DECOUPLED, HAS_G2, PULL>(t, pr, (row * q.in_f + col0 + seg * 16) >> 4, clip, s, e);
    else zero16(e);
    int4_tile_quantize(e, q.group, sm);
    __syncthreads();
    const int64_t left = rows - band * 32;
    const int valid = left < 32 ? (int)left : 32;
    int4_tile_store_multi<S, kMaxPeers>(sm, q.out_f, q.row0 + band * 32, valid, col0, q.group, q.p0, q.p1, q.n);
    __syncthreads();
  }
}

// ----------------------------------------------------------------------- NVFP4
// Second pass of an NVFP4 step: the master copy the step kernel left on the device is
// quantized with the now known tensor scale and stored into every replica.
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_push_kernel(const float* x, int64_t nblocks, const float* amax, float* global_scale_out,
                           int scale_words_ok, const int* abort_flag, Replicas q) {
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  float global, inv_global;
  nvfp4_global(*amax, global, inv_global);
  if (global_scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *global_scale_out = global;
  const int lane = threadIdx.x & 31;
  const int64_t b0 = (q.row0 * q.in_f) >> 4;  // block index of this launch's first block
  for (int64_t base = (int64_t)blockIdx.x * kThreads + (threadIdx.x & ~31); base < nblocks;
       base += (int64_t)gridDim.x * kThreads) {
    const int64_t b = base + lane;
    const bool live = b < nblocks;
    uint8_t s8 = 0;
    uint32_t w0 = 0, w1 = 0;
    if (live) {
      float e[16];
      Elem<float>::load16(x + b * 16, e);
      nvfp4_pack16(e, global, inv_global, s8, w0, w1);
    }
    uint32_t s32 = s8;
    s32 |= __shfl_down_sync(0xffffffffu, (uint32_t)s8, 1) << 8;
    s32 |= __shfl_down_sync(0xffffffffu, s32, 2) << 16;
    if (!live) continue;
    const bool word = scale_words_ok && b + 3 < nblocks;
#pragma unroll
    for (int j = 0; j < kMaxPeers; ++j)
      if (j < q.n) {
        *reinterpret_cast<uint2*>(q.p0[j] + (b0 + b) * 8) = make_uint2(w0, w1);
        if (word) {
          if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(q.p1[j] + b0 + b) = s32;
        } else {
          q.p1[j][b0 + b] = s8;
        }
      }
  }
}

Replicas make_replicas(const QuantPushArgs& q) {
  Replicas r;
  r.n = q.n_replicas;
  r.group = q.group;
  r.out_f = q.out_f;
  r.in_f = q.in_f;
  r.row0 = q.row0;
  for (int j = 0; j < kMaxPeers; ++j) {
    r.p0[j] = static_cast<uint8_t*>(q.payload0[j < q.n_replicas ? j : 0]);
    r.p1[j] = static_cast<uint8_t*>(q.payload1[j < q.n_replicas ? j : 0]);
  }
  return r;
}

bool al(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

constexpr int64_t kInt8MaxInF = 48 * 1024;  // the row lives in shared memory: 4 bytes per column

}  // namespace

bool adam_quant_supported(int format, int64_t in_f, int group) {
  switch (format) {
    case kQNF4: return group >= 16 && group <= 512 && (group & (group - 1)) == 0 && in_f % group == 0;
    case kQInt4: return (group == 32 || group == 64 || group == 128) && in_f % 128 == 0;
    case kQInt8: return in_f % 16 == 0 && in_f <= kInt8MaxInF;
    case kQNVFP4: return in_f % 16 == 0;
    default: return false;
  }
}

cudaError_t launch_adam_quant_push(const AdamStepArgs& a, const QuantPushArgs& q, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  if (a.mode != kModeFP32Master || a.extra == nullptr) return cudaErrorInvalidValue;
  if (q.format == kQNVFP4 || !adam_quant_supported(q.format, q.in_f, q.group)) return cudaErrorInvalidValue;
  if (q.n_replicas < 1 || q.n_replicas > kMaxPeers || a.n % q.in_f != 0) return cudaErrorInvalidValue;
  if (a.n_g_peers > kMaxPeers || (a.n_g_peers == 0 && a.g == nullptr)) return cudaErrorInvalidValue;
  const int64_t rows = a.n / q.in_f;
  if (q.row0 < 0 || q.row0 + rows > q.out_f) return cudaErrorInvalidValue;

  Ptrs t{nullptr, (const uint16_t*)a.g, (const uint16_t*)a.g2, (uint16_t*)a.m, (uint16_t*)a.v, a.extra, a.extra_copy};
  Peers pr;
  pr.n_g = a.n_g_peers;
  pr.n_p = 0;
  pr.g_scale = a.g_scale;
  for (int j = 0; j < kMaxPeers; ++j) {
    pr.g[j] = (const uint16_t*)a.g_peers[j];
    pr.p[j] = nullptr;
  }
  if (a.n_g_peers > 0) { t.g = pr.g[0]; t.g2 = nullptr; }
  // the vector path is the only path: whole rows of a weight whose in_f is a multiple of 16
  bool ok = al(t.g, 32) && al(t.g2, 32) && al(a.m, 32) && al(a.v, 32) && al(a.extra, 32) && al(a.extra_copy, 32);
  for (int j = 0; j < a.n_g_peers; ++j) ok = ok && al(a.g_peers[j], 32);
  for (int j = 0; j < q.n_replicas; ++j)
    ok = ok && q.payload0[j] != nullptr && q.payload1[j] != nullptr && al(q.payload0[j], 16) && al(q.payload1[j], 4);
  if (!ok) return cudaErrorInvalidValue;

  AdamScalars s;
  s.lr = a.lr;
  s.wd = a.wd;
  s.lr_wd = a.lr * a.wd;
  s.one_m_b1h = 1.0f - a.beta1_hat;
  s.one_m_b2h = 1.0f - a.beta2_hat;
  s.eps = a.eps;
  const Replicas r = make_replicas(q);
  const bool pull = a.n_g_peers > 0, g2 = !pull && a.g2 != nullptr;
  const int cap = a.max_ctas > 0 ? a.max_ctas : kNumSMs * 8;
  auto grid_of = [&](int64_t want) { return (int)(want < 1 ? 1 : (want > cap ? cap : want)); };
  count_launch();

#define OAB_VARIANTS(KERNEL, GRID, SMEM, COUNT)                                                     \
  do {                                                                                              \
    if (pull) {                                                                                     \
      if (a.decoupled) KERNEL(true, false, true, GRID, SMEM, COUNT); else KERNEL(false, false, true, GRID, SMEM, COUNT); \
    } else if (g2) {                                                                                \
      if (a.decoupled) KERNEL(true, true, false, GRID, SMEM, COUNT); else KERNEL(false, true, false, GRID, SMEM, COUNT); \
    } else {                                                                                        \
      if (a.decoupled) KERNEL(true, false, false, GRID, SMEM, COUNT); else KERNEL(false, false, false, GRID, SMEM, COUNT); \
    }                                                                                               \
  } while (0)

  if (q.format == kQNF4) {
#define OAB_NF4(DEC, G2, PULL, GRID, SMEM, COUNT)                                                   \
  adam_nf4_push_kernel<DEC, G2, PULL><<<GRID, kThreads, 0, stream>>>(t, pr, COUNT, s, a.clip_coef, a.abort_flag, r)
    const int grid = grid_of(((a.n >> 4) + kThreads - 1) / kThreads);
    OAB_VARIANTS(OAB_NF4, grid, 0, a.n);
#undef OAB_NF4
    return cudaGetLastError();
  }

  auto with_scale = [&](auto launch) -> cudaError_t {
    switch (q.scale_dtype) {
      case kF32: return launch(float{});
      case kBF16: return launch(__nv_bfloat16{});
      case kF16: return launch(__half{});
      default: return cudaErrorInvalidValue;
    }
  };

  if (q.format == kQInt8) {
    const size_t smem = (size_t)q.in_f * sizeof(float);
    const int grid = grid_of(rows);
    return with_scale([&](auto tag) -> cudaError_t {
      using S = decltype(tag);
#define OAB_INT8(DEC, G2, PULL, GRID, SMEM, COUNT)                                                  \
  do {                                                                                              \
    auto kern = adam_int8_push_kernel<S, DEC, G2, PULL>;                                            \
    if (SMEM > 48 * 1024) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); \
      if (e != cudaSuccess) return e;                                                               \
    }                                                                                               \
    kern<<<GRID, kThreads, SMEM, stream>>>(t, pr, COUNT, s, a.clip_coef, a.abort_flag, r);          \
  } while (0)
      OAB_VARIANTS(OAB_INT8, grid, smem, rows);
#undef OAB_INT8
      return cudaGetLastError();
    });
  }

  if (q.format == kQInt4) {
    const int grid = grid_of(((rows + 31) / 32) * (q.in_f / 128));
    return with_scale([&](auto tag) -> cudaError_t {
      using S = decltype(tag);
#define OAB_INT4(DEC, G2, PULL, GRID, SMEM, COUNT)                                                  \
  adam_int4_push_kernel<S, DEC, G2, PULL><<<GRID, kThreads, 0, stream>>>(t, pr, COUNT, s, a.clip_coef, a.abort_flag, r)
      OAB_VARIANTS(OAB_INT4, grid, 0, rows);
#undef OAB_INT4
      return cudaGetLastError();
    });
  }
#undef OAB_VARIANTS
  return cudaErrorInvalidValue;
}

cudaError_t launch_nvfp4_quantize_push(const float* master, int64_t n, const QuantPushArgs& q,
                                       const int* abort_flag, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (q.format != kQNVFP4 || q.in_f % 16 != 0 || n % q.in_f != 0 || q.tensor_amax == nullptr) return cudaErrorInvalidValue;
  if (q.n_replicas < 1 || q.n_replicas > kMaxPeers || !al(master, 32)) return cudaErrorInvalidValue;
  if (q.row0 < 0 || q.row0 + n / q.in_f > q.out_f) return cudaErrorInvalidValue;
  const int64_t b0 = (q.row0 * q.in_f) >> 4;
  int words_ok = (b0 & 3) == 0;
  for (int j = 0; j < q.n_replicas; ++j) {
    if (q.payload0[j] == nullptr || q.payload1[j] == nullptr || !al(q.payload0[j], 8)) return cudaErrorInvalidValue;
    words_ok = words_ok && al(q.payload1[j], 4);
  }
  const Replicas r = make_replicas(q);
  const int64_t nb = n >> 4;
  const int64_t want = (nb + kThreads - 1) / kThreads;
  const int grid = (int)(want > kNumSMs * 8 ? kNumSMs * 8 : want);
  count_launch();
  nvfp4_quantize_push_kernel<<<grid, kThreads, 0, stream>>>(master, nb, q.tensor_amax, q.global_scale_out,
                                                            words_ok, abort_flag, r);
  return cudaGetLastError();
}

}  // namespace oab
