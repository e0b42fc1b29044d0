// Fused Adam/AdamW step kernels for sm_100a.
//
// One kernel template covers the four parameter-precision schemes of the
// reference optimizer (reference: src/offload_adam/kernels/*.py) and folds in
// the work the reference does in separate passes around its step kernel:
//   * the clip coefficient is read from a device scalar and applied in fp32
//     (reference: grad.mul_(clip_coef), src/offload_adam/offload_adam.py:451);
//   * an optional second gradient term is added and rounded to bf16 exactly as
//     an in-place bf16 `add_` would (reference: offload_adam.py:398), so the
//     accumulated host gradient never has to be materialised on the device;
//   * an optional running max of |master| feeds the NVFP4 tensor scale.
//
// The kernel is a grid-stride stream over groups of 16 elements.  Every operand
// moves with Blackwell's 256-bit global loads/stores (one 32-byte request per
// bf16 stream, two for the fp32 master), all issued before the first use, so a
// thread keeps 160-224 bytes in flight and a warp request always covers whole,
// contiguous 1 KiB runs; that is what both HBM3e and a PCIe link (when operands
// are mapped host memory) need to stay busy.
#include "adam_math.cuh"
#include "adam_step.h"

namespace oab {

unsigned long long g_launch_count = 0;

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 16;  // elements per thread per iteration (one 32-byte bf16 vector)

struct Ptrs {
  uint16_t* p;
  const uint16_t* g;
  const uint16_t* g2;
  uint16_t* m;
  uint16_t* v;
  void* extra;
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

// One element.  p16/e16/master are in/out depending on MODE.
template <int MODE, bool DECOUPLED>
__device__ __forceinline__ float element_step(uint32_t& p16, uint32_t g16, bool has_g2,
                                              uint32_t g2_16, uint32_t& m16, uint32_t& v16,
                                              float& master, int16_t& err, float clip,
                                              const AdamScalars& s, uint32_t rand16) {
  float g = bf16_bits_to_f32(g16);
  if (has_g2) {
    g = bf16_bits_to_f32(f32_to_bf16_rne_bits(__fadd_rn(g, bf16_bits_to_f32(g2_16))));
  }
  g = __fmul_rn(g, clip);
  float m = bf16_bits_to_f32(m16);
  float v = bf16_bits_to_f32(v16);
  float p;
  if (MODE == kModeSR) p = bf16_bits_to_f32(p16);
  else if (MODE == kModeFP32Master) p = master;
  else if (MODE == kModeFP31) p = fp31_reconstruct(p16, err);
  else p = custom_reconstruct(p16, err);

  adam_math<DECOUPLED>(p, g, m, v, s);

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

template <int MODE, bool DECOUPLED, bool HAS_G2, bool PEERS>
__device__ __forceinline__ float compute_store_vec(VecRegs<MODE>& r, const Ptrs& t, const Peers& pr,
                                                   int64_t vec, float clip, const AdamScalars& s,
                                                   uint64_t seed, int64_t elem_offset) {
  const int64_t e = vec * kVec;
  Philox4 rnd[2];
  if (MODE == kModeSR) {
    const uint64_t c = (uint64_t)((elem_offset + e) >> 3);
    rnd[0] = philox4x32_10(c, seed);
    rnd[1] = philox4x32_10(c + 1, seed);
  }
  V8 pout = r.p;
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    uint32_t p16 = (MODE != kModeFP32Master) ? half_of(r.p, j) : 0u;
    uint32_t m16 = half_of(r.m, j), v16 = half_of(r.v, j);
    float master = 0.f;
    int16_t err = 0;
    if (MODE == kModeFP32Master) master = __uint_as_float(j < 8 ? r.e0.w[j & 7] : r.e1.w[j & 7]);
    if (MODE == kModeFP31 || MODE == kModeCustom) err = (int16_t)half_of(r.e0, j);
    uint32_t rand16 = (MODE == kModeSR) ? philox_word16(rnd[j >> 3], j & 7) : 0u;
    float pf = element_step<MODE, DECOUPLED>(p16, half_of(r.g, j), HAS_G2,
                                             HAS_G2 ? half_of(r.g2, j) : 0u, m16, v16, master,
                                             err, clip, s, rand16);
    amax = fmaxf(amax, fabsf(pf));
    set_half(pout, j, p16);
    set_half(r.m, j, m16);
    set_half(r.v, j, v16);
    if (MODE == kModeFP32Master) {
      if (j < 8) r.e0.w[j & 7] = __float_as_uint(master); else r.e1.w[j & 7] = __float_as_uint(master);
    }
    if (MODE == kModeFP31 || MODE == kModeCustom) set_half(r.e0, j, (uint32_t)(uint16_t)err);
  }
  if (PEERS && pr.n_p > 0) {
    // push the new rows into every replica (all-gather folded into the update)
#pragma unroll
    for (int j = 0; j < kMaxPeers; ++j)
      if (j < pr.n_p) st32(pr.p[j] + e, pout);
  } else if (t.p != nullptr) {
    st32(t.p + e, pout);
  }
  st32_stream(t.m + e, r.m);
  st32_stream(t.v + e, r.v);
  if (MODE == kModeFP32Master) {
    float* mp = reinterpret_cast<float*>(t.extra) + e;
    st32_stream(mp, r.e0);
    st32_stream(mp + 8, r.e1);
  } else if (MODE == kModeFP31 || MODE == kModeCustom) {
    st32_stream(reinterpret_cast<int16_t*>(t.extra) + e, r.e0);
  }
  return amax;
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
  if (MODE == kModeFP32Master) reinterpret_cast<float*>(t.extra)[i] = master;
  if (MODE == kModeFP31 || MODE == kModeCustom) reinterpret_cast<int16_t*>(t.extra)[i] = err;
  return fabsf(pf);
}

template <int MODE, bool DECOUPLED, bool HAS_G2, bool PEERS>
__global__ void __launch_bounds__(kThreads)
adam_step_kernel(Ptrs t, Peers pr, int64_t n, AdamScalars s, const float* __restrict__ clip_ptr,
                 uint64_t seed, int64_t elem_offset, float* amax_out, int vector_ok,
                 const int* abort_flag) {
  __shared__ float red[kThreads / 32];
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  const float clip = clip_ptr ? *clip_ptr : 1.0f;
  float amax = 0.f;
  const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * kThreads;
  int64_t scalar_begin = 0;
  if (vector_ok) {
    const int64_t nvec = n / kVec;
    scalar_begin = nvec * kVec;
    for (int64_t vec = tid; vec < nvec; vec += nthreads) {
      VecRegs<MODE> r;
      load_vec<MODE, HAS_G2, PEERS>(r, t, pr, vec);
      amax = fmaxf(amax, compute_store_vec<MODE, DECOUPLED, HAS_G2, PEERS>(r, t, pr, vec, clip, s,
                                                                           seed, elem_offset));
    }
  }
  for (int64_t i = scalar_begin + tid; i < n; i += nthreads)
    amax = fmaxf(amax, scalar_element<MODE, DECOUPLED, PEERS>(t, i, HAS_G2, clip, s, seed, elem_offset, &pr));

  if (amax_out != nullptr) {
    float bm = block_max<kThreads>(amax, red);
    if (threadIdx.x == 0 && bm > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax_out), __float_as_uint(bm));
  }
}

template <int MODE>
cudaError_t dispatch(const AdamStepArgs& a, const Ptrs& t, const Peers& pr, const AdamScalars& s,
                     int grid, int vector_ok, cudaStream_t st) {
#define OAB_LAUNCH(DEC, G2, PE)                                                                \
  adam_step_kernel<MODE, DEC, G2, PE><<<grid, kThreads, 0, st>>>(                              \
      t, pr, a.n, s, a.clip_coef, a.seed, a.elem_offset, a.amax_out, vector_ok, a.abort_flag)
  const bool peers = a.n_g_peers > 0 || a.n_p_peers > 0;
  if (peers) {
    if (a.decoupled) OAB_LAUNCH(true, false, true); else OAB_LAUNCH(false, false, true);
  } else if (a.decoupled) {
    if (a.g2) OAB_LAUNCH(true, true, false); else OAB_LAUNCH(true, false, false);
  } else {
    if (a.g2) OAB_LAUNCH(false, true, false); else OAB_LAUNCH(false, false, false);
  }
#undef OAB_LAUNCH
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_adam_step(const AdamStepArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  if (a.mode != kModeFP32Master && a.p == nullptr) return cudaErrorInvalidValue;
  if (a.mode != kModeSR && a.extra == nullptr) return cudaErrorInvalidValue;
  Ptrs t{(uint16_t*)a.p, (const uint16_t*)a.g, (const uint16_t*)a.g2,
         (uint16_t*)a.m, (uint16_t*)a.v, a.extra};
  if (a.n_g_peers > kMaxPeers || a.n_p_peers > kMaxPeers) return cudaErrorInvalidValue;
  if (a.n_g_peers == 0 && a.g == nullptr) return cudaErrorInvalidValue;
  Peers pr;
  pr.n_g = a.n_g_peers;
  pr.n_p = a.n_p_peers;
  pr.g_scale = a.g_scale;
  for (int j = 0; j < kMaxPeers; ++j) {
    pr.g[j] = (const uint16_t*)a.g_peers[j];
    pr.p[j] = (uint16_t*)a.p_peers[j];
  }
  // with a pulled gradient the local `g` is unused; point it somewhere valid
  if (a.n_g_peers > 0) { t.g = pr.g[0]; t.g2 = nullptr; }
  AdamScalars s;
  s.lr = a.lr;
  s.wd = a.wd;
  s.lr_wd = a.lr * a.wd;  // fp32 product, same as the device's __fmul_rn
  s.one_m_b1h = 1.0f - a.beta1_hat;
  s.one_m_b2h = 1.0f - a.beta2_hat;
  s.eps = a.eps;
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  int vector_ok = al(a.p) && al(t.g) && al(t.g2) && al(a.m) && al(a.v) && al(a.extra) &&
                  ((a.elem_offset & 7) == 0);
  for (int j = 0; j < a.n_g_peers; ++j) vector_ok = vector_ok && al(a.g_peers[j]);
  for (int j = 0; j < a.n_p_peers; ++j) vector_ok = vector_ok && al(a.p_peers[j]);
  const int64_t nvec = (a.n + kVec - 1) / kVec;
  int64_t want = (nvec + kThreads - 1) / kThreads;
  int cap = a.max_ctas > 0 ? a.max_ctas : kNumSMs * 8;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  count_launch();
  switch (a.mode) {
    case kModeSR: return dispatch<kModeSR>(a, t, pr, s, grid, vector_ok, stream);
    case kModeFP32Master: return dispatch<kModeFP32Master>(a, t, pr, s, grid, vector_ok, stream);
    case kModeFP31: return dispatch<kModeFP31>(a, t, pr, s, grid, vector_ok, stream);
    case kModeCustom: return dispatch<kModeCustom>(a, t, pr, s, grid, vector_ok, stream);
    default: return cudaErrorInvalidValue;
  }
}

// ----------------------------------------------------------------------------
// Multi-tensor variant: one launch updates every small (GPU-resident) tensor.
// block_map[b] = {tensor index, chunk index}; each block handles kChunk elements.
// (reference: the per-parameter loop of OffloadAdam._step_inplace,
//  src/offload_adam/offload_adam.py:456-467, one kernel + one zero_ per tensor)
// ----------------------------------------------------------------------------
namespace {
constexpr int kChunk = 8192;

template <int MODE, bool DECOUPLED>
__global__ void __launch_bounds__(kThreads)
multi_tensor_adam_kernel(const MultiTensorEntry* __restrict__ table,
                         const int2* __restrict__ block_map, AdamScalars s,
                         const float* __restrict__ clip_ptr, uint64_t seed, int zero_grad) {
  const int2 bm = block_map[blockIdx.x];
  const MultiTensorEntry e = table[bm.x];
  const float clip = clip_ptr ? *clip_ptr : 1.0f;
  Ptrs t{(uint16_t*)e.p, (const uint16_t*)e.g, nullptr, (uint16_t*)e.m, (uint16_t*)e.v, e.extra};
  const int64_t begin = (int64_t)bm.y * kChunk;
  int64_t end = begin + kChunk;
  if (end > e.n) end = e.n;
  for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
    scalar_element<MODE, DECOUPLED>(t, i, false, clip, s, seed, e.elem_offset);
    if (zero_grad) const_cast<uint16_t*>(t.g)[i] = 0;
  }
}
}  // namespace

cudaError_t launch_multi_tensor_adam(const MultiTensorEntry* dev_table, int n_tensors,
                                     const int2* dev_block_map, int n_blocks, int mode,
                                     bool decoupled, float lr, float wd, float beta1_hat,
                                     float beta2_hat, float eps, const float* clip_coef,
                                     uint64_t seed, bool zero_grad, cudaStream_t stream) {
  if (n_blocks <= 0 || n_tensors <= 0) return cudaSuccess;
  AdamScalars s;
  s.lr = lr; s.wd = wd; s.lr_wd = lr * wd;
  s.one_m_b1h = 1.0f - beta1_hat; s.one_m_b2h = 1.0f - beta2_hat; s.eps = eps;
  count_launch();
#define OAB_MT(M)                                                                              \
  if (decoupled)                                                                               \
    multi_tensor_adam_kernel<M, true><<<n_blocks, kThreads, 0, stream>>>(                      \
        dev_table, dev_block_map, s, clip_coef, seed, zero_grad ? 1 : 0);                      \
  else                                                                                         \
    multi_tensor_adam_kernel<M, false><<<n_blocks, kThreads, 0, stream>>>(                     \
        dev_table, dev_block_map, s, clip_coef, seed, zero_grad ? 1 : 0)
  switch (mode) {
    case kModeSR: OAB_MT(kModeSR); break;
    case kModeFP32Master: OAB_MT(kModeFP32Master); break;
    case kModeFP31: OAB_MT(kModeFP31); break;
    case kModeCustom: OAB_MT(kModeCustom); break;
    default: return cudaErrorInvalidValue;
  }
#undef OAB_MT
  return cudaGetLastError();
}

int multi_tensor_chunk() { return kChunk; }

}  // namespace oab
