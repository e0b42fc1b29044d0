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
#include "adam_vec.cuh"

namespace oab {

unsigned long long g_launch_count = 0;

namespace {

using namespace vec;

template <int MODE, bool DECOUPLED, bool HAS_G2, bool PEERS, bool AMAX>
__global__ void __launch_bounds__(kThreads, PEERS ? ((MODE == kModeSR || AMAX) ? 1 : 2) : 3)
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
      const float a = compute_vec<MODE, DECOUPLED, HAS_G2 && !PEERS, AMAX>(r, vec, clip, s, seed, elem_offset);
      if (AMAX) amax = fmaxf(amax, a);
      store_vec<MODE, PEERS>(r, t, pr, vec);
    }
  }
  for (int64_t i = scalar_begin + tid; i < n; i += nthreads)
    amax = fmaxf(amax, scalar_element<MODE, DECOUPLED, PEERS>(t, i, HAS_G2, clip, s, seed, elem_offset, &pr));

  if (AMAX && amax_out != nullptr) {
    float bm = block_max<kThreads>(amax, red);
    if (threadIdx.x == 0 && bm > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax_out), __float_as_uint(bm));
  }
}

template <int MODE>
cudaError_t dispatch(const AdamStepArgs& a, const Ptrs& t, const Peers& pr, const AdamScalars& s,
                     int grid, int vector_ok, cudaStream_t st) {
#define OAB_LAUNCH2(DEC, G2, PE, AM)                                                           \
  adam_step_kernel<MODE, DEC, G2, PE, AM><<<grid, kThreads, 0, st>>>(                          \
      t, pr, a.n, s, a.clip_coef, a.seed, a.elem_offset, a.amax_out, vector_ok, a.abort_flag)
  // the running max of |master| only exists for fp32_master (it feeds the NVFP4 tensor scale)
#define OAB_LAUNCH(DEC, G2, PE)                                                                \
  do {                                                                                         \
    if (MODE == kModeFP32Master && a.amax_out != nullptr) OAB_LAUNCH2(DEC, G2, PE, (MODE == kModeFP32Master)); \
    else OAB_LAUNCH2(DEC, G2, PE, false);                                                      \
  } while (0)
  const bool peers = a.n_g_peers > 0 || a.n_p_peers > 0;
  if (peers) {
    if (a.decoupled) OAB_LAUNCH(true, false, true); else OAB_LAUNCH(false, false, true);
  } else if (a.decoupled) {
    if (a.g2) OAB_LAUNCH(true, true, false); else OAB_LAUNCH(true, false, false);
  } else {
    if (a.g2) OAB_LAUNCH(false, true, false); else OAB_LAUNCH(false, false, false);
  }
#undef OAB_LAUNCH2
#undef OAB_LAUNCH
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_adam_step(const AdamStepArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  if (a.mode != kModeFP32Master && a.p == nullptr) return cudaErrorInvalidValue;
  if (a.mode != kModeSR && a.extra == nullptr) return cudaErrorInvalidValue;
  if (a.amax_out != nullptr && a.mode != kModeFP32Master) return cudaErrorInvalidValue;
  if (a.extra_copy != nullptr && a.mode != kModeFP32Master) return cudaErrorInvalidValue;
  Ptrs t{(uint16_t*)a.p, (const uint16_t*)a.g, (const uint16_t*)a.g2,
         (uint16_t*)a.m, (uint16_t*)a.v, a.extra, a.extra_copy};
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
  int vector_ok = al(a.p) && al(t.g) && al(t.g2) && al(a.m) && al(a.v) && al(a.extra) && al(a.extra_copy) &&
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
  Ptrs t{(uint16_t*)e.p, (const uint16_t*)e.g, nullptr, (uint16_t*)e.m, (uint16_t*)e.v, e.extra, nullptr};
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
