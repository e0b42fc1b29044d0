// Gradient kernels for sm_100a: bf16 accumulate fused with the squared-L2-norm
// reduction, and the clip-coefficient finalisation.
//
// They replace three separate library passes of the reference optimizer
// (reference: src/offload_adam/offload_adam.py:398 `device_grad.add_(p.grad)`,
// :505 `torch.norm(grad, 2.0)` and :555-561 stack + vector_norm + clamp).  The
// norm is accumulated in fp32 from the bf16-rounded sums, i.e. from exactly the
// values a later step will consume.
#include "common.cuh"
#include "grad_ops.h"

namespace oab {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sq_acc_pair(uint32_t w, float acc) {
  float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
  acc = __fadd_rn(acc, __fmul_rn(lo, lo));
  acc = __fadd_rn(acc, __fmul_rn(hi, hi));
  return acc;
}
__device__ __forceinline__ uint32_t add_pair(uint32_t a, uint32_t b) {
  float lo = __fadd_rn(__uint_as_float(a << 16), __uint_as_float(b << 16));
  float hi = __fadd_rn(__uint_as_float(a & 0xffff0000u), __uint_as_float(b & 0xffff0000u));
  return f32_to_bf16_rne_bits(lo) | (f32_to_bf16_rne_bits(hi) << 16);
}

template <bool HAS_B, bool STORE, bool SUMSQ>
__global__ void __launch_bounds__(kThreads)
grad_accumulate_kernel(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n,
                       float* sumsq_out, int accumulate, float* scratch, int vector_ok) {
  __shared__ float red[kThreads / 32];
  __shared__ int is_last;
  float acc = 0.f;
  const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * kThreads;
  int64_t scalar_begin = 0;
  if (vector_ok) {
    const int64_t nvec = n >> 4;
    scalar_begin = nvec << 4;
    for (int64_t base = tid; base < nvec; base += 2 * nthreads) {
      V8 ra[2], rb[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        int64_t vec = base + u * nthreads;
        if (vec < nvec) {
          ra[u] = ld32_stream(a + vec * 16);
          if (HAS_B) rb[u] = ld32_stream(b + vec * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        int64_t vec = base + u * nthreads;
        if (vec < nvec) {
          V8 r = ra[u];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (HAS_B) r.w[j] = add_pair(r.w[j], rb[u].w[j]);
            if (SUMSQ) acc = sq_acc_pair(r.w[j], acc);
          }
          if (STORE) st32_stream(out + vec * 16, r);
        }
      }
    }
  }
  for (int64_t i = scalar_begin + tid; i < n; i += nthreads) {
    uint32_t r = a[i];
    if (HAS_B) r = f32_to_bf16_rne_bits(__fadd_rn(bf16_bits_to_f32(r), bf16_bits_to_f32(b[i])));
    if (SUMSQ) { float f = bf16_bits_to_f32(r); acc = __fadd_rn(acc, __fmul_rn(f, f)); }
    if (STORE) out[i] = (uint16_t)r;
  }
  if (!SUMSQ) return;

  grid_sum_to<kThreads>(acc, red, &is_last, scratch, sumsq_out, accumulate != 0);
}

__global__ void __launch_bounds__(kThreads)
clip_finalize_kernel(const float* __restrict__ slots, const int* __restrict__ index, int n,
                     const float* __restrict__ extra_sq, float max_norm, float* coef_norm,
                     float* total_sq_out) {
  __shared__ float red[kThreads / 32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += kThreads) s += slots[index ? index[i] : i];
  float total = block_sum<kThreads>(s, red);
  if (threadIdx.x == 0) {
    if (extra_sq) total += *extra_sq;
    if (total_sq_out) *total_sq_out = total;
    if (coef_norm) {
      float norm = __fsqrt_rn(total);
      float coef = __fdiv_rn(max_norm, __fadd_rn(norm, 1e-6f));
      coef_norm[0] = coef > 1.0f ? 1.0f : coef;
      coef_norm[1] = norm;
    }
  }
}

}  // namespace

cudaError_t launch_grad_accumulate(const AccumArgs& a, cudaStream_t stream) {
  if (a.n <= 0) {
    if (a.sumsq_out && !a.sumsq_accumulate) return cudaMemsetAsync(a.sumsq_out, 0, sizeof(float), stream);
    return cudaSuccess;
  }
  if (a.sumsq_out && !a.scratch) return cudaErrorInvalidValue;
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  int vector_ok = al(a.out) && al(a.a) && al(a.b);
  const int64_t nvec = (a.n + 15) / 16;
  int64_t want = (nvec + kThreads * 2 - 1) / (kThreads * 2);
  int cap = a.max_ctas > 0 ? (a.max_ctas < kMaxPartials ? a.max_ctas : kMaxPartials) : kMaxPartials;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  count_launch();
  uint16_t* o = (uint16_t*)a.out;
  const uint16_t* pa = (const uint16_t*)a.a;
  const uint16_t* pb = (const uint16_t*)a.b;
  int acc = a.sumsq_accumulate ? 1 : 0;
#define OAB_ACC(HB, ST, SQ) \
  grad_accumulate_kernel<HB, ST, SQ><<<grid, kThreads, 0, stream>>>(o, pa, pb, a.n, a.sumsq_out, acc, a.scratch, vector_ok)
  const bool hb = pb != nullptr, st = o != nullptr, sq = a.sumsq_out != nullptr;
  if (hb && st && sq) OAB_ACC(true, true, true);
  else if (hb && st && !sq) OAB_ACC(true, true, false);
  else if (hb && !st && sq) OAB_ACC(true, false, true);
  else if (!hb && st && sq) OAB_ACC(false, true, true);
  else if (!hb && st && !sq) OAB_ACC(false, true, false);
  else if (!hb && !st && sq) OAB_ACC(false, false, true);
  else return cudaErrorInvalidValue;
#undef OAB_ACC
  return cudaGetLastError();
}

cudaError_t launch_clip_finalize(const float* slots, const int* index, int n, const float* extra_sq,
                                 float max_norm, float* coef_norm, float* total_sq_out,
                                 cudaStream_t stream) {
  count_launch();
  clip_finalize_kernel<<<1, kThreads, 0, stream>>>(slots, index, n, extra_sq, max_norm, coef_norm,
                                                   total_sq_out);
  return cudaGetLastError();
}

namespace {
__global__ void check_canary_kernel(const uint32_t* guard, int words, int* status, int tag) {
  for (int i = threadIdx.x; i < words; i += blockDim.x)
    if (guard[i] != kCanaryWord && atomicCAS(status, 0, 1) == 0) status[1] = tag;
}
}  // namespace

cudaError_t launch_check_canary(const void* guard, int words, int* status, int tag, cudaStream_t stream) {
  if (guard == nullptr || status == nullptr || words <= 0) return cudaErrorInvalidValue;
  count_launch();
  check_canary_kernel<<<1, 64, 0, stream>>>(static_cast<const uint32_t*>(guard), words, status, tag);
  return cudaGetLastError();
}

}  // namespace oab
