// Host-side launch interface of the gradient kernels (grad_ops.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oab {

// The scratch area handed to the reduction kernels holds 148 * 8 partial sums
// followed by one 32-bit ticket counter (see common.cuh).
constexpr size_t kSumsqScratchBytes = (148 * 8 + 4) * sizeof(float);

// out[i] = bf16(a[i] + b[i])   (b == nullptr: out[i] = a[i]; out == nullptr: no store)
// and, when sumsq_out != nullptr, sumsq_out (+)= sum_i float(out[i])^2, reduced in a
// fixed order so that the result is bitwise reproducible for a given n.
// Any operand may be mapped pinned host memory.
struct AccumArgs {
  void* out = nullptr;
  const void* a = nullptr;
  const void* b = nullptr;
  int64_t n = 0;
  float* sumsq_out = nullptr;
  bool sumsq_accumulate = false;  // add to *sumsq_out instead of overwriting it
  float* scratch = nullptr;       // kSumsqScratchBytes, zero-initialised ticket
  int max_ctas = 0;
};
cudaError_t launch_grad_accumulate(const AccumArgs& a, cudaStream_t stream);

// coef_norm[0] = min(1, max_norm / (sqrt(total) + 1e-6)), coef_norm[1] = sqrt(total)
// with total = extra_sq[0] (if given) + sum_i slots[index[i]]  (index may be null: all slots).
cudaError_t launch_clip_finalize(const float* slots, const int* index, int n, const float* extra_sq,
                                 float max_norm, float* coef_norm, float* total_sq_out,
                                 cudaStream_t stream);

// Debugging aid: compares `words` 32-bit words at `guard` with kCanaryWord and, on the first
// mismatch, stores {1, tag} into status[0..1] (device memory; first failure wins).  Never traps.
constexpr uint32_t kCanaryWord = 0xA5A5A5A5u;
cudaError_t launch_check_canary(const void* guard, int words, int* status, int tag, cudaStream_t stream);

}  // namespace oab
