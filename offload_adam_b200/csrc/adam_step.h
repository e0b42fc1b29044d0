// Host-side launch interface of the fused Adam step kernels (adam_step.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oab {

constexpr int kMaxPeers = 8;  // ranks of one NVSwitch domain

enum AdamMode : int {
  kModeSR = 0,          // bf16 params, stochastic rounding on write-back
  kModeFP32Master = 1,  // fp32 master copy, bf16 param is RNE(master)
  kModeFP31 = 2,        // bf16 param + int16 (error >> 1), master keeps 31 bits
  kModeCustom = 3,      // bf16 param (round-half-up) + int16 error, lossless fp32
};

// All pointers may be device memory or pinned host memory mapped into the
// device address space: the kernel is a pure stream over its operands, so the
// same code serves the HBM-resident path and the zero-copy path in which the
// optimizer state is read from and written back to host RAM over PCIe by the
// kernel itself.
struct AdamStepArgs {
  int mode = 0;              // AdamMode
  bool decoupled = false;    // AdamW-style decay
  void* p = nullptr;         // bf16 parameter (in/out; out only for fp32_master; may be
                             // null for fp32_master when no bf16 write-back is wanted)
  const void* g = nullptr;   // bf16 gradient
  const void* g2 = nullptr;  // optional second bf16 gradient term: g := bf16(g + g2)
  void* m = nullptr;         // bf16 exp_avg (in/out)
  void* v = nullptr;         // bf16 exp_avg_sq (in/out)
  void* extra = nullptr;     // fp32 master (fp32_master) or int16 rounding error
  void* extra_copy = nullptr;  // fp32_master only: the updated master is stored here as well
                               // (device memory; lets a later pass re-quantize the weight
                               // after `extra`, a staging chunk, has gone back to the host)
  int64_t n = 0;             // elements
  float lr = 0.f, wd = 0.f, beta1_hat = 0.f, beta2_hat = 0.f, eps = 0.f;
  const float* clip_coef = nullptr;  // optional device scalar multiplied into g (fp32)
  uint64_t seed = 0;                 // stochastic rounding stream
  int64_t elem_offset = 0;           // global index of element 0 (keeps SR stream
                                     // independent of how a tensor is chunked)
  float* amax_out = nullptr;         // optional, fp32_master only: atomic max of |updated master| (fp32 bits)
  int max_ctas = 0;                  // 0 = size for HBM streaming; small values keep
                                     // most SMs free for concurrent GEMMs

  // ---- ZeRO-1 collectives fused into the same pass (all optional) ----
  // Gradient pulled from the replicas of every rank (peer-mapped pointers, NVLink):
  //   g := bf16(g_scale * sum_j g_peers[j][i]), summed in fp32 in index order.
  // When n_g_peers > 0, `g`/`g2` are ignored.
  const void* g_peers[kMaxPeers] = {};
  int n_g_peers = 0;
  float g_scale = 1.0f;
  // The updated bf16 parameter is stored to each of these (the replicas of all ranks,
  // the local one included) instead of `p`; `p` is still the source of the old value.
  void* p_peers[kMaxPeers] = {};
  int n_p_peers = 0;
  // Device-visible status word; when it is non-zero at launch the kernel returns
  // without touching memory (an earlier bounded wait gave up).
  const int* abort_flag = nullptr;
};

// Enqueues one launch on `stream`.  Returns cudaGetLastError().
cudaError_t launch_adam_step(const AdamStepArgs& a, cudaStream_t stream);

// Table-driven step over many small tensors in one launch.
struct MultiTensorEntry {
  void* p;
  const void* g;
  void* m;
  void* v;
  void* extra;
  int64_t n;
  int64_t elem_offset;  // SR stream offset of this tensor
};
cudaError_t launch_multi_tensor_adam(const MultiTensorEntry* dev_table, int n_tensors,
                                     const int2* dev_block_map, int n_blocks, int mode,
                                     bool decoupled, float lr, float wd, float beta1_hat,
                                     float beta2_hat, float eps, const float* clip_coef,
                                     uint64_t seed, bool zero_grad, cudaStream_t stream);

// Elements covered by one block of the multi-tensor kernel.
int multi_tensor_chunk();

}  // namespace oab
