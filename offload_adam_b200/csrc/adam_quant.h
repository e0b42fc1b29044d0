// Host-side launch interface of the kernels that step a quantized weight: Adam on the
// fp32 master, re-quantization of the updated rows and the store of the packed rows
// into every replica, in one pass (adam_quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "adam_step.h"
#include "quant.h"

namespace oab {

// Where the packed rows go.  A weight has `out_f` rows of `in_f` columns; a launch
// covers rows [row0, row0 + n / in_f) of it.  payload0 / payload1 are the base
// addresses of the WHOLE payload tensors in each replica (this rank's own and, over
// NVLink peer mappings, the other ranks'):
//   NVFP4  payload0 = packed codes (out_f, in_f / 2) u8, payload1 = block scales (out_f, in_f / 16) e4m3
//   NF4    payload0 = packed indices (out_f, in_f / 2) u8, payload1 = absmax (out_f * in_f / group) fp32
//   int4   payload0 = qweight (in_f / 8, out_f) int32,    payload1 = scales (in_f / group, out_f) scale_dtype
//   int8   payload0 = weight (out_f, in_f) int8,          payload1 = scales (out_f) scale_dtype
// A row shard of the GPTQ int4 layout is a column slab of both tensors; the kernel
// addresses it through out_f and row0.
struct QuantPushArgs {
  int format = kQNone;   // QFormat
  int64_t out_f = 0, in_f = 0;
  int64_t row0 = 0;
  int group = 0;         // NF4 block size / int4 group size
  int scale_dtype = kBF16;
  int n_replicas = 0;    // 1: this GPU only
  void* payload0[kMaxPeers] = {};
  void* payload1[kMaxPeers] = {};
  // NVFP4 only: device scalar with max|master| over the whole weight, and where this
  // rank's copy of the fp32 tensor scale goes (written by the quantize pass)
  const float* tensor_amax = nullptr;
  float* global_scale_out = nullptr;
};

// True when launch_adam_quant_push can take the weight (else the caller steps the master
// with launch_adam_step and re-quantizes with the stand-alone kernels).
bool adam_quant_supported(int format, int64_t in_f, int group);

// fp32_master Adam over a.n elements (a.n % in_f == 0: whole rows) whose updated master
// is quantized and stored into q.payload*[0 .. n_replicas).  a.p is ignored (a quantized
// weight has no bf16 copy); a.g / a.g2 / a.g_peers, a.clip_coef, a.abort_flag as in
// launch_adam_step.  NVFP4 is not accepted here: its tensor scale depends on the whole
// updated weight, so it runs launch_adam_step (with amax_out and extra_copy) followed by
// launch_nvfp4_quantize_push once the maximum is known.
cudaError_t launch_adam_quant_push(const AdamStepArgs& a, const QuantPushArgs& q, cudaStream_t stream);

// NVFP4 second pass: quantizes `n` fp32 values starting at row q.row0 (n % in_f == 0)
// and stores codes and block scales into every replica; writes q.global_scale_out.
cudaError_t launch_nvfp4_quantize_push(const float* master, int64_t n, const QuantPushArgs& q,
                                       const int* abort_flag, cudaStream_t stream);

}  // namespace oab
