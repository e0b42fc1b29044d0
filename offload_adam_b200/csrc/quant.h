// Host-side launch interface of the weight-only quantization kernels (quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oab {

enum QDtype : int { kF32 = 0, kBF16 = 1, kF16 = 2 };
enum QFormat : int { kQNone = 0, kQNVFP4 = 1, kQNF4 = 2, kQInt4 = 3, kQInt8 = 4 };

// out[0] = max(out[0], max |x|) (fp32 bits compared as unsigned); zero `out` first.
cudaError_t launch_absmax(const void* x, int dtype, int64_t n, float* out, cudaStream_t st);

// NVFP4: numel % 16 == 0.  `amax` is a device scalar holding max |x| of the tensor.
cudaError_t launch_nvfp4_quantize(const void* x, int dtype, int64_t numel, const float* amax,
                                  uint8_t* packed, uint8_t* scales, float* global_scale,
                                  cudaStream_t st);
cudaError_t launch_nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales,
                                    const float* global_scale, int64_t numel, void* out, int dtype,
                                    cudaStream_t st);

// NF4: blocksize in {16, 32, 64, 128, 256, 512}, in_f % blocksize == 0.
cudaError_t launch_nf4_quantize(const void* x, int dtype, int64_t numel, int blocksize,
                                uint8_t* packed, float* absmax, cudaStream_t st);
cudaError_t launch_nf4_dequantize(const uint8_t* packed, const float* absmax, int64_t numel,
                                  int blocksize, void* out, int dtype, cudaStream_t st);

// int8 per-row; scales and the dequantized output share `scale_dtype`.
cudaError_t launch_int8_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int8_t* q,
                                 void* scales, int scale_dtype, cudaStream_t st);
cudaError_t launch_int8_dequantize(const int8_t* q, const void* scales, int scale_dtype,
                                   int64_t out_f, int64_t in_f, void* out, cudaStream_t st);

// GPTQ int4: in_f % 128 == 0, group in {32, 64, 128}.
cudaError_t launch_int4_quantize(const void* x, int dtype, int64_t out_f, int64_t in_f, int group,
                                 int32_t* qweight, void* scales, int scale_dtype, cudaStream_t st);
cudaError_t launch_int4_dequantize(const int32_t* qweight, const void* scales, int scale_dtype,
                                   int64_t out_f, int64_t in_f, int group, void* out,
                                   cudaStream_t st);

// out = dequantize(quantize(x)) in x's dtype, in one pass and without a payload:
// x and out are (out_f, in_f) row-major of `dtype`.  `group` is the NF4 block size or
// the int4 group size; `scale_dtype` the dtype the int4 / int8 scales would be stored
// in; `tensor_amax` (NVFP4 only) a device scalar holding max|x|.  Bit-identical to
// running the format's quantize and dequantize kernels one after the other.
cudaError_t launch_fake_quant(int format, const void* x, void* out, int dtype, int64_t out_f,
                              int64_t in_f, int group, int scale_dtype, const float* tensor_amax,
                              cudaStream_t st);

}  // namespace oab
