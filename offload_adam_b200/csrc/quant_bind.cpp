// Python bindings of the quantization kernels.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <optional>

#include "quant.h"

namespace py = pybind11;
using at::Tensor;

namespace {

int qdtype(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return oab::kF32;
    case at::kBFloat16: return oab::kBF16;
    case at::kHalf: return oab::kF16;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
  return -1;
}
cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }
void ok(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }
void dense(const Tensor& t, const char* n) { TORCH_CHECK(t.is_cuda() && t.is_contiguous(), n, " must be a contiguous CUDA tensor"); }

void absmax(const Tensor& x, Tensor out) {
  dense(x, "x");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.numel() >= 1, "out: CUDA fp32");
  ok(oab::launch_absmax(x.data_ptr(), qdtype(x), x.numel(), out.data_ptr<float>(), cur()), "absmax");
}

void nvfp4_quantize(const Tensor& x, const Tensor& amax, Tensor packed, Tensor scales, Tensor global_scale) {
  dense(x, "x"); dense(packed, "packed"); dense(scales, "scales");
  TORCH_CHECK(x.numel() % 16 == 0 && packed.numel() * 2 == x.numel() && scales.numel() * 16 == x.numel(), "nvfp4 shapes");
  TORCH_CHECK(packed.element_size() == 1 && scales.element_size() == 1, "nvfp4 payload dtypes");
  TORCH_CHECK(amax.is_cuda() && amax.scalar_type() == at::kFloat && global_scale.is_cuda() && global_scale.scalar_type() == at::kFloat, "scalars: CUDA fp32");
  ok(oab::launch_nvfp4_quantize(x.data_ptr(), qdtype(x), x.numel(), amax.data_ptr<float>(),
                                (uint8_t*)packed.data_ptr(), (uint8_t*)scales.data_ptr(),
                                global_scale.data_ptr<float>(), cur()), "nvfp4_quantize");
}

void nvfp4_dequantize(const Tensor& packed, const Tensor& scales, const Tensor& global_scale, Tensor out) {
  dense(packed, "packed"); dense(scales, "scales"); dense(out, "out");
  TORCH_CHECK(out.numel() == packed.numel() * 2 && scales.numel() * 16 == out.numel(), "nvfp4 shapes");
  ok(oab::launch_nvfp4_dequantize((const uint8_t*)packed.data_ptr(), (const uint8_t*)scales.data_ptr(),
                                  global_scale.data_ptr<float>(), out.numel(), out.data_ptr(), qdtype(out), cur()), "nvfp4_dequantize");
}

void nf4_quantize(const Tensor& x, int64_t blocksize, Tensor packed, Tensor absmax_out) {
  dense(x, "x"); dense(packed, "packed"); dense(absmax_out, "absmax");
  TORCH_CHECK(x.numel() % blocksize == 0 && packed.numel() * 2 == x.numel() && absmax_out.numel() * blocksize == x.numel(), "nf4 shapes");
  TORCH_CHECK(absmax_out.scalar_type() == at::kFloat, "absmax: fp32");
  ok(oab::launch_nf4_quantize(x.data_ptr(), qdtype(x), x.numel(), (int)blocksize, (uint8_t*)packed.data_ptr(),
                              absmax_out.data_ptr<float>(), cur()), "nf4_quantize");
}

void nf4_dequantize(const Tensor& packed, const Tensor& absmax_in, int64_t blocksize, Tensor out) {
  dense(packed, "packed"); dense(absmax_in, "absmax"); dense(out, "out");
  TORCH_CHECK(out.numel() == packed.numel() * 2 && absmax_in.numel() * blocksize == out.numel(), "nf4 shapes");
  ok(oab::launch_nf4_dequantize((const uint8_t*)packed.data_ptr(), absmax_in.data_ptr<float>(), out.numel(),
                                (int)blocksize, out.data_ptr(), qdtype(out), cur()), "nf4_dequantize");
}

void int8_quantize(const Tensor& x, Tensor q, Tensor scales) {
  dense(x, "x"); dense(q, "q"); dense(scales, "scales");
  TORCH_CHECK(x.dim() == 2 && q.sizes() == x.sizes() && q.scalar_type() == at::kChar && scales.numel() == x.size(0), "int8 shapes");
  ok(oab::launch_int8_quantize(x.data_ptr(), qdtype(x), x.size(0), x.size(1), q.data_ptr<int8_t>(),
                               scales.data_ptr(), qdtype(scales), cur()), "int8_quantize");
}

void int8_dequantize(const Tensor& q, const Tensor& scales, Tensor out) {
  dense(q, "q"); dense(scales, "scales"); dense(out, "out");
  TORCH_CHECK(q.dim() == 2 && out.sizes() == q.sizes() && out.scalar_type() == scales.scalar_type(), "int8 shapes/dtypes");
  ok(oab::launch_int8_dequantize(q.data_ptr<int8_t>(), scales.data_ptr(), qdtype(scales), q.size(0), q.size(1),
                                 out.data_ptr(), cur()), "int8_dequantize");
}

void int4_quantize(const Tensor& x, int64_t group, Tensor qweight, Tensor scales) {
  dense(x, "x"); dense(qweight, "qweight"); dense(scales, "scales");
  const int64_t out_f = x.size(0), in_f = x.size(1);
  TORCH_CHECK(in_f % 128 == 0 && (group == 32 || group == 64 || group == 128), "int4 kernel: in_f % 128 == 0, group in {32,64,128}");
  TORCH_CHECK(qweight.scalar_type() == at::kInt && qweight.size(0) == in_f / 8 && qweight.size(1) == out_f, "qweight shape");
  TORCH_CHECK(scales.size(0) == in_f / group && scales.size(1) == out_f, "scales shape");
  ok(oab::launch_int4_quantize(x.data_ptr(), qdtype(x), out_f, in_f, (int)group, qweight.data_ptr<int32_t>(),
                               scales.data_ptr(), qdtype(scales), cur()), "int4_quantize");
}

void int4_dequantize(const Tensor& qweight, const Tensor& scales, int64_t group, Tensor out) {
  dense(qweight, "qweight"); dense(scales, "scales"); dense(out, "out");
  const int64_t out_f = out.size(0), in_f = out.size(1);
  TORCH_CHECK(in_f % 128 == 0 && (group == 32 || group == 64 || group == 128), "int4 kernel: in_f % 128 == 0, group in {32,64,128}");
  TORCH_CHECK(out.scalar_type() == scales.scalar_type(), "int4 dequant output dtype = scale dtype");
  ok(oab::launch_int4_dequantize(qweight.data_ptr<int32_t>(), scales.data_ptr(), qdtype(scales), out_f, in_f,
                                 (int)group, out.data_ptr(), cur()), "int4_dequantize");
}

void fake_quant(int64_t format, const Tensor& x, Tensor out, int64_t group, int64_t scale_dtype, const std::optional<Tensor>& amax) {
  dense(x, "x"); dense(out, "out");
  TORCH_CHECK(x.dim() == 2 && out.sizes() == x.sizes() && out.scalar_type() == x.scalar_type(), "fake_quant: out like x (2-D)");
  const float* ap = nullptr;
  if (amax.has_value() && amax->defined()) {
    TORCH_CHECK(amax->is_cuda() && amax->scalar_type() == at::kFloat, "amax: CUDA fp32");
    ap = amax->data_ptr<float>();
  }
  ok(oab::launch_fake_quant((int)format, x.data_ptr(), out.data_ptr(), qdtype(x), x.size(0), x.size(1), (int)group,
                            (int)scale_dtype, ap, cur()), "fake_quant");
}

}  // namespace

void bind_quant(py::module_& m) {
  m.def("absmax", &absmax);
  m.def("nvfp4_quantize", &nvfp4_quantize);
  m.def("nvfp4_dequantize", &nvfp4_dequantize);
  m.def("nf4_quantize", &nf4_quantize);
  m.def("nf4_dequantize", &nf4_dequantize);
  m.def("int8_quantize", &int8_quantize);
  m.def("int8_dequantize", &int8_dequantize);
  m.def("int4_quantize", &int4_quantize);
  m.def("int4_dequantize", &int4_dequantize);
  m.def("fake_quant", &fake_quant, py::arg("format"), py::arg("x"), py::arg("out"), py::arg("group"),
        py::arg("scale_dtype"), py::arg("amax") = py::none());
}
