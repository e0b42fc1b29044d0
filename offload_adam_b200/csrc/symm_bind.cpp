// Python bindings of the symmetric-memory kernels.  Peer addresses arrive as plain
// integers (device pointers obtained from the symmetric-memory rendezvous).
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <optional>

#include "symm_ops.h"

namespace py = pybind11;
using at::Tensor;
using OptT = std::optional<Tensor>;

namespace {

cudaStream_t pick(int64_t h) { return h ? reinterpret_cast<cudaStream_t>(h) : at::cuda::getCurrentCUDAStream().stream(); }
void ok(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }

// status words live in pinned host memory mapped into the device, so the host can
// read them without synchronising
int* status_ptr(const Tensor& status) {
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1, "status: int32 tensor");
  if (status.is_cuda()) return status.data_ptr<int>();
  void* d = nullptr;
  TORCH_CHECK(cudaHostGetDevicePointer(&d, status.data_ptr(), 0) == cudaSuccess, "status must be CUDA or pinned host memory");
  return reinterpret_cast<int*>(d);
}

void peer_reduce(Tensor out, const std::vector<int64_t>& peers, double scale, const OptT& sumsq,
                 const OptT& scratch, const OptT& status, int64_t max_ctas, int64_t stream, const OptT& acc) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16, "out: contiguous CUDA bf16");
  TORCH_CHECK(!peers.empty() && peers.size() <= (size_t)oab::kMaxPeers, "1..8 peers");
  oab::PeerReduceArgs a;
  a.out = out.data_ptr();
  a.n = out.numel();
  a.n_peers = (int)peers.size();
  for (size_t j = 0; j < peers.size(); ++j) a.peers[j] = reinterpret_cast<const void*>(peers[j]);
  a.scale = (float)scale;
  if (acc.has_value() && acc->defined()) {
    TORCH_CHECK(acc->is_cuda() && acc->is_contiguous() && acc->scalar_type() == at::kBFloat16 && acc->numel() == out.numel(),
                "acc: contiguous CUDA bf16 of out's size");
    a.acc_in = acc->data_ptr();
  }
  if (sumsq.has_value() && sumsq->defined()) {
    TORCH_CHECK(scratch.has_value() && scratch->defined(), "sumsq needs scratch");
    a.sumsq_out = sumsq->data_ptr<float>();
    a.scratch = reinterpret_cast<float*>(scratch->data_ptr());
  }
  if (status.has_value() && status->defined()) a.abort_flag = status_ptr(*status);
  a.max_ctas = (int)max_ctas;
  ok(oab::launch_peer_reduce(a, pick(stream)), "peer_reduce");
}

void wait_flags(const Tensor& flags, int64_t offset, int64_t n, int64_t epoch, double timeout_ms,
                const Tensor& status, int64_t code, int64_t stream) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && offset >= 0 && offset + n <= flags.numel(), "flags: CUDA int32");
  ok(oab::launch_wait_flags(reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()) + offset, (int)n,
                            (uint32_t)epoch, (uint64_t)(timeout_ms * 1e6), status_ptr(status), (int)code,
                            pick(stream)), "wait_flags");
}

void signal(const std::vector<int64_t>& ptrs, int64_t value, int64_t stream) {
  TORCH_CHECK(ptrs.size() <= (size_t)oab::kMaxPeers, "at most 8 targets");
  uint32_t* p[oab::kMaxPeers] = {};
  for (size_t j = 0; j < ptrs.size(); ++j) p[j] = reinterpret_cast<uint32_t*>(ptrs[j]);
  ok(oab::launch_signal(p, (int)ptrs.size(), (uint32_t)value, pick(stream)), "signal");
}

void signal_many(const std::vector<int64_t>& bases, int64_t first, int64_t stride, int64_t count, int64_t value,
                 int64_t stream) {
  TORCH_CHECK(bases.size() <= (size_t)oab::kMaxPeers, "at most 8 targets");
  uint32_t* p[oab::kMaxPeers] = {};
  for (size_t j = 0; j < bases.size(); ++j) p[j] = reinterpret_cast<uint32_t*>(bases[j]);
  ok(oab::launch_signal_many(p, (int)bases.size(), (int)first, (int)stride, (int)count, (uint32_t)value, pick(stream)),
     "signal_many");
}

void scalar_exchange(const Tensor& my_value, const std::vector<int64_t>& peer_slots,
                     const std::vector<int64_t>& peer_flags, const Tensor& local_slots,
                     const Tensor& local_flags, int64_t rank, int64_t epoch, double timeout_ms,
                     const Tensor& status, Tensor out, int64_t stream, bool op_max) {
  const size_t n = peer_slots.size();
  TORCH_CHECK(n >= 1 && n <= (size_t)oab::kMaxPeers && peer_flags.size() == n, "1..8 peers");
  TORCH_CHECK(my_value.is_cuda() && out.is_cuda() && local_slots.is_cuda() && local_flags.is_cuda(), "CUDA tensors");
  TORCH_CHECK(local_slots.numel() >= (int64_t)n && local_flags.numel() >= (int64_t)n, "slot arrays too small");
  oab::ScalarExchangeArgs a;
  a.my_value = my_value.data_ptr<float>();
  for (size_t j = 0; j < n; ++j) {
    a.peer_slots[j] = reinterpret_cast<float*>(peer_slots[j]);
    a.peer_flags[j] = reinterpret_cast<uint32_t*>(peer_flags[j]);
  }
  a.local_slots = local_slots.data_ptr<float>();
  a.local_flags = reinterpret_cast<const uint32_t*>(local_flags.data_ptr<int>());
  a.n = (int)n;
  a.rank = (int)rank;
  a.epoch = (uint32_t)epoch;
  a.timeout_ns = (uint64_t)(timeout_ms * 1e6);
  a.status = status_ptr(status);
  a.out = out.data_ptr<float>();
  a.op_max = op_max;
  ok(oab::launch_scalar_exchange(a, pick(stream)), "scalar_exchange");
}

void mirror_words(const Tensor& src, const Tensor& dst, int64_t stream) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kInt && dst.scalar_type() == at::kInt &&
                  dst.numel() >= src.numel() && src.numel() <= 32, "mirror_words: int32, at most 32 words");
  ok(oab::launch_mirror_words(src.data_ptr<int>(), status_ptr(dst), (int)src.numel(), pick(stream)), "mirror_words");
}

}  // namespace

void bind_symm(py::module_& m) {
  m.def("mirror_words", &mirror_words, py::arg("src"), py::arg("dst"), py::arg("stream") = 0);
  m.def("peer_reduce", &peer_reduce, py::arg("out"), py::arg("peers"), py::arg("scale"),
        py::arg("sumsq") = py::none(), py::arg("scratch") = py::none(), py::arg("status") = py::none(),
        py::arg("max_ctas") = 0, py::arg("stream") = 0, py::arg("acc") = py::none());
  m.def("wait_flags", &wait_flags, py::arg("flags"), py::arg("offset"), py::arg("n"), py::arg("epoch"),
        py::arg("timeout_ms"), py::arg("status"), py::arg("code"), py::arg("stream") = 0);
  m.def("signal", &signal, py::arg("ptrs"), py::arg("value"), py::arg("stream") = 0);
  m.def("signal_many", &signal_many, py::arg("bases"), py::arg("first"), py::arg("stride"), py::arg("count"),
        py::arg("value"), py::arg("stream") = 0);
  m.def("scalar_exchange", &scalar_exchange, py::arg("my_value"), py::arg("peer_slots"),
        py::arg("peer_flags"), py::arg("local_slots"), py::arg("local_flags"), py::arg("rank"),
        py::arg("epoch"), py::arg("timeout_ms"), py::arg("status"), py::arg("out"), py::arg("stream") = 0,
        py::arg("op_max") = false);
  m.attr("SYMM_TIMEOUT_GRAD") = (int)oab::kSymmTimeoutGrad;
  m.attr("SYMM_TIMEOUT_PARAM") = (int)oab::kSymmTimeoutParam;
  m.attr("SYMM_TIMEOUT_SCALAR") = (int)oab::kSymmTimeoutScalar;
}
