// Python bindings of the native runtime (module offload_adam_b200._C).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>

#include "adam_quant.h"
#include "adam_step.h"
#include "grad_ops.h"
#include "offload_engine.h"
#include "pinned_arena.h"
#include "symm_ops.h"

namespace py = pybind11;
using at::Tensor;

namespace oab {
extern unsigned long long g_launch_count;
}

namespace {

using OptT = std::optional<Tensor>;

void cu_check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

// Device-visible address of a tensor: CUDA tensors as is, pinned CPU tensors
// through their mapping into the device address space (zero-copy access).
void* dev_ptr(const Tensor& t) {
  if (t.is_cuda()) return t.data_ptr();
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, t.data_ptr(), 0);
  TORCH_CHECK(e == cudaSuccess, "tensor is neither CUDA nor registered pinned host memory: ",
              cudaGetErrorString(e));
  return d;
}
void* dev_ptr(const OptT& t) { return (t.has_value() && t->defined()) ? dev_ptr(*t) : nullptr; }

cudaStream_t pick_stream(int64_t handle) {
  return handle ? reinterpret_cast<cudaStream_t>(handle) : at::cuda::getCurrentCUDAStream().stream();
}

void check_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void set_peers(oab::AdamStepArgs& a, const std::vector<int64_t>& g_peers, double g_scale,
               const std::vector<int64_t>& p_peers, const OptT& status) {
  TORCH_CHECK(g_peers.size() <= (size_t)oab::kMaxPeers && p_peers.size() <= (size_t)oab::kMaxPeers,
              "at most ", oab::kMaxPeers, " peers");
  a.n_g_peers = (int)g_peers.size();
  a.n_p_peers = (int)p_peers.size();
  a.g_scale = (float)g_scale;
  for (size_t j = 0; j < g_peers.size(); ++j) a.g_peers[j] = reinterpret_cast<const void*>(g_peers[j]);
  for (size_t j = 0; j < p_peers.size(); ++j) a.p_peers[j] = reinterpret_cast<void*>(p_peers[j]);
  if (status.has_value() && status->defined()) a.abort_flag = reinterpret_cast<const int*>(dev_ptr(*status));
}

oab::AdamStepArgs make_args(int64_t mode, const OptT& p, const OptT& g_opt, const OptT& g2,
                            const Tensor& m, const Tensor& v, const OptT& extra, double lr,
                            double wd, double b1h, double b2h, double eps, bool decoupled,
                            const OptT& clip, int64_t seed, int64_t elem_offset, const OptT& amax,
                            int64_t max_ctas) {
  TORCH_CHECK(m.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "exp_avg/exp_avg_sq must be bfloat16");
  const int64_t n = m.numel();
  TORCH_CHECK(v.numel() == n, "state size mismatch");
  check_contig(m, "exp_avg"); check_contig(v, "exp_avg_sq");
  oab::AdamStepArgs a;
  const bool has_g = g_opt.has_value() && g_opt->defined();
  if (has_g) {
    TORCH_CHECK(g_opt->scalar_type() == at::kBFloat16 && g_opt->numel() == n, "grad must be bf16 of the state's size");
    check_contig(*g_opt, "grad");
  }
  a.mode = (int)mode;
  a.decoupled = decoupled;
  if (p.has_value() && p->defined()) {
    TORCH_CHECK(p->scalar_type() == at::kBFloat16 && p->numel() == n, "params must be bf16 of grad's size");
    check_contig(*p, "params");
    a.p = dev_ptr(*p);
  }
  if (has_g) a.g = dev_ptr(*g_opt);
  if (g2.has_value() && g2->defined()) {
    TORCH_CHECK(g2->scalar_type() == at::kBFloat16 && g2->numel() == n, "grad2 mismatch");
    a.g2 = dev_ptr(*g2);
  }
  a.m = dev_ptr(m);
  a.v = dev_ptr(v);
  if (extra.has_value() && extra->defined()) {
    if (mode == oab::kModeFP32Master) {
      TORCH_CHECK(extra->scalar_type() == at::kFloat, "master_params must be fp32");
    } else {
      TORCH_CHECK(extra->scalar_type() == at::kShort, "rounding_error must be int16");
    }
    TORCH_CHECK(extra->numel() == n, "extra state size mismatch");
    check_contig(*extra, "extra state");
    a.extra = dev_ptr(*extra);
  }
  a.n = n;
  a.lr = (float)lr; a.wd = (float)wd; a.beta1_hat = (float)b1h; a.beta2_hat = (float)b2h; a.eps = (float)eps;
  if (clip.has_value() && clip->defined()) {
    TORCH_CHECK(clip->is_cuda() && clip->scalar_type() == at::kFloat, "clip_coef must be a CUDA fp32 scalar");
    a.clip_coef = clip->data_ptr<float>();
  }
  a.seed = (uint64_t)seed;
  a.elem_offset = elem_offset;
  if (amax.has_value() && amax->defined()) {
    TORCH_CHECK(amax->is_cuda() && amax->scalar_type() == at::kFloat, "amax must be a CUDA fp32 scalar");
    a.amax_out = amax->data_ptr<float>();
  }
  a.max_ctas = (int)max_ctas;
  return a;
}

void adam_step(int64_t mode, const OptT& p, const OptT& g, const OptT& g2, const Tensor& m,
               const Tensor& v, const OptT& extra, double lr, double wd, double b1h, double b2h,
               double eps, bool decoupled, const OptT& clip, int64_t seed, int64_t elem_offset,
               const OptT& amax, int64_t max_ctas, int64_t stream, const std::vector<int64_t>& g_peers,
               double g_scale, const std::vector<int64_t>& p_peers, const OptT& status, const OptT& extra_copy) {
  auto a = make_args(mode, p, g, g2, m, v, extra, lr, wd, b1h, b2h, eps, decoupled, clip, seed,
                     elem_offset, amax, max_ctas);
  set_peers(a, g_peers, g_scale, p_peers, status);
  if (extra_copy.has_value() && extra_copy->defined()) {
    TORCH_CHECK(extra_copy->is_cuda() && extra_copy->scalar_type() == at::kFloat && extra_copy->numel() == a.n,
                "extra_copy: CUDA fp32 of the state's size");
    a.extra_copy = extra_copy->data_ptr();
  }
  TORCH_CHECK(a.g != nullptr || a.n_g_peers > 0, "adam_step needs a gradient");
  cu_check(oab::launch_adam_step(a, pick_stream(stream)), "adam_step launch");
}

void grad_accumulate(const OptT& out, const Tensor& a, const OptT& b, const OptT& sumsq,
                     bool sumsq_accumulate, const OptT& scratch, int64_t max_ctas, int64_t stream) {
  TORCH_CHECK(a.scalar_type() == at::kBFloat16, "grad_accumulate: bf16 only");
  check_contig(a, "a");
  oab::AccumArgs x;
  x.out = dev_ptr(out);
  x.a = dev_ptr(a);
  x.b = dev_ptr(b);
  x.n = a.numel();
  if (out.has_value() && out->defined()) {
    TORCH_CHECK(out->numel() == x.n && out->scalar_type() == at::kBFloat16, "out mismatch");
  }
  if (b.has_value() && b->defined()) {
    TORCH_CHECK(b->numel() == x.n && b->scalar_type() == at::kBFloat16, "b mismatch");
  }
  if (sumsq.has_value() && sumsq->defined()) {
    TORCH_CHECK(sumsq->is_cuda() && sumsq->scalar_type() == at::kFloat, "sumsq must be CUDA fp32");
    TORCH_CHECK(scratch.has_value() && scratch->is_cuda() &&
                    (size_t)scratch->numel() * scratch->element_size() >= oab::kSumsqScratchBytes,
                "sumsq needs a CUDA scratch buffer of sumsq_scratch_bytes()");
    x.sumsq_out = sumsq->data_ptr<float>();
    x.scratch = reinterpret_cast<float*>(scratch->data_ptr());
  }
  x.sumsq_accumulate = sumsq_accumulate;
  x.max_ctas = (int)max_ctas;
  cu_check(oab::launch_grad_accumulate(x, pick_stream(stream)), "grad_accumulate launch");
}

void clip_finalize(const OptT& slots, const OptT& index, const OptT& extra_sq, double max_norm,
                   const OptT& coef_norm, const OptT& total_sq, int64_t stream) {
  const float* sp = nullptr; const int* ip = nullptr; int n = 0;
  if (slots.has_value() && slots->defined()) {
    TORCH_CHECK(slots->is_cuda() && slots->scalar_type() == at::kFloat, "slots: CUDA fp32");
    sp = slots->data_ptr<float>();
    n = (int)slots->numel();
  }
  if (index.has_value() && index->defined()) {
    TORCH_CHECK(index->is_cuda() && index->scalar_type() == at::kInt, "index: CUDA int32");
    ip = index->data_ptr<int>();
    n = (int)index->numel();
  }
  const float* ep = (extra_sq.has_value() && extra_sq->defined()) ? extra_sq->data_ptr<float>() : nullptr;
  float* cp = (coef_norm.has_value() && coef_norm->defined()) ? coef_norm->data_ptr<float>() : nullptr;
  float* tp = (total_sq.has_value() && total_sq->defined()) ? total_sq->data_ptr<float>() : nullptr;
  if (cp) {
    TORCH_CHECK(coef_norm->numel() >= 2, "coef_norm needs 2 floats");
  }
  cu_check(oab::launch_clip_finalize(sp, ip, n, ep, (float)max_norm, cp, tp, pick_stream(stream)), "clip_finalize launch");
}

void multi_tensor_adam(const Tensor& table, const Tensor& block_map, int64_t mode, bool decoupled,
                       double lr, double wd, double b1h, double b2h, double eps, const OptT& clip,
                       int64_t seed, bool zero_grad, int64_t stream) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.dim() == 2 &&
                  table.size(1) == 7 && table.is_contiguous(), "table: CUDA int64 [n,7]");
  TORCH_CHECK(block_map.is_cuda() && block_map.scalar_type() == at::kInt && block_map.dim() == 2 &&
                  block_map.size(1) == 2 && block_map.is_contiguous(), "block_map: CUDA int32 [nb,2]");
  static_assert(sizeof(oab::MultiTensorEntry) == 7 * sizeof(int64_t), "table layout");
  const float* cp = (clip.has_value() && clip->defined()) ? clip->data_ptr<float>() : nullptr;
  cu_check(oab::launch_multi_tensor_adam(
               reinterpret_cast<const oab::MultiTensorEntry*>(table.data_ptr()), (int)table.size(0),
               reinterpret_cast<const int2*>(block_map.data_ptr()), (int)block_map.size(0), (int)mode,
               decoupled, (float)lr, (float)wd, (float)b1h, (float)b2h, (float)eps, cp, (uint64_t)seed,
               zero_grad, pick_stream(stream)),
           "multi_tensor_adam launch");
}

// ---------------------------------------------------------------------------
// Quantized weights: where the packed rows of a step go
// ---------------------------------------------------------------------------
struct PyQuantSpec {
  oab::QuantPushArgs q;
  Tensor amax_keep, gscale_keep;  // keep the scalars alive
  PyQuantSpec(int64_t format, int64_t out_f, int64_t in_f, int64_t row0, int64_t group, int64_t scale_dtype,
              const std::vector<int64_t>& payload0, const std::vector<int64_t>& payload1, const OptT& tensor_amax,
              const OptT& global_scale) {
    TORCH_CHECK(!payload0.empty() && payload0.size() <= (size_t)oab::kMaxPeers && payload1.size() == payload0.size(),
                "1..", oab::kMaxPeers, " replicas, two payload tensors each");
    q.format = (int)format;
    q.out_f = out_f;
    q.in_f = in_f;
    q.row0 = row0;
    q.group = (int)group;
    q.scale_dtype = (int)scale_dtype;
    q.n_replicas = (int)payload0.size();
    for (size_t j = 0; j < payload0.size(); ++j) {
      q.payload0[j] = reinterpret_cast<void*>(payload0[j]);
      q.payload1[j] = reinterpret_cast<void*>(payload1[j]);
    }
    if (tensor_amax.has_value() && tensor_amax->defined()) {
      TORCH_CHECK(tensor_amax->is_cuda() && tensor_amax->scalar_type() == at::kFloat, "tensor_amax: CUDA fp32");
      amax_keep = *tensor_amax;
      q.tensor_amax = amax_keep.data_ptr<float>();
    }
    if (global_scale.has_value() && global_scale->defined()) {
      TORCH_CHECK(global_scale->is_cuda() && global_scale->scalar_type() == at::kFloat, "global_scale: CUDA fp32");
      gscale_keep = *global_scale;
      q.global_scale_out = gscale_keep.data_ptr<float>();
    }
  }
};

// Adam + re-quantize + push on device-resident operands (tests, micro-benchmarks; the
// optimizers go through OffloadEngine.staged_step).
void adam_quant_push(const PyQuantSpec& spec, const OptT& g, const OptT& g2, const Tensor& m, const Tensor& v,
                     const Tensor& master, double lr, double wd, double b1h, double b2h, double eps, bool decoupled,
                     const OptT& clip, int64_t max_ctas, int64_t stream, const std::vector<int64_t>& g_peers,
                     double g_scale, const OptT& status) {
  auto a = make_args(oab::kModeFP32Master, OptT(), g, g2, m, v, OptT(master), lr, wd, b1h, b2h, eps, decoupled,
                     clip, 0, 0, OptT(), max_ctas);
  set_peers(a, g_peers, g_scale, {}, status);
  cu_check(oab::launch_adam_quant_push(a, spec.q, pick_stream(stream)), "adam_quant_push launch");
}

void nvfp4_quantize_push(const PyQuantSpec& spec, int64_t master_ptr, int64_t n, const OptT& status, int64_t stream) {
  const int* abort_flag = (status.has_value() && status->defined()) ? reinterpret_cast<const int*>(dev_ptr(*status)) : nullptr;
  cu_check(oab::launch_nvfp4_quantize_push(reinterpret_cast<const float*>(master_ptr), n, spec.q, abort_flag,
                                           pick_stream(stream)),
           "nvfp4_quantize_push launch");
}

// ---------------------------------------------------------------------------
// Pinned arena
// ---------------------------------------------------------------------------
struct PyArena {
  std::shared_ptr<oab::PinnedArena> arena;
  PyArena(const std::vector<int64_t>& sizes, int64_t numa_node, bool register_cuda, bool huge_pages,
          int64_t touch_threads, int64_t segment_bytes, int64_t alignment) {
    oab::ArenaOptions o;
    o.numa_node = (int)numa_node;
    o.register_cuda = register_cuda;
    o.huge_pages = huge_pages;
    o.touch_threads = (int)touch_threads;
    if (segment_bytes > 0) o.segment_bytes = (size_t)segment_bytes;
    if (alignment > 0) o.alignment = (size_t)alignment;
    std::vector<size_t> s(sizes.begin(), sizes.end());
    {
      py::gil_scoped_release nogil;
      arena = std::make_shared<oab::PinnedArena>(s, o);
    }
  }
  Tensor tensor(int64_t i, std::vector<int64_t> shape, py::object dtype_obj) {
    auto dtype = torch::python::detail::py_object_to_dtype(dtype_obj);
    TORCH_CHECK(i >= 0 && (size_t)i < arena->num_tensors(), "arena index out of range");
    int64_t numel = 1;
    for (auto d : shape) numel *= d;
    TORCH_CHECK((size_t)numel * c10::elementSize(dtype) <= arena->size(i), "tensor larger than its arena slot");
    auto keep = arena;
    return at::from_blob(arena->ptr(i), shape, [keep](void*) {}, at::TensorOptions().dtype(dtype).device(at::kCPU));
  }
  py::dict stats() const {
    py::dict d;
    d["total_bytes"] = arena->total_bytes();
    d["segments"] = arena->num_segments();
    d["registered"] = arena->registered();
    d["numa_node"] = arena->numa_node();
    d["numa_bound"] = arena->numa_bound();
    d["seconds_map"] = arena->seconds_map();
    d["seconds_touch"] = arena->seconds_touch();
    d["seconds_register"] = arena->seconds_register();
    return d;
  }
};

// ---------------------------------------------------------------------------
// Engine
// ---------------------------------------------------------------------------
struct PyEngine {
  std::unique_ptr<oab::OffloadEngine> eng;
  Tensor workspace;  // keeps the staging buffer alive
  // the engine (helper threads, copies in flight) must be gone before the buffer is
  ~PyEngine() { eng.reset(); }
  PyEngine(int64_t device, int64_t compute, int64_t h2d, int64_t d2h, Tensor ws, int64_t chunk_elems,
           int64_t max_ctas, int64_t n_tensors, bool async_writeback, bool canaries, bool lazy_resident)
      : workspace(std::move(ws)) {
    oab::EngineOptions o;
    o.chunk_elems = chunk_elems;
    o.max_ctas = (int)max_ctas;
    o.async_writeback = async_writeback;
    o.canaries = canaries;
    o.lazy_resident = lazy_resident;
    TORCH_CHECK(workspace.is_cuda(), "engine workspace must be a CUDA tensor");
    eng = std::make_unique<oab::OffloadEngine>(
        (int)device, reinterpret_cast<cudaStream_t>(compute), reinterpret_cast<cudaStream_t>(h2d),
        reinterpret_cast<cudaStream_t>(d2h), workspace.data_ptr(),
        (size_t)workspace.numel() * workspace.element_size(), o, (int)n_tensors);
  }
  int64_t staged_step(int64_t pid, int64_t mode, const OptT& p, const OptT& g, const OptT& host_grad,
                      const Tensor& m, const Tensor& v, const OptT& extra, double lr, double wd, double b1h,
                      double b2h, double eps, bool decoupled, const OptT& clip, int64_t seed,
                      int64_t elem_offset, const OptT& amax, const std::vector<int64_t>& g_peers,
                      double g_scale, const std::vector<int64_t>& p_peers, const OptT& status, int64_t chunk,
                      const PyQuantSpec* quant, const OptT& master_copy) {
    TORCH_CHECK(!m.is_cuda() && !v.is_cuda(), "staged_step: state tensors must be pinned host tensors");
    oab::StagedStepArgs a;
    a.pid = (int)pid;
    oab::AdamStepArgs& k = a.k;
    k.mode = (int)mode;
    k.decoupled = decoupled;
    k.n = m.numel();
    if (p.has_value() && p->defined()) { TORCH_CHECK(p->is_cuda() && p->numel() == k.n, "p"); k.p = p->data_ptr(); }
    if (g.has_value() && g->defined()) { TORCH_CHECK(g->is_cuda() && g->numel() == k.n, "g"); k.g = g->data_ptr(); }
    if (host_grad.has_value() && host_grad->defined()) {
      TORCH_CHECK(!host_grad->is_cuda() && host_grad->numel() == k.n, "host_grad");
      a.host_grad = host_grad->data_ptr();
    }
    set_peers(k, g_peers, g_scale, p_peers, status);
    TORCH_CHECK(k.g != nullptr || a.host_grad != nullptr || k.n_g_peers > 0, "staged_step needs a gradient");
    k.m = m.data_ptr(); k.v = v.data_ptr();
    if (extra.has_value() && extra->defined()) k.extra = extra->data_ptr();
    k.lr = (float)lr; k.wd = (float)wd; k.beta1_hat = (float)b1h; k.beta2_hat = (float)b2h; k.eps = (float)eps;
    if (clip.has_value() && clip->defined()) k.clip_coef = clip->data_ptr<float>();
    k.seed = (uint64_t)seed;
    k.elem_offset = elem_offset;
    if (amax.has_value() && amax->defined()) k.amax_out = amax->data_ptr<float>();
    a.chunk = chunk;
    if (quant != nullptr) a.quant = &quant->q;
    if (master_copy.has_value() && master_copy->defined()) {
      TORCH_CHECK(master_copy->is_cuda() && master_copy->scalar_type() == at::kFloat && master_copy->numel() >= k.n,
                  "master_copy: CUDA fp32 of at least the tensor's size");
      a.master_copy = master_copy->data_ptr();
    }
    void* where = nullptr;
    {
      // may wait for staging space (write-backs issued by the helper thread)
      py::gil_scoped_release nogil;
      where = eng->staged_step(a);
    }
    return reinterpret_cast<int64_t>(where);
  }
  bool make_resident(int64_t pid, int64_t mode, int64_t n) { return eng->make_resident((int)pid, (int)mode, n); }
  bool is_resident(int64_t pid) const { return eng->is_resident((int)pid); }
  int64_t resident_bytes() const { return (int64_t)eng->resident_bytes(); }
  void staged_grad_to_host(int64_t pid, const Tensor& host_grad, const Tensor& dev_grad, bool first,
                           const OptT& sumsq, const OptT& scratch) {
    TORCH_CHECK(!host_grad.is_cuda() && dev_grad.is_cuda() && host_grad.numel() == dev_grad.numel(), "grad buffers");
    float* sq = (sumsq.has_value() && sumsq->defined()) ? sumsq->data_ptr<float>() : nullptr;
    float* sc = (scratch.has_value() && scratch->defined()) ? reinterpret_cast<float*>(scratch->data_ptr()) : nullptr;
    eng->staged_grad_to_host((int)pid, host_grad.data_ptr(), dev_grad.data_ptr(), dev_grad.numel(), first, sq, sc);
  }
  std::pair<int64_t, bool> prefetch(int64_t pid, int64_t mode, const OptT& host_grad, const Tensor& m,
                                    const Tensor& v, const OptT& extra, int64_t from_off,
                                    int64_t max_chunks, int64_t max_inflight, int64_t chunk) {
    TORCH_CHECK(!m.is_cuda() && !v.is_cuda(), "prefetch: state tensors must be pinned host tensors");
    oab::StagedStepArgs a;
    a.pid = (int)pid;
    a.k.mode = (int)mode;
    a.k.n = m.numel();
    a.k.m = m.data_ptr();
    a.k.v = v.data_ptr();
    if (extra.has_value() && extra->defined()) a.k.extra = extra->data_ptr();
    if (host_grad.has_value() && host_grad->defined()) a.host_grad = host_grad->data_ptr();
    a.chunk = chunk;
    bool full = false;
    int64_t off = eng->prefetch(a, from_off, max_chunks, (int)max_inflight, &full);
    return {off, full};
  }
  void start_prefetch(int64_t mode, const std::vector<std::tuple<int64_t, Tensor, Tensor, OptT, int64_t>>& items,
                      int64_t max_inflight) {
    std::vector<oab::OffloadEngine::PrefetchItem> plan;
    plan.reserve(items.size());
    for (const auto& it : items) {
      oab::OffloadEngine::PrefetchItem x;
      x.pid = (int)std::get<0>(it);
      x.mode = (int)mode;
      const Tensor& m = std::get<1>(it);
      const Tensor& v = std::get<2>(it);
      const OptT& extra = std::get<3>(it);
      TORCH_CHECK(!m.is_cuda() && !v.is_cuda() && m.is_contiguous() && v.is_contiguous(), "host state expected");
      x.n = m.numel();
      x.m = m.data_ptr();
      x.v = v.data_ptr();
      if (extra.has_value() && extra->defined()) x.extra = extra->data_ptr();
      x.chunk = std::get<4>(it);
      plan.push_back(x);
    }
    py::gil_scoped_release nogil;
    eng->start_prefetch(std::move(plan), (int)max_inflight);
  }
  void stop_prefetch() {
    py::gil_scoped_release nogil;
    eng->stop_prefetch();
  }
  void join(int64_t stream) {
    cudaStream_t s = pick_stream(stream);
    py::gil_scoped_release nogil;
    eng->join(s);
  }
  void join_compute(int64_t stream) { eng->join_compute(pick_stream(stream)); }
  void wait_host_grad(int64_t pid) { eng->wait_host_grad((int)pid); }
  void discard_prefetched() { eng->discard_prefetched(); }
  int64_t prefetched_chunks() const { return eng->prefetched_chunks(); }
  int64_t prefetched_bytes() const { return eng->prefetched_bytes(); }
  int64_t ring_bytes() const { return (int64_t)eng->ring_bytes(); }
  void synchronize() { py::gil_scoped_release nogil; eng->synchronize(); }
  void wait_writebacks() { py::gil_scoped_release nogil; eng->wait_writebacks(); }
  int64_t bytes_h2d() const { return eng->bytes_h2d(); }
  int64_t bytes_d2h() const { return eng->bytes_d2h(); }
  void reset_counters() { eng->reset_counters(); }
};

}  // namespace

void bind_quant(py::module_& m);
void bind_symm(py::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "offload_adam_b200 native runtime (sm_100a kernels, pinned arena, copy engine)";
  m.def("adam_step", &adam_step, py::arg("mode"), py::arg("p"), py::arg("g"), py::arg("g2"),
        py::arg("m"), py::arg("v"), py::arg("extra"), py::arg("lr"), py::arg("wd"),
        py::arg("beta1_hat"), py::arg("beta2_hat"), py::arg("eps"), py::arg("decoupled"),
        py::arg("clip") = py::none(), py::arg("seed") = 0, py::arg("elem_offset") = 0,
        py::arg("amax") = py::none(), py::arg("max_ctas") = 0, py::arg("stream") = 0,
        py::arg("g_peers") = std::vector<int64_t>(), py::arg("g_scale") = 1.0,
        py::arg("p_peers") = std::vector<int64_t>(), py::arg("status") = py::none(),
        py::arg("extra_copy") = py::none());
  m.def("grad_accumulate", &grad_accumulate, py::arg("out"), py::arg("a"), py::arg("b"),
        py::arg("sumsq") = py::none(), py::arg("sumsq_accumulate") = false,
        py::arg("scratch") = py::none(), py::arg("max_ctas") = 0, py::arg("stream") = 0);
  m.def("clip_finalize", &clip_finalize, py::arg("slots"), py::arg("index"), py::arg("extra_sq"),
        py::arg("max_norm"), py::arg("coef_norm"), py::arg("total_sq"), py::arg("stream") = 0);
  m.def("multi_tensor_adam", &multi_tensor_adam);
  m.def("multi_tensor_chunk", &oab::multi_tensor_chunk);
  m.def("sumsq_scratch_bytes", []() { return (int64_t)oab::kSumsqScratchBytes; });
  m.def("launch_count", []() { return (int64_t)oab::g_launch_count; });
  m.def("reset_launch_count", []() { oab::g_launch_count = 0; });

  m.def("gpu_numa_node", &oab::gpu_numa_node);
  m.def("numa_node_free_bytes", &oab::numa_node_free_bytes);
  m.def("numa_node_total_bytes", &oab::numa_node_total_bytes);
  m.def("numa_num_nodes", &oab::numa_num_nodes);
  m.def("pci_bus_id", &oab::pci_bus_id);
  m.def("arena_inject_failure", &oab::inject_failure);
  m.def("arena_reset_syscalls", &oab::reset_syscalls);

  py::class_<PyArena>(m, "PinnedArena")
      .def(py::init<const std::vector<int64_t>&, int64_t, bool, bool, int64_t, int64_t, int64_t>(),
           py::arg("sizes"), py::arg("numa_node") = -1, py::arg("register_cuda") = true,
           py::arg("huge_pages") = true, py::arg("touch_threads") = 0, py::arg("segment_bytes") = 0,
           py::arg("alignment") = 0)
      .def("tensor", &PyArena::tensor)
      .def("stats", &PyArena::stats);

  py::class_<PyQuantSpec>(m, "QuantSpec")
      .def(py::init<int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, const std::vector<int64_t>&,
                    const std::vector<int64_t>&, const OptT&, const OptT&>(),
           py::arg("format"), py::arg("out_f"), py::arg("in_f"), py::arg("row0"), py::arg("group"),
           py::arg("scale_dtype"), py::arg("payload0"), py::arg("payload1"), py::arg("tensor_amax") = py::none(),
           py::arg("global_scale") = py::none());
  m.def("adam_quant_supported", [](int64_t format, int64_t in_f, int64_t group) {
    return oab::adam_quant_supported((int)format, in_f, (int)group);
  });
  m.def("adam_quant_push", &adam_quant_push, py::arg("spec"), py::arg("g"), py::arg("g2"), py::arg("m"), py::arg("v"),
        py::arg("master"), py::arg("lr"), py::arg("wd"), py::arg("beta1_hat"), py::arg("beta2_hat"), py::arg("eps"),
        py::arg("decoupled"), py::arg("clip") = py::none(), py::arg("max_ctas") = 0, py::arg("stream") = 0,
        py::arg("g_peers") = std::vector<int64_t>(), py::arg("g_scale") = 1.0, py::arg("status") = py::none());
  m.def("nvfp4_quantize_push", &nvfp4_quantize_push, py::arg("spec"), py::arg("master_ptr"), py::arg("n"),
        py::arg("status") = py::none(), py::arg("stream") = 0);
  m.attr("QFMT_NVFP4") = (int)oab::kQNVFP4;
  m.attr("QFMT_NF4") = (int)oab::kQNF4;
  m.attr("QFMT_INT4") = (int)oab::kQInt4;
  m.attr("QFMT_INT8") = (int)oab::kQInt8;
  m.attr("QDT_F32") = (int)oab::kF32;
  m.attr("QDT_BF16") = (int)oab::kBF16;
  m.attr("QDT_F16") = (int)oab::kF16;

  py::class_<PyEngine>(m, "OffloadEngine")
      .def(py::init<int64_t, int64_t, int64_t, int64_t, Tensor, int64_t, int64_t, int64_t, bool, bool, bool>(),
           py::arg("device"), py::arg("compute"), py::arg("h2d"), py::arg("d2h"), py::arg("workspace"),
           py::arg("chunk_elems"), py::arg("max_ctas"), py::arg("n_tensors"), py::arg("async_writeback"),
           py::arg("canaries") = false, py::arg("lazy_resident") = false)
      .def_static("min_ring_bytes", [](int64_t chunk_elems) {
        return (int64_t)oab::OffloadEngine::min_ring_bytes(chunk_elems);
      })
      .def("staged_step", &PyEngine::staged_step, py::arg("pid"), py::arg("mode"), py::arg("p"),
           py::arg("g"), py::arg("host_grad"), py::arg("m"), py::arg("v"), py::arg("extra"),
           py::arg("lr"), py::arg("wd"), py::arg("beta1_hat"), py::arg("beta2_hat"), py::arg("eps"),
           py::arg("decoupled"), py::arg("clip"), py::arg("seed"), py::arg("elem_offset"),
           py::arg("amax"), py::arg("g_peers") = std::vector<int64_t>(), py::arg("g_scale") = 1.0,
           py::arg("p_peers") = std::vector<int64_t>(), py::arg("status") = py::none(), py::arg("chunk") = 0,
           py::arg("quant") = nullptr, py::arg("master_copy") = py::none())
      .def("make_resident", &PyEngine::make_resident)
      .def("is_resident", &PyEngine::is_resident)
      .def("resident_bytes", &PyEngine::resident_bytes)
      .def("staged_grad_to_host", &PyEngine::staged_grad_to_host)
      .def("prefetch", &PyEngine::prefetch, py::arg("pid"), py::arg("mode"), py::arg("host_grad"), py::arg("m"),
           py::arg("v"), py::arg("extra"), py::arg("from_off"), py::arg("max_chunks"), py::arg("max_inflight"),
           py::arg("chunk") = 0)
      .def("join", &PyEngine::join)
      .def("join_compute", &PyEngine::join_compute)
      .def("wait_host_grad", &PyEngine::wait_host_grad)
      .def("discard_prefetched", &PyEngine::discard_prefetched)
      .def("wait_writebacks", &PyEngine::wait_writebacks)
      .def("start_prefetch", &PyEngine::start_prefetch)
      .def("stop_prefetch", &PyEngine::stop_prefetch)
      .def("prefetched_chunks", &PyEngine::prefetched_chunks)
      .def("prefetched_bytes", &PyEngine::prefetched_bytes)
      .def("ring_bytes", &PyEngine::ring_bytes)
      .def("synchronize", &PyEngine::synchronize)
      .def("bytes_h2d", &PyEngine::bytes_h2d)
      .def("bytes_d2h", &PyEngine::bytes_d2h)
      .def("reset_counters", &PyEngine::reset_counters);

  bind_quant(m);
  bind_symm(m);
}
