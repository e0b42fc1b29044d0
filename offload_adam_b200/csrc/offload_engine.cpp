#include "offload_engine.h"

#include <stdexcept>
#include <string>

#include "grad_ops.h"

namespace oab {

namespace {
size_t elem_extra_bytes(int mode) {
  return mode == kModeFP32Master ? 4 : (mode == kModeSR ? 0 : 2);
}
}  // namespace

size_t OffloadEngine::workspace_bytes(const EngineOptions& opt) {
  // g, m, v (bf16) + widest extra (fp32) per element
  return (size_t)opt.slots * (size_t)opt.chunk_elems * 10;
}

void OffloadEngine::check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("OffloadEngine: ") + what + ": " + cudaGetErrorString(e));
}

OffloadEngine::OffloadEngine(int device, cudaStream_t compute, cudaStream_t h2d, cudaStream_t d2h,
                             void* workspace, size_t ws_bytes, const EngineOptions& opt,
                             int n_tensors)
    : device_(device), compute_(compute), h2d_(h2d), d2h_(d2h), opt_(opt) {
  if (opt_.chunk_elems % 8 != 0 || opt_.chunk_elems <= 0)
    throw std::invalid_argument("OffloadEngine: chunk_elems must be a positive multiple of 8");
  if (opt_.slots < 2) throw std::invalid_argument("OffloadEngine: need at least 2 slots");
  if (ws_bytes < workspace_bytes(opt_))
    throw std::invalid_argument("OffloadEngine: workspace too small");
  slot_bytes_ = (size_t)opt_.chunk_elems * 10;
  slots_.resize(opt_.slots);
  for (int i = 0; i < opt_.slots; ++i) {
    slots_[i].base = (char*)workspace + (size_t)i * slot_bytes_;
    check(cudaEventCreateWithFlags(&slots_[i].h2d_done, cudaEventDisableTiming), "event");
    check(cudaEventCreateWithFlags(&slots_[i].k_done, cudaEventDisableTiming), "event");
    check(cudaEventCreateWithFlags(&slots_[i].free_ev, cudaEventDisableTiming), "event");
  }
  host_ready_.resize(n_tensors, nullptr);
  host_ready_set_.assign(n_tensors, 0);
  for (auto& e : host_ready_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  grad_ready_.resize(n_tensors, nullptr);
  grad_ready_set_.assign(n_tensors, 0);
  for (auto& e : grad_ready_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  check(cudaEventCreateWithFlags(&tmp_ev_, cudaEventDisableTiming), "event");
  for (auto& e : join_ev_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
}

OffloadEngine::~OffloadEngine() {
  for (auto& s : slots_) {
    if (s.h2d_done) cudaEventDestroy(s.h2d_done);
    if (s.k_done) cudaEventDestroy(s.k_done);
    if (s.free_ev) cudaEventDestroy(s.free_ev);
  }
  for (auto& e : host_ready_) if (e) cudaEventDestroy(e);
  for (auto& e : grad_ready_) if (e) cudaEventDestroy(e);
  if (tmp_ev_) cudaEventDestroy(tmp_ev_);
  for (auto& e : join_ev_) if (e) cudaEventDestroy(e);
}

OffloadEngine::Slot& OffloadEngine::next_slot() {
  // never hand out a slot that still holds prefetched, unconsumed state
  if (!loaded_.empty() && loaded_.front() == cursor_) discard_prefetched();
  Slot& s = slots_[cursor_];
  cursor_ = (cursor_ + 1) % (int)slots_.size();
  return s;
}

void OffloadEngine::load_chunk(Slot& s, const StagedStepArgs& a, int64_t off, int64_t len) {
  const AdamStepArgs& k = a.k;
  const int64_t C = opt_.chunk_elems;
  const size_t xb = elem_extra_bytes(k.mode);
  char* sg = s.base;
  char* sm = s.base + 2 * C;
  char* sv = s.base + 4 * C;
  char* sx = s.base + 6 * C;
  if (s.used) check(cudaStreamWaitEvent(h2d_, s.free_ev, 0), "wait slot");
  if (a.host_grad) {
    check(cudaMemcpyAsync(sg, (const char*)a.host_grad + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d g");
    bytes_h2d_ += 2 * len;
  }
  check(cudaMemcpyAsync(sm, (const char*)k.m + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d m");
  check(cudaMemcpyAsync(sv, (const char*)k.v + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d v");
  bytes_h2d_ += 4 * len;
  if (xb) {
    check(cudaMemcpyAsync(sx, (const char*)k.extra + xb * off, xb * len, cudaMemcpyHostToDevice, h2d_), "h2d x");
    bytes_h2d_ += xb * len;
  }
  check(cudaEventRecord(s.h2d_done, h2d_), "record");
  s.used = true;
  s.pid = a.pid;
  s.off = off;
  s.len = len;
  s.has_grad = a.host_grad != nullptr;
}

void OffloadEngine::discard_prefetched() {
  loaded_.clear();
  inflight_.clear();
}

int64_t OffloadEngine::prefetch(const StagedStepArgs& a, int64_t from_off, int64_t max_chunks,
                                int max_inflight) {
  const AdamStepArgs& k = a.k;
  const int64_t C = opt_.chunk_elems;
  int64_t off = from_off;
  bool waited = false;
  int64_t issued = 0;
  while (off < k.n && (int)loaded_.size() < (int)slots_.size() - 1 &&
         (max_chunks <= 0 || issued < max_chunks)) {
    if (max_inflight > 0) {
      while (!inflight_.empty() && cudaEventQuery(slots_[inflight_.front()].h2d_done) == cudaSuccess)
        inflight_.pop_front();
      (void)cudaGetLastError();  // cudaErrorNotReady is not an error
      if ((int)inflight_.size() >= max_inflight) break;
    }
    ++issued;
    if (!waited) {
      // the host copy must be complete: previous step's write-back of this tensor
      if (a.pid >= 0 && a.pid < (int)host_ready_.size() && host_ready_set_[a.pid])
        check(cudaStreamWaitEvent(h2d_, host_ready_[a.pid], 0), "wait host_ready");
      if (a.host_grad && a.pid >= 0 && a.pid < (int)grad_ready_.size() && grad_ready_set_[a.pid])
        check(cudaStreamWaitEvent(h2d_, grad_ready_[a.pid], 0), "wait grad_ready");
      waited = true;
    }
    const int64_t len = (k.n - off < C) ? (k.n - off) : C;
    const int idx = cursor_;
    Slot& s = next_slot();
    load_chunk(s, a, off, len);
    loaded_.push_back(idx);
    if (max_inflight > 0) inflight_.push_back(idx);
    off += len;
  }
  return off;
}

void OffloadEngine::staged_step(const StagedStepArgs& a) {
  const AdamStepArgs& k = a.k;
  const int64_t C = opt_.chunk_elems;
  const size_t xb = elem_extra_bytes(k.mode);
  bool waited = false;
  for (int64_t off = 0; off < k.n; off += C) {
    const int64_t len = (k.n - off < C) ? (k.n - off) : C;
    Slot* sp = nullptr;
    if (!loaded_.empty()) {
      Slot& f = slots_[loaded_.front()];
      if (f.pid == a.pid && f.off == off && f.len == len && f.has_grad == (a.host_grad != nullptr)) {
        sp = &f;  // already on its way: prefetched
        loaded_.pop_front();
      } else {
        discard_prefetched();  // out-of-order step: give the slots back
      }
    }
    if (sp == nullptr) {
      if (!waited) {
        if (a.pid >= 0 && a.pid < (int)host_ready_.size() && host_ready_set_[a.pid])
          check(cudaStreamWaitEvent(h2d_, host_ready_[a.pid], 0), "wait host_ready");
        if (a.host_grad && a.pid >= 0 && a.pid < (int)grad_ready_.size() && grad_ready_set_[a.pid])
          check(cudaStreamWaitEvent(h2d_, grad_ready_[a.pid], 0), "wait grad_ready");
        waited = true;
      }
      sp = &next_slot();
      load_chunk(*sp, a, off, len);
    }
    Slot& s = *sp;
    char* sg = s.base;
    char* sm = s.base + 2 * C;
    char* sv = s.base + 4 * C;
    char* sx = s.base + 6 * C;
    check(cudaStreamWaitEvent(compute_, s.h2d_done, 0), "wait h2d");

    AdamStepArgs c = k;
    c.n = len;
    c.elem_offset = k.elem_offset + off;
    c.p = k.p ? (char*)k.p + 2 * off : nullptr;
    if (k.n_g_peers > 0) { c.g = nullptr; c.g2 = nullptr; }
    else if (k.g && a.host_grad) { c.g = (const char*)k.g + 2 * off; c.g2 = sg; }
    else if (k.g) { c.g = (const char*)k.g + 2 * off; c.g2 = nullptr; }
    else { c.g = sg; c.g2 = nullptr; }
    c.m = sm; c.v = sv; c.extra = xb ? sx : nullptr;
    c.max_ctas = opt_.max_ctas;
    for (int j = 0; j < k.n_g_peers; ++j) c.g_peers[j] = (const char*)k.g_peers[j] + 2 * off;
    for (int j = 0; j < k.n_p_peers; ++j) c.p_peers[j] = (char*)k.p_peers[j] + 2 * off;
    check(launch_adam_step(c, compute_), "adam_step");
    check(cudaEventRecord(s.k_done, compute_), "record");
    check(cudaStreamWaitEvent(d2h_, s.k_done, 0), "wait k");

    check(cudaMemcpyAsync((char*)k.m + 2 * off, sm, 2 * len, cudaMemcpyDeviceToHost, d2h_), "d2h m");
    check(cudaMemcpyAsync((char*)k.v + 2 * off, sv, 2 * len, cudaMemcpyDeviceToHost, d2h_), "d2h v");
    bytes_d2h_ += 4 * len;
    if (xb) {
      check(cudaMemcpyAsync((char*)k.extra + xb * off, sx, xb * len, cudaMemcpyDeviceToHost, d2h_), "d2h x");
      bytes_d2h_ += xb * len;
    }
    check(cudaEventRecord(s.free_ev, d2h_), "record");
  }
  if (a.pid >= 0 && a.pid < (int)host_ready_.size()) {
    check(cudaEventRecord(host_ready_[a.pid], d2h_), "record host_ready");
    host_ready_set_[a.pid] = 1;
  }
}

void OffloadEngine::staged_grad_to_host(int pid, void* host_grad, const void* dev_grad, int64_t n,
                                        bool first, float* sumsq_out, float* scratch) {
  const bool tracked = pid >= 0 && pid < (int)grad_ready_.size();
  const int64_t C = opt_.chunk_elems;
  if (first && sumsq_out == nullptr) {
    // nothing to add to: one DMA straight out of the gradient tensor
    check(cudaEventRecord(tmp_ev_, compute_), "record");
    check(cudaStreamWaitEvent(d2h_, tmp_ev_, 0), "wait");
    check(cudaMemcpyAsync(host_grad, dev_grad, 2 * n, cudaMemcpyDeviceToHost, d2h_), "d2h g");
    bytes_d2h_ += 2 * n;
    if (tracked) {
      check(cudaEventRecord(grad_ready_[pid], d2h_), "record grad_ready");
      grad_ready_set_[pid] = 1;
    }
    return;
  }
  if (!first && tracked && grad_ready_set_[pid])
    check(cudaStreamWaitEvent(h2d_, grad_ready_[pid], 0), "wait grad_ready");
  bool first_chunk = true;
  for (int64_t off = 0; off < n; off += C) {
    const int64_t len = (n - off < C) ? (n - off) : C;
    Slot& s = next_slot();
    char* sg = s.base;
    if (s.used) check(cudaStreamWaitEvent(h2d_, s.free_ev, 0), "wait slot");
    if (!first) {
      check(cudaMemcpyAsync(sg, (const char*)host_grad + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d g");
      bytes_h2d_ += 2 * len;
    }
    check(cudaEventRecord(s.h2d_done, h2d_), "record");
    check(cudaStreamWaitEvent(compute_, s.h2d_done, 0), "wait h2d");
    AccumArgs acc;
    acc.out = sg;
    acc.a = (const char*)dev_grad + 2 * off;
    acc.b = first ? nullptr : sg;
    acc.n = len;
    acc.sumsq_out = sumsq_out;
    acc.sumsq_accumulate = !first_chunk;
    acc.scratch = scratch;
    acc.max_ctas = opt_.max_ctas;
    check(launch_grad_accumulate(acc, compute_), "grad_accumulate");
    check(cudaEventRecord(s.k_done, compute_), "record");
    check(cudaStreamWaitEvent(d2h_, s.k_done, 0), "wait k");
    check(cudaMemcpyAsync((char*)host_grad + 2 * off, sg, 2 * len, cudaMemcpyDeviceToHost, d2h_), "d2h g");
    bytes_d2h_ += 2 * len;
    check(cudaEventRecord(s.free_ev, d2h_), "record");
    s.used = true;
    first_chunk = false;
  }
  if (tracked) {
    check(cudaEventRecord(grad_ready_[pid], d2h_), "record grad_ready");
    grad_ready_set_[pid] = 1;
  }
}

void OffloadEngine::join(cudaStream_t stream) {
  cudaStream_t src[3] = {compute_, h2d_, d2h_};
  for (int i = 0; i < 3; ++i) {
    check(cudaEventRecord(join_ev_[i], src[i]), "record join");
    check(cudaStreamWaitEvent(stream, join_ev_[i], 0), "wait join");
  }
}

void OffloadEngine::join_compute(cudaStream_t stream) {
  check(cudaEventRecord(join_ev_[0], compute_), "record join");
  check(cudaStreamWaitEvent(stream, join_ev_[0], 0), "wait join");
}

void OffloadEngine::synchronize() {
  check(cudaStreamSynchronize(compute_), "sync compute");
  check(cudaStreamSynchronize(h2d_), "sync h2d");
  check(cudaStreamSynchronize(d2h_), "sync d2h");
}

}  // namespace oab
