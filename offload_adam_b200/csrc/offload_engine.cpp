#include "offload_engine.h"

#include <chrono>
#include <stdexcept>
#include <string>

#include "grad_ops.h"

namespace oab {

namespace {
// Host-side waits on the helper threads are bounded as well: a wait that sees no progress
// for this long reports an error instead of hanging the training process.
constexpr auto kHostWaitLimit = std::chrono::seconds(300);

size_t elem_extra_bytes(int mode) {
  return mode == kModeFP32Master ? 4 : (mode == kModeSR ? 0 : 2);
}
size_t up256(size_t x) { return (x + 255) / 256 * 256; }
}  // namespace

size_t OffloadEngine::min_ring_bytes(int64_t chunk_elems) {
  // three full-width chunks (g, m, v, fp32 extra) so that load, compute and
  // write-back of consecutive chunks overlap
  // (+ room for the guard words of the debugging option and its status block)
  return 3 * (up256(2 * chunk_elems) * 3 + up256(4 * chunk_elems)) + 8 * 256;
}

void OffloadEngine::check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("OffloadEngine: ") + what + ": " + cudaGetErrorString(e));
}

OffloadEngine::OffloadEngine(int device, cudaStream_t compute, cudaStream_t h2d, cudaStream_t d2h,
                             void* workspace, size_t ws_bytes, const EngineOptions& opt,
                             int n_tensors)
    : device_(device), compute_(compute), h2d_(h2d), d2h_(d2h), opt_(opt),
      res_(n_tensors > 0 ? (size_t)n_tensors : 0) {
  if (opt_.chunk_elems % 16 != 0 || opt_.chunk_elems <= 0)
    throw std::invalid_argument("OffloadEngine: chunk_elems must be a positive multiple of 16");
  if (ws_bytes < min_ring_bytes(opt_.chunk_elems))
    throw std::invalid_argument("OffloadEngine: staging buffer smaller than min_ring_bytes(chunk_elems)");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    throw std::invalid_argument("OffloadEngine: staging buffer must be 256-byte aligned");
  ring_ = static_cast<char*>(workspace);
  ring_bytes_ = ws_bytes / 256 * 256;
  if (opt_.canaries) {
    if (ring_bytes_ < min_ring_bytes(opt_.chunk_elems) + 4 * kGuardBytes)
      throw std::invalid_argument("OffloadEngine: staging buffer too small for canaries");
    ring_bytes_ -= 256;
    canary_status_ = reinterpret_cast<int*>(ring_ + ring_bytes_);
    check(cudaMemsetAsync(canary_status_, 0, 256, compute_), "clear canary status");
  }
  host_ready_.resize(n_tensors, nullptr);
  host_ready_set_.assign(n_tensors, 0);
  grad_ready_.resize(n_tensors, nullptr);
  grad_ready_set_.assign(n_tensors, 0);
  for (auto& e : host_ready_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  for (auto& e : grad_ready_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  check(cudaEventCreateWithFlags(&tmp_ev_, cudaEventDisableTiming), "event");
  for (auto& e : join_ev_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  wb_submitted_.assign(n_tensors, 0);
  wb_issued_.reset(new std::atomic<int64_t>[n_tensors > 0 ? n_tensors : 1]);
  for (int i = 0; i < n_tensors; ++i) wb_issued_[i].store(0);
  for (auto& e : wb_throttle_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  if (opt_.async_writeback) writer_ = std::thread([this] { writer_loop(); });
  loader_ = std::thread([this] { loader_loop(); });
}

OffloadEngine::~OffloadEngine() {
  if (loader_.joinable()) {
    pf_stop_.store(true);
    {
      std::lock_guard<std::mutex> lk(pf_mu_);
      pf_exit_ = true;
    }
    pf_cv_.notify_all();
    loader_.join();
  }
  if (writer_.joinable()) {
    {
      std::lock_guard<std::mutex> lk(wb_mu_);
      wb_stop_ = true;
    }
    wb_cv_.notify_all();
    writer_.join();
  }
  // copies already enqueued still read and write the staging buffer and the host
  // state; let them finish before the owner releases either (errors are ignored: at
  // interpreter shutdown the context may be gone)
  (void)cudaStreamSynchronize(compute_);
  (void)cudaStreamSynchronize(h2d_);
  (void)cudaStreamSynchronize(d2h_);
  (void)cudaGetLastError();
  for (auto& e : all_events_) cudaEventDestroy(e);
  for (auto& e : wb_throttle_) if (e) cudaEventDestroy(e);
  for (auto& e : host_ready_) if (e) cudaEventDestroy(e);
  for (auto& e : grad_ready_) if (e) cudaEventDestroy(e);
  if (tmp_ev_) cudaEventDestroy(tmp_ev_);
  for (auto& e : join_ev_) if (e) cudaEventDestroy(e);
}

cudaEvent_t OffloadEngine::take_event() {
  if (!pool_.empty()) {
    cudaEvent_t e = pool_.back();
    pool_.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  all_events_.push_back(e);
  return e;
}

// ---------------------------------------------------------------- write-backs
void OffloadEngine::issue_writeback(const WbJob& j, cudaError_t* err) {
  cudaError_t e = cudaStreamWaitEvent(d2h_, j.k_done, 0);
  for (int i = 0; i < j.n && e == cudaSuccess; ++i)
    e = cudaMemcpyAsync(j.host[i], j.dev[i], j.bytes[i], cudaMemcpyDeviceToHost, d2h_);
  if (e == cudaSuccess) e = cudaEventRecord(j.free_ev, d2h_);
  if (e == cudaSuccess && j.pid >= 0) e = cudaEventRecord(host_ready_[j.pid], d2h_);
  // retire even after an error: nobody may wait for this chunk forever
  j.e->retired.store(true, std::memory_order_release);
  if (j.pid >= 0) wb_issued_[j.pid].fetch_add(1, std::memory_order_release);
  *err = e;
}

void OffloadEngine::submit_writeback(const WbJob& j) {
  if (j.pid >= 0) {
    ++wb_submitted_[j.pid];
    host_ready_set_[j.pid] = 1;
  }
  if (!writer_.joinable()) {
    cudaError_t e = cudaSuccess;
    issue_writeback(j, &e);
    check(e, "write-back");
    return;
  }
  j.e->queued = true;
  {
    std::lock_guard<std::mutex> lk(wb_mu_);
    if (!wb_error_.empty()) throw std::runtime_error("OffloadEngine: write-back failed: " + wb_error_);
    wb_q_.push_back(j);
  }
  wb_cv_.notify_one();
}

void OffloadEngine::writer_loop() {
  cudaSetDevice(device_);
  for (;;) {
    WbJob j;
    {
      std::unique_lock<std::mutex> lk(wb_mu_);
      wb_cv_.wait(lk, [&] { return wb_stop_ || !wb_q_.empty(); });
      if (wb_q_.empty()) return;  // stop requested and everything issued
      j = wb_q_.front();
      wb_q_.pop_front();
      wb_busy_ = true;
    }
    // throttle: a new group of jobs may start once the group issued kWbGroups groups
    // earlier has completed on the device (poll and sleep, never block in the driver)
    const int group = (int)((wb_jobs_ / kWbGroup) % kWbGroups);
    if (wb_jobs_ % kWbGroup == 0 && wb_throttle_used_[group]) {
      for (;;) {
        const cudaError_t q = cudaEventQuery(wb_throttle_[group]);
        if (q != cudaErrorNotReady) break;  // done (or failed: the issue below reports it)
        (void)cudaGetLastError();
        std::this_thread::sleep_for(std::chrono::microseconds(100));
      }
      (void)cudaGetLastError();
      wb_throttle_used_[group] = false;
    }
    cudaError_t e = cudaSuccess;
    issue_writeback(j, &e);
    if (wb_jobs_ % kWbGroup == kWbGroup - 1 && e == cudaSuccess &&
        cudaEventRecord(wb_throttle_[group], d2h_) == cudaSuccess)
      wb_throttle_used_[group] = true;
    ++wb_jobs_;
    {
      std::lock_guard<std::mutex> lk(wb_mu_);
      wb_busy_ = false;
      if (e != cudaSuccess && wb_error_.empty()) wb_error_ = cudaGetErrorString(e);
      if (wb_q_.empty()) wb_idle_cv_.notify_all();
    }
  }
}

void OffloadEngine::drain_writer() {
  if (!writer_.joinable()) return;
  std::unique_lock<std::mutex> lk(wb_mu_);
  // progress is one issued job; the limit applies to the time without any
  size_t seen = wb_q_.size();
  while (!(wb_q_.empty() && !wb_busy_)) {
    if (!wb_idle_cv_.wait_for(lk, kHostWaitLimit, [&] { return (wb_q_.empty() && !wb_busy_) || wb_q_.size() != seen; }))
      throw std::runtime_error("OffloadEngine: the write-back thread made no progress for 300 s");
    seen = wb_q_.size();
  }
  if (!wb_error_.empty()) throw std::runtime_error("OffloadEngine: write-back failed: " + wb_error_);
}

void OffloadEngine::discard_prefetched() {
  stop_prefetch();
  // resident state the host has not seen yet goes back first (lazy write-back): the
  // reload below then reads it again, and no step is ever lost
  flush_resident();
  discard_impl();
  // the host copy may change behind the engine's back from here on: resident state is
  // loaded again at its next step, behind the write-back above
  for (Resident& r : res_) r.loaded = false;
}

void OffloadEngine::discard_impl() {
  // the chunks stay where they are until their space is needed; nothing reads them
  for (Entry* e : loaded_) e->retired.store(true, std::memory_order_release);
  loaded_.clear();
  inflight_.clear();
  loaded_bytes_ = 0;
}

// Circular allocation.  Live chunks occupy the buffer in allocation order, so the
// chunks a new allocation runs into are always the oldest ones; they can be evicted
// once their write-back has been issued (the H2D stream then waits for it to finish).
void OffloadEngine::arm_guard(char* guard, cudaStream_t stream) {
  if (guard != nullptr) check(cudaMemsetAsync(guard, 0xA5, kGuardBytes, stream), "arm canary");
}

void OffloadEngine::verify_guard(const char* guard, int pid) {
  if (guard != nullptr)
    check(launch_check_canary(guard, (int)(kGuardBytes / 4), canary_status_, pid, compute_), "check canary");
}

void OffloadEngine::check_canaries() {
  if (canary_status_ == nullptr) return;
  int host[2] = {0, 0};
  check(cudaMemcpyAsync(host, canary_status_, sizeof(host), cudaMemcpyDeviceToHost, compute_), "read canary status");
  check(cudaStreamSynchronize(compute_), "sync compute");
  if (host[0] != 0)
    throw std::runtime_error("OffloadEngine: a kernel wrote past the staging chunk (or resident buffers) of tensor " +
                             std::to_string(host[1]) + ": the guard words behind it were overwritten");
}

OffloadEngine::Entry* OffloadEngine::allocate(size_t bytes, bool may_discard) {
  bytes = up256(bytes);
  const size_t content = bytes;
  if (opt_.canaries) bytes += kGuardBytes;
  if (bytes > ring_bytes_) throw std::runtime_error("OffloadEngine: chunk larger than the staging buffer");
  for (int attempt = 0; attempt < 2; ++attempt) {
    size_t start = head_;
    bool wrapped = false;
    if (start + bytes > ring_bytes_) { start = 0; wrapped = true; }
    const size_t end = start + bytes;
    auto overlaps = [&](const Entry& e) {
      return (e.off < end && start < e.off + e.bytes) || (wrapped && e.off >= head_);
    };
    bool blocked = false;
    for (const Entry& e : live_) {
      if (!overlaps(e)) break;
      if (e.queued) {
        // its write-back is with the helper thread: it will be issued, wait for that
        const auto deadline = std::chrono::steady_clock::now() + kHostWaitLimit;
        while (!e.retired.load(std::memory_order_acquire)) {
          std::this_thread::sleep_for(std::chrono::microseconds(20));  // chunks take milliseconds
          if (std::chrono::steady_clock::now() > deadline)
            throw std::runtime_error("OffloadEngine: the write-back thread made no progress for 300 s");
        }
      }
      if (!e.retired.load(std::memory_order_acquire)) { blocked = true; break; }
    }
    if (blocked) {
      if (may_discard && !loaded_.empty()) { discard_impl(); continue; }
      return nullptr;
    }
    while (!live_.empty() && overlaps(live_.front())) {
      Entry& old = live_.front();
      check(cudaStreamWaitEvent(h2d_, old.free_ev, 0), "wait for staging space");
      for (auto it = inflight_.begin(); it != inflight_.end();)
        it = (*it == &old) ? inflight_.erase(it) : it + 1;
      pool_.push_back(old.h2d_done);
      pool_.push_back(old.k_done);
      pool_.push_back(old.free_ev);
      live_.pop_front();
    }
    live_.emplace_back();
    Entry& e = live_.back();
    e.off = start;
    e.bytes = bytes;
    e.h2d_done = take_event();
    e.k_done = take_event();
    e.free_ev = take_event();
    e.guard = opt_.canaries ? ring_ + start + content : nullptr;
    head_ = end;
    return &e;
  }
  return nullptr;
}

void OffloadEngine::wait_host_copy(const StagedStepArgs& a) {
  // the host copy must be complete: the previous write-back of this tensor
  if (a.pid >= 0 && a.pid < (int)host_ready_.size() && host_ready_set_[a.pid]) {
    // the event must have been recorded by the helper thread before it can be waited for
    const auto deadline = std::chrono::steady_clock::now() + kHostWaitLimit;
    while (wb_issued_[a.pid].load(std::memory_order_acquire) < wb_submitted_[a.pid]) {
      std::this_thread::sleep_for(std::chrono::microseconds(20));
      if (std::chrono::steady_clock::now() > deadline)
        throw std::runtime_error("OffloadEngine: the write-back thread made no progress for 300 s");
    }
    check(cudaStreamWaitEvent(h2d_, host_ready_[a.pid], 0), "wait host_ready");
  }
  if (a.host_grad && a.pid >= 0 && a.pid < (int)grad_ready_.size() && grad_ready_set_[a.pid])
    check(cudaStreamWaitEvent(h2d_, grad_ready_[a.pid], 0), "wait grad_ready");
}

OffloadEngine::Entry* OffloadEngine::load_chunk(const StagedStepArgs& a, int64_t off, int64_t len,
                                                bool may_discard) {
  const AdamStepArgs& k = a.k;
  const size_t xb = elem_extra_bytes(k.mode);
  const size_t gb = a.host_grad ? up256(2 * len) : 0;
  const size_t sb = up256(2 * len);
  Entry* e = allocate(gb + 2 * sb + up256(xb * len), may_discard);
  if (e == nullptr) return nullptr;
  char* base = ring_ + e->off;
  e->g = base;
  e->m = base + gb;
  e->v = e->m + sb;
  e->x = e->v + sb;
  if (a.host_grad) {
    check(cudaMemcpyAsync(e->g, (const char*)a.host_grad + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d g");
    bytes_h2d_ += 2 * len;
  }
  check(cudaMemcpyAsync(e->m, (const char*)k.m + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d m");
  check(cudaMemcpyAsync(e->v, (const char*)k.v + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d v");
  bytes_h2d_ += 4 * len;
  if (xb) {
    check(cudaMemcpyAsync(e->x, (const char*)k.extra + xb * off, xb * len, cudaMemcpyHostToDevice, h2d_), "h2d x");
    bytes_h2d_ += xb * len;
  }
  arm_guard(e->guard, h2d_);
  check(cudaEventRecord(e->h2d_done, h2d_), "record");
  e->pid = a.pid;
  e->eoff = off;
  e->len = len;
  e->has_grad = a.host_grad != nullptr;
  return e;
}

// ------------------------------------------------------------- prefetch thread
void OffloadEngine::start_prefetch(std::vector<PrefetchItem> items, int max_inflight) {
  stop_prefetch();
  {
    std::lock_guard<std::mutex> lk(pf_mu_);
    pf_plan_ = std::move(items);
    pf_inflight_ = max_inflight > 0 ? max_inflight : 1;
    pf_has_plan_ = true;
    pf_active_.store(true);
  }
  pf_cv_.notify_all();
}

void OffloadEngine::stop_prefetch() {
  if (!pf_active_.load()) return;
  pf_stop_.store(true);
  std::string err;
  {
    std::unique_lock<std::mutex> lk(pf_mu_);
    pf_has_plan_ = false;
    pf_plan_.clear();
    if (!pf_idle_cv_.wait_for(lk, kHostWaitLimit, [&] { return !pf_running_; }))
      throw std::runtime_error("OffloadEngine: the prefetch thread did not stop within 300 s");
    err.swap(pf_error_);
  }
  pf_stop_.store(false);
  pf_active_.store(false);
  if (!err.empty()) throw std::runtime_error("OffloadEngine: prefetch failed: " + err);
}

void OffloadEngine::loader_loop() {
  cudaSetDevice(device_);
  for (;;) {
    std::vector<PrefetchItem> plan;
    int inflight = 1;
    {
      std::unique_lock<std::mutex> lk(pf_mu_);
      pf_cv_.wait(lk, [&] { return pf_exit_ || pf_has_plan_; });
      if (pf_exit_) return;
      plan.swap(pf_plan_);
      pf_has_plan_ = false;
      pf_running_ = true;
      inflight = pf_inflight_;
    }
    std::string err;
    try {
      bool done = false;
      for (size_t i = 0; i < plan.size() && !done; ++i) {
        StagedStepArgs a;
        a.pid = plan[i].pid;
        a.k.mode = plan[i].mode;
        a.k.n = plan[i].n;
        a.k.m = plan[i].m;
        a.k.v = plan[i].v;
        a.k.extra = plan[i].extra;
        a.chunk = plan[i].chunk;
        int64_t off = 0;
        while (off < a.k.n) {
          if (pf_stop_.load()) { done = true; break; }
          bool full = false;
          const int64_t now = prefetch_impl(a, off, 0, inflight, &full);
          if (full) { done = true; break; }
          if (now == off) std::this_thread::sleep_for(std::chrono::microseconds(200));
          off = now;
        }
      }
    } catch (const std::exception& ex) {
      err = ex.what();
    }
    {
      std::lock_guard<std::mutex> lk(pf_mu_);
      pf_running_ = false;
      if (!err.empty()) pf_error_ = err;
    }
    pf_idle_cv_.notify_all();
  }
}

int64_t OffloadEngine::prefetch(const StagedStepArgs& a, int64_t from_off, int64_t max_chunks,
                                int max_inflight, bool* full) {
  stop_prefetch();
  return prefetch_impl(a, from_off, max_chunks, max_inflight, full);
}

int64_t OffloadEngine::prefetch_impl(const StagedStepArgs& a, int64_t from_off, int64_t max_chunks,
                                     int max_inflight, bool* full) {
  const AdamStepArgs& k = a.k;
  const int64_t C = chunk_of(a);
  int64_t off = from_off, issued = 0;
  bool waited = false;
  if (full) *full = false;
  if (is_resident(a.pid)) {
    // loaded once; afterwards there is nothing to bring in for this tensor
    Resident& r = res_[a.pid];
    if (!r.loaded) load_resident(a, r);
    return k.n;
  }
  while (off < k.n && (max_chunks <= 0 || issued < max_chunks)) {
    if (max_inflight > 0) {
      while (!inflight_.empty() && cudaEventQuery(inflight_.front()->h2d_done) == cudaSuccess)
        inflight_.pop_front();
      (void)cudaGetLastError();  // cudaErrorNotReady is not an error
      if ((int)inflight_.size() >= max_inflight) break;
    }
    if (!waited) { wait_host_copy(a); waited = true; }
    const int64_t len = (k.n - off < C) ? (k.n - off) : C;
    Entry* e = load_chunk(a, off, len, /*may_discard=*/false);
    if (e == nullptr) {
      if (full) *full = true;
      break;
    }
    loaded_.push_back(e);
    loaded_bytes_ += e->bytes;
    if (max_inflight > 0) inflight_.push_back(e);
    off += len;
    ++issued;
  }
  return off;
}

cudaError_t OffloadEngine::launch_chunk(const StagedStepArgs& a, const AdamStepArgs& c, int64_t off) {
  if (a.quant == nullptr) return launch_adam_step(c, compute_);
  if (a.quant->format == kQNVFP4) return launch_adam_step(c, compute_);  // quantized by a later pass
  QuantPushArgs q = *a.quant;
  q.row0 = a.quant->row0 + off / q.in_f;
  return launch_adam_quant_push(c, q, compute_);
}

bool OffloadEngine::make_resident(int pid, int mode, int64_t n) {
  if (pid < 0 || pid >= (int)res_.size() || n <= 0) return false;
  if (res_[pid].on) return true;
  stop_prefetch();
  if (!live_.empty() || head_ != 0)
    throw std::runtime_error("OffloadEngine: make_resident after the staging buffer came into use");
  const size_t xb = elem_extra_bytes(mode);
  const size_t need = 2 * up256(2 * n) + up256(xb * n) + (opt_.canaries ? kGuardBytes : 0);
  if (need + min_ring_bytes(opt_.chunk_elems) + (opt_.canaries ? kGuardBytes : 0) > ring_bytes_) return false;
  Resident& r = res_[pid];
  r.on = true;
  r.loaded = false;
  r.mode = mode;
  r.n = n;
  r.m = ring_;
  r.v = r.m + up256(2 * n);
  r.x = r.v + up256(2 * n);
  r.guard = opt_.canaries ? r.x + up256(xb * n) : nullptr;
  r.h2d_done = take_event();
  r.k_done = take_event();
  r.free_ev = take_event();
  ring_ += need;
  ring_bytes_ -= need;
  res_bytes_ += need;
  return true;
}

void OffloadEngine::load_resident(const StagedStepArgs& a, Resident& r) {
  const AdamStepArgs& k = a.k;
  const size_t xb = elem_extra_bytes(k.mode);
  if (k.n != r.n || k.mode != r.mode) throw std::runtime_error("OffloadEngine: resident tensor changed size or mode");
  wait_host_copy(a);
  check(cudaMemcpyAsync(r.m, k.m, 2 * r.n, cudaMemcpyHostToDevice, h2d_), "h2d m");
  check(cudaMemcpyAsync(r.v, k.v, 2 * r.n, cudaMemcpyHostToDevice, h2d_), "h2d v");
  if (xb) check(cudaMemcpyAsync(r.x, k.extra, xb * r.n, cudaMemcpyHostToDevice, h2d_), "h2d x");
  bytes_h2d_ += (int64_t)((4 + xb) * r.n);
  arm_guard(r.guard, h2d_);
  check(cudaEventRecord(r.h2d_done, h2d_), "record");
  r.loaded = true;
}

void* OffloadEngine::step_resident(const StagedStepArgs& a, Resident& r) {
  const AdamStepArgs& k = a.k;
  const size_t xb = elem_extra_bytes(k.mode);
  if (a.host_grad != nullptr)
    throw std::runtime_error("OffloadEngine: resident tensors take their gradient from the device");
  const bool fresh = !r.loaded;
  if (fresh) load_resident(a, r);
  if (k.n != r.n || k.mode != r.mode) throw std::runtime_error("OffloadEngine: resident tensor changed size or mode");
  // the last load (first step after a (re)load) and the last write-back (it still reads
  // the buffers this step overwrites) come first
  check(cudaStreamWaitEvent(compute_, r.h2d_done, 0), "wait h2d");
  if (!fresh && host_ready_set_[a.pid]) {
    const auto deadline = std::chrono::steady_clock::now() + kHostWaitLimit;
    while (wb_issued_[a.pid].load(std::memory_order_acquire) < wb_submitted_[a.pid]) {
      std::this_thread::sleep_for(std::chrono::microseconds(20));
      if (std::chrono::steady_clock::now() > deadline)
        throw std::runtime_error("OffloadEngine: the write-back thread made no progress for 300 s");
    }
    check(cudaStreamWaitEvent(compute_, host_ready_[a.pid], 0), "wait write-back");
  }
  if (a.quant != nullptr && a.quant->format == kQNVFP4 && k.amax_out != nullptr)
    check(cudaMemsetAsync(k.amax_out, 0, sizeof(float), compute_), "clear amax");
  AdamStepArgs c = k;
  if (k.n_g_peers > 0) { c.g = nullptr; c.g2 = nullptr; }
  c.m = r.m; c.v = r.v; c.extra = xb ? r.x : nullptr;
  c.extra_copy = nullptr;  // the resident master is the device copy
  c.max_ctas = opt_.max_ctas;
  check(launch_chunk(a, c, 0), "adam_step");
  verify_guard(r.guard, a.pid);
  check(cudaEventRecord(r.k_done, compute_), "record");

  r.hm = k.m; r.hv = k.v; r.hx = xb ? k.extra : nullptr;
  if (opt_.lazy_resident) r.dirty = true;
  else writeback_resident(a.pid, r);
  return (a.quant != nullptr && a.quant->format == kQNVFP4) ? (void*)r.x : nullptr;
}

void OffloadEngine::writeback_resident(int pid, Resident& r) {
  const size_t xb = elem_extra_bytes(r.mode);
  WbJob j;
  r.wb.retired.store(false, std::memory_order_relaxed);
  j.e = &r.wb;
  j.k_done = r.k_done;
  j.free_ev = r.free_ev;
  j.host[0] = r.hm; j.dev[0] = r.m; j.bytes[0] = 2 * r.n;
  j.host[1] = r.hv; j.dev[1] = r.v; j.bytes[1] = 2 * r.n;
  j.n = 2;
  if (xb) { j.host[2] = r.hx; j.dev[2] = r.x; j.bytes[2] = xb * r.n; j.n = 3; }
  bytes_d2h_ += (int64_t)((4 + xb) * r.n);
  j.pid = pid;
  r.dirty = false;
  submit_writeback(j);
}

void OffloadEngine::flush_resident() {
  for (size_t i = 0; i < res_.size(); ++i)
    if (res_[i].on && res_[i].dirty) writeback_resident((int)i, res_[i]);
}

void* OffloadEngine::staged_step(const StagedStepArgs& a) {
  stop_prefetch();
  const AdamStepArgs& k = a.k;
  if (a.quant != nullptr) {
    if (k.mode != kModeFP32Master) throw std::invalid_argument("OffloadEngine: quantized weights need fp32_master");
    if (a.quant->in_f <= 0 || k.n % a.quant->in_f != 0 || chunk_of(a) % a.quant->in_f != 0)
      throw std::invalid_argument("OffloadEngine: chunks of a quantized weight must be whole rows");
  }
  if (is_resident(a.pid)) return step_resident(a, res_[a.pid]);
  const bool nvfp4 = a.quant != nullptr && a.quant->format == kQNVFP4;
  if (nvfp4 && a.master_copy == nullptr)
    throw std::invalid_argument("OffloadEngine: an NVFP4 step needs master_copy");
  const int64_t C = chunk_of(a);
  const size_t xb = elem_extra_bytes(k.mode);
  bool waited = false;
  // the step kernels of an NVFP4 weight combine max|master| with atomicMax: start from zero
  if (nvfp4 && k.amax_out != nullptr) check(cudaMemsetAsync(k.amax_out, 0, sizeof(float), compute_), "clear amax");
  for (int64_t off = 0; off < k.n; off += C) {
    const int64_t len = (k.n - off < C) ? (k.n - off) : C;
    Entry* e = nullptr;
    if (!loaded_.empty()) {
      Entry* f = loaded_.front();
      if (f->pid == a.pid && f->eoff == off && f->len == len && f->has_grad == (a.host_grad != nullptr)) {
        e = f;  // already on its way: prefetched
        loaded_.pop_front();
        loaded_bytes_ -= e->bytes;
      } else {
        discard_impl();  // out-of-order step: give the space back
      }
    }
    if (e == nullptr) {
      if (!waited) { wait_host_copy(a); waited = true; }
      e = load_chunk(a, off, len, /*may_discard=*/true);
      if (e == nullptr) throw std::runtime_error("OffloadEngine: staging buffer exhausted");
    }
    check(cudaStreamWaitEvent(compute_, e->h2d_done, 0), "wait h2d");

    AdamStepArgs c = k;
    c.n = len;
    c.elem_offset = k.elem_offset + off;
    c.p = k.p ? (char*)k.p + 2 * off : nullptr;
    if (k.n_g_peers > 0) { c.g = nullptr; c.g2 = nullptr; }
    else if (k.g && a.host_grad) { c.g = (const char*)k.g + 2 * off; c.g2 = e->g; }
    else if (k.g) { c.g = (const char*)k.g + 2 * off; c.g2 = nullptr; }
    else { c.g = e->g; c.g2 = nullptr; }
    c.m = e->m; c.v = e->v; c.extra = xb ? e->x : nullptr;
    c.extra_copy = nvfp4 ? (char*)a.master_copy + 4 * off : nullptr;
    c.max_ctas = opt_.max_ctas;
    for (int j = 0; j < k.n_g_peers; ++j) c.g_peers[j] = (const char*)k.g_peers[j] + 2 * off;
    for (int j = 0; j < k.n_p_peers; ++j) c.p_peers[j] = (char*)k.p_peers[j] + 2 * off;
    check(launch_chunk(a, c, off), "adam_step");
    verify_guard(e->guard, a.pid);
    check(cudaEventRecord(e->k_done, compute_), "record");

    WbJob j;
    j.e = e;
    j.k_done = e->k_done;
    j.free_ev = e->free_ev;
    j.host[0] = (char*)k.m + 2 * off; j.dev[0] = e->m; j.bytes[0] = 2 * len;
    j.host[1] = (char*)k.v + 2 * off; j.dev[1] = e->v; j.bytes[1] = 2 * len;
    j.n = 2;
    bytes_d2h_ += 4 * len;
    if (xb) {
      j.host[2] = (char*)k.extra + xb * off; j.dev[2] = e->x; j.bytes[2] = xb * len;
      j.n = 3;
      bytes_d2h_ += xb * len;
    }
    const bool last = off + C >= k.n;
    j.pid = (last && a.pid >= 0 && a.pid < (int)host_ready_.size()) ? a.pid : -1;
    submit_writeback(j);
  }
  return nvfp4 ? a.master_copy : nullptr;
}

void OffloadEngine::staged_grad_to_host(int pid, void* host_grad, const void* dev_grad, int64_t n,
                                        bool first, float* sumsq_out, float* scratch) {
  stop_prefetch();  // this call allocates staging space on the caller's thread
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
    Entry* e = allocate(2 * len, /*may_discard=*/true);
    if (e == nullptr) throw std::runtime_error("OffloadEngine: staging buffer exhausted");
    char* sg = ring_ + e->off;
    if (!first) {
      check(cudaMemcpyAsync(sg, (const char*)host_grad + 2 * off, 2 * len, cudaMemcpyHostToDevice, h2d_), "h2d g");
      bytes_h2d_ += 2 * len;
    }
    arm_guard(e->guard, h2d_);
    check(cudaEventRecord(e->h2d_done, h2d_), "record");
    check(cudaStreamWaitEvent(compute_, e->h2d_done, 0), "wait h2d");
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
    verify_guard(e->guard, pid);
    check(cudaEventRecord(e->k_done, compute_), "record");
    check(cudaStreamWaitEvent(d2h_, e->k_done, 0), "wait k");
    check(cudaMemcpyAsync((char*)host_grad + 2 * off, sg, 2 * len, cudaMemcpyDeviceToHost, d2h_), "d2h g");
    bytes_d2h_ += 2 * len;
    check(cudaEventRecord(e->free_ev, d2h_), "record");
    e->retired.store(true, std::memory_order_release);
    first_chunk = false;
  }
  if (tracked) {
    check(cudaEventRecord(grad_ready_[pid], d2h_), "record grad_ready");
    grad_ready_set_[pid] = 1;
  }
}

void OffloadEngine::wait_host_grad(int pid) {
  if (pid >= 0 && pid < (int)grad_ready_.size() && grad_ready_set_[pid])
    check(cudaStreamWaitEvent(compute_, grad_ready_[pid], 0), "wait grad_ready");
}

void OffloadEngine::join(cudaStream_t stream) {
  drain_writer();
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

void OffloadEngine::wait_writebacks() {
  flush_resident();
  drain_writer();
  check(cudaStreamSynchronize(d2h_), "sync d2h");
}

void OffloadEngine::synchronize() {
  stop_prefetch();
  flush_resident();
  drain_writer();
  check(cudaStreamSynchronize(compute_), "sync compute");
  check(cudaStreamSynchronize(h2d_), "sync h2d");
  check(cudaStreamSynchronize(d2h_), "sync d2h");
  check_canaries();
}

}  // namespace oab
