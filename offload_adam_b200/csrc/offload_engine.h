// Copy engine for optimizer state that lives in pinned host memory.
//
// Two ways of moving state through the step are provided; both run entirely on
// side streams so that they overlap the rest of backward:
//
//  * staged: each tensor is cut into chunks that flow through a byte-addressed
//    circular staging buffer in device memory: H2D (copy stream A) -> kernel
//    (compute stream) -> D2H (copy stream B).  Many chunks are in flight at any
//    time, so both DMA directions and the SMs work concurrently, and device memory
//    use is bounded by the size of the buffer, independent of tensor size.  A
//    chunk takes exactly the bytes it needs, so small tensors waste nothing.
//    The same buffer holds state brought in ahead of its step (prefetch) and state
//    whose write-back is still draining after the step.
//  * zero-copy: the kernel reads and writes the mapped host buffers itself; no
//    staging memory at all (see adam_step.h).  Issued directly by the caller.
//
// The reference moves whole tensors with one `.to(device)` / `copy_` per state
// on two side streams whose H2D side waits for the main stream at every hook
// (reference: src/offload_adam/offload_adam.py:347-372), so a transfer can
// neither start early nor overlap the kernel of the previous tensor.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "adam_quant.h"
#include "adam_step.h"

namespace oab {

struct EngineOptions {
  int64_t chunk_elems = int64_t(8) << 20;  // largest chunk, in elements
  int max_ctas = 0;                        // grid cap for kernels on the compute stream
  // Issue the D2H write-backs of a step from a helper thread.  A stream accepts only
  // a bounded number of pending operations (about a thousand); beyond that the
  // enqueueing call blocks.  A step of many chunks puts five operations per chunk on
  // the D2H stream, so with inline issue the caller stalls as soon as the kernels are
  // a couple of hundred chunks ahead of the write-backs, the remaining kernels are
  // launched at the pace of the D2H link and whatever the caller wanted to launch next
  // (the next forward pass) waits too.  With the helper thread only that thread blocks.
  bool async_writeback = true;
  // Debugging aid against kernels that write past their operands: every chunk in the staging
  // buffer (and every resident tensor) is followed by a 256-byte guard filled with a known
  // pattern; a small kernel verifies it after the chunk's kernel, and synchronize() raises
  // when a guard was overwritten (naming the tensor).  Costs one memset and one tiny launch
  // per chunk.
  bool canaries = false;
  // Resident state is copied back to the host only when somebody asks for the host copy
  // (wait_writebacks, synchronize) instead of after every step.
  bool lazy_resident = false;
};

struct StagedStepArgs {
  int pid = -1;          // slot in the per-tensor "host copy is up to date" event table
  AdamStepArgs k;        // p and (optionally) g are device pointers for the whole tensor;
                         // m/v/extra are the HOST pointers of the state
  const void* host_grad = nullptr;  // optional host-resident accumulated gradient
                                    // (added to k.g as the kernel's second term, or used
                                    // alone when k.g == nullptr)
  int64_t chunk = 0;                // elements per chunk of this tensor (0: the engine's
                                    // default); a multiple of in_f for quantized weights,
                                    // whose chunks must be whole rows
  // Quantized weight (fp32_master): the updated master is re-quantized and the packed
  // rows are stored into every replica in the same pass (adam_quant.h).  quant->row0 is
  // the first row of this tensor (or shard) within the weight.
  const QuantPushArgs* quant = nullptr;
  // NVFP4 only (its tensor scale needs the whole updated weight first): k.amax_out
  // receives max|master| and the updated master is kept on the device for the quantize
  // pass that follows, in this buffer of k.n floats unless the tensor is resident.
  void* master_copy = nullptr;
};

class OffloadEngine {
 public:
  // `workspace` is the staging buffer: workspace_bytes of device memory, 256-byte
  // aligned, at least min_ring_bytes(opt.chunk_elems).
  OffloadEngine(int device, cudaStream_t compute, cudaStream_t h2d, cudaStream_t d2h,
                void* workspace, size_t workspace_bytes, const EngineOptions& opt, int n_tensors);
  ~OffloadEngine();
  // Smallest staging buffer that can pipeline chunks of `chunk_elems` elements.
  static size_t min_ring_bytes(int64_t chunk_elems);

  // Adam step of one tensor through the staging buffer.  The caller has already
  // made the compute stream wait for the gradient producer.  Chunks that
  // prefetch() already brought in are consumed in place.  Returns the device address
  // at which the updated fp32 master of the whole tensor can be read by later work on
  // the compute stream when a.quant is NVFP4 (a.master_copy, or the resident copy),
  // nullptr otherwise.
  void* staged_step(const StagedStepArgs& a);

  // Resident tensors.  The front of the staging buffer can be given to the state of
  // chosen tensors for good: it is loaded once, every step runs as ONE launch on the
  // whole tensor and is followed by one write-back copy per state tensor, and no
  // byte of it crosses the host link towards the device again.  The host copy stays
  // current (it is written after every step) and authoritative (discard_prefetched()
  // makes the engine load it again).  Call before the first step or prefetch; returns
  // false, changing nothing, when the state does not fit in front of a ring of at
  // least min_ring_bytes.
  bool make_resident(int pid, int mode, int64_t n);
  bool is_resident(int pid) const { return pid >= 0 && pid < (int)res_.size() && res_[pid].on; }
  size_t resident_bytes() const { return res_bytes_; }

  // Early H2D: copies the host state (and host gradient, if given) of the tensor
  // into free staging space, chunk by chunk from `from_off`, before its gradient
  // exists.  Stops when the buffer is full, after `max_chunks` chunks (<= 0: no limit)
  // or, with max_inflight > 0, while that many earlier prefetch copies are still
  // running (checked with cudaEventQuery, never blocking), which bounds how long
  // somebody else's H2D copy can wait behind ours.  Returns the element offset up to
  // which the tensor is now loaded (== n when complete); *full is set when the buffer
  // could not take the next chunk.  Only the pid, mode, n and host pointers of `a` are
  // used.  Tensors must later be stepped in the order they were prefetched; a step
  // that finds other chunks at the head of the queue discards them (their H2D is
  // wasted, nothing else).
  int64_t prefetch(const StagedStepArgs& a, int64_t from_off, int64_t max_chunks, int max_inflight,
                   bool* full);
  // The same early H2D, driven by a helper thread instead of by calls from the
  // training loop: the thread walks `items` in order and keeps `max_inflight` chunk
  // copies outstanding (polling their events every 200 us) until the staging
  // buffer is full, the plan is done or stop_prefetch() is called.  Pacing then does
  // not depend on where the host thread is relative to the GPU.  Between
  // start_prefetch() and stop_prefetch() the helper thread owns the staging buffer;
  // every entry point that touches the buffer stops it first.
  struct PrefetchItem {
    int pid = -1;
    int mode = 0;
    int64_t n = 0;
    void *m = nullptr, *v = nullptr, *extra = nullptr;
    int64_t chunk = 0;  // as StagedStepArgs::chunk
  };
  void start_prefetch(std::vector<PrefetchItem> items, int max_inflight);
  void stop_prefetch();
  int64_t prefetched_chunks() const { return (int64_t)loaded_.size(); }
  int64_t prefetched_bytes() const { return (int64_t)loaded_bytes_; }
  void discard_prefetched();

  // host_grad (+)= dev_grad through the buffer, optionally producing sum of squares of
  // the result into *sumsq_out (device pointer).  first == true: plain D2H copy.
  void staged_grad_to_host(int pid, void* host_grad, const void* dev_grad, int64_t n, bool first,
                           float* sumsq_out, float* scratch);

  // Makes the compute stream wait for the last D2H copy into the host gradient buffer of
  // tensor `pid` (for kernels that read that pinned buffer directly).
  void wait_host_grad(int pid);

  // Makes `stream` wait until every transfer/kernel enqueued so far has finished.
  void join(cudaStream_t stream);
  // Makes `stream` wait for the kernels enqueued so far (parameters are updated) but
  // not for the trailing D2H write-backs of the state.
  void join_compute(cudaStream_t stream);
  // Blocks the host until the engine streams are idle (stops the prefetch thread,
  // issues every pending write-back first).
  void synchronize();
  // Blocks the host until the state of every step enqueued so far is back in host
  // memory; early loads keep running.
  void wait_writebacks();

  int64_t bytes_h2d() const { return bytes_h2d_; }
  int64_t bytes_d2h() const { return bytes_d2h_; }
  void reset_counters() { bytes_h2d_ = bytes_d2h_ = 0; }
  size_t ring_bytes() const { return ring_bytes_; }

 private:
  // One chunk resident in the staging buffer.
  struct Entry {
    size_t off = 0, bytes = 0;  // placement in the buffer
    cudaEvent_t h2d_done = nullptr, k_done = nullptr, free_ev = nullptr;
    std::atomic<bool> retired{false};  // its D2H has been issued (or it was discarded): the
                                       // memory may be reused once free_ev has fired
    bool queued = false;   // handed to the write-back thread, which will retire it
    // content, for prefetched chunks
    int pid = -1;
    int64_t eoff = 0, len = 0;
    bool has_grad = false;
    char *g = nullptr, *m = nullptr, *v = nullptr, *x = nullptr;  // sub-buffers
    char* guard = nullptr;  // canary words behind the chunk (EngineOptions::canaries)
  };
  // One chunk's write-back, as handed to the helper thread (everything by value).
  struct WbJob {
    Entry* e = nullptr;
    void* host[3] = {nullptr, nullptr, nullptr};
    const void* dev[3] = {nullptr, nullptr, nullptr};
    size_t bytes[3] = {0, 0, 0};
    int n = 0;
    cudaEvent_t k_done = nullptr, free_ev = nullptr;
    int pid = -1;  // >= 0: last chunk of that tensor, record host_ready_[pid] after it
  };
  // State of one tensor kept in the front part of the staging buffer.
  struct Resident {
    bool on = false, loaded = false;
    int mode = 0;
    int64_t n = 0;
    char *m = nullptr, *v = nullptr, *x = nullptr, *guard = nullptr;
    cudaEvent_t h2d_done = nullptr, k_done = nullptr, free_ev = nullptr;
    Entry wb;  // stands in for a ring chunk in the write-back job
    // lazy write-back: the host addresses of the last step, copied to at the next flush
    bool dirty = false;
    void *hm = nullptr, *hv = nullptr, *hx = nullptr;
  };
  void writeback_resident(int pid, Resident& r);
  void flush_resident();
  void load_resident(const StagedStepArgs& a, Resident& r);
  void* step_resident(const StagedStepArgs& a, Resident& r);
  cudaError_t launch_chunk(const StagedStepArgs& a, const AdamStepArgs& c, int64_t off);
  void arm_guard(char* guard, cudaStream_t stream);
  void verify_guard(const char* guard, int pid);
  void check_canaries();
  static constexpr size_t kGuardBytes = 256;
  int* canary_status_ = nullptr;  // device: {flag, pid}; carved from the end of the workspace
  int64_t chunk_of(const StagedStepArgs& a) const { return a.chunk > 0 ? a.chunk : opt_.chunk_elems; }
  int64_t prefetch_impl(const StagedStepArgs& a, int64_t from_off, int64_t max_chunks,
                        int max_inflight, bool* full);
  void discard_impl();
  void loader_loop();
  void issue_writeback(const WbJob& j, cudaError_t* err);
  void submit_writeback(const WbJob& j);
  void writer_loop();
  void drain_writer();
  Entry* allocate(size_t bytes, bool may_discard);
  Entry* load_chunk(const StagedStepArgs& a, int64_t off, int64_t len, bool may_discard);
  cudaEvent_t take_event();
  void wait_host_copy(const StagedStepArgs& a);
  void check(cudaError_t e, const char* what);

  int device_;
  cudaStream_t compute_, h2d_, d2h_;
  EngineOptions opt_;
  char* ring_ = nullptr;
  size_t ring_bytes_ = 0, head_ = 0;
  std::vector<Resident> res_;
  size_t res_bytes_ = 0;  // taken from the front of the workspace; the ring starts behind it
  std::list<Entry> live_;        // allocation order, oldest first
  std::deque<Entry*> loaded_;    // prefetched, not yet consumed (consumption order)
  std::deque<Entry*> inflight_;  // prefetch copies possibly still running
  size_t loaded_bytes_ = 0;
  std::vector<cudaEvent_t> pool_;
  std::vector<cudaEvent_t> all_events_;
  std::vector<cudaEvent_t> host_ready_;  // per tensor: last D2H of its state finished
  std::vector<char> host_ready_set_;
  std::vector<cudaEvent_t> grad_ready_;  // per tensor: last D2H of its host gradient finished
  std::vector<char> grad_ready_set_;
  cudaEvent_t tmp_ev_ = nullptr;
  cudaEvent_t join_ev_[3] = {nullptr, nullptr, nullptr};
  int64_t bytes_h2d_ = 0, bytes_d2h_ = 0;
  // write-back thread
  std::thread writer_;
  std::mutex wb_mu_;
  std::condition_variable wb_cv_, wb_idle_cv_;
  std::deque<WbJob> wb_q_;
  bool wb_stop_ = false, wb_busy_ = false;
  std::string wb_error_;
  // prefetch thread
  std::thread loader_;
  std::mutex pf_mu_;
  std::condition_variable pf_cv_, pf_idle_cv_;
  std::vector<PrefetchItem> pf_plan_;
  int pf_inflight_ = 1;
  bool pf_has_plan_ = false, pf_running_ = false, pf_exit_ = false;
  std::atomic<bool> pf_stop_{false}, pf_active_{false};
  std::string pf_error_;
  // The helper thread keeps at most kWbGroups * kWbGroup chunks (about 500 stream
  // operations, half of what a stream takes) pending on the D2H stream and sleeps
  // between polls when that many are: it must never sit inside a blocking enqueue call,
  // which would hold up launches of the other threads as well.
  static constexpr int kWbGroup = 8, kWbGroups = 12;
  cudaEvent_t wb_throttle_[kWbGroups] = {};
  bool wb_throttle_used_[kWbGroups] = {};
  int64_t wb_jobs_ = 0;  // jobs issued by the helper thread
  std::vector<int64_t> wb_submitted_;                  // per tensor, by the caller
  std::unique_ptr<std::atomic<int64_t>[]> wb_issued_;  // per tensor, by the helper thread
};

}  // namespace oab
