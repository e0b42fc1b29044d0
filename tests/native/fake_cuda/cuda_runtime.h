// A stand-in for the CUDA runtime that runs on the CPU, for testing the host-side
// logic of the copy engine (ring allocation, helper threads, event ordering) without a
// GPU.  Streams are worker threads that execute their operations in order with random
// delays; events follow CUDA's rules (a wait captures the record that is current when
// it is enqueued; a query reports on the most recent record); enqueueing blocks while a
// stream holds `fake_cuda::queue_capacity` pending operations, like a real stream whose
// queue is full.  "Device" memory is ordinary host memory.
#pragma once
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <random>
#include <thread>

typedef int cudaError_t;
enum { cudaSuccess = 0, cudaErrorInvalidValue = 1, cudaErrorNotReady = 600 };
enum cudaMemcpyKind { cudaMemcpyHostToHost = 0, cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2,
                      cudaMemcpyDeviceToDevice = 3 };
#define cudaEventDisableTiming 2
struct int2 {
  int x, y;
};

namespace fake_cuda {
inline std::atomic<size_t> queue_capacity{64};
inline std::atomic<int> max_delay_us{60};
inline std::atomic<long> ops_executed{0};

struct Event {
  std::mutex mu;
  std::condition_variable cv;
  uint64_t recorded = 0, completed = 0;
};

struct Stream {
  std::mutex mu;
  std::condition_variable cv_work, cv_space, cv_idle;
  std::deque<std::function<void()>> q;
  bool stop = false, busy = false;
  int extra_delay_us = 0;  // makes this stream slow relative to the others
  std::thread worker;
  std::mt19937 rng;
  explicit Stream(unsigned seed) : rng(seed) {
    worker = std::thread([this] { run(); });
  }
  ~Stream() {
    {
      std::lock_guard<std::mutex> lk(mu);
      stop = true;
    }
    cv_work.notify_all();
    worker.join();
  }
  void run() {
    for (;;) {
      std::function<void()> op;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_work.wait(lk, [&] { return stop || !q.empty(); });
        if (q.empty()) return;
        op = std::move(q.front());
        q.pop_front();
        busy = true;
      }
      cv_space.notify_all();
      const int d = max_delay_us.load();
      if (d > 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % (unsigned)(d + 1)));
      if (extra_delay_us > 0) std::this_thread::sleep_for(std::chrono::microseconds(extra_delay_us));
      op();
      ops_executed.fetch_add(1);
      {
        std::lock_guard<std::mutex> lk(mu);
        busy = false;
        if (q.empty()) cv_idle.notify_all();
      }
    }
  }
  void push(std::function<void()> op) {
    std::unique_lock<std::mutex> lk(mu);
    cv_space.wait(lk, [&] { return q.size() < queue_capacity.load(); });  // a full queue blocks the caller
    q.push_back(std::move(op));
    cv_work.notify_all();
  }
  void drain() {
    std::unique_lock<std::mutex> lk(mu);
    cv_idle.wait(lk, [&] { return q.empty() && !busy; });
  }
};
}  // namespace fake_cuda

typedef fake_cuda::Event* cudaEvent_t;
typedef fake_cuda::Stream* cudaStream_t;

inline cudaError_t cudaSetDevice(int) { return cudaSuccess; }
inline cudaError_t cudaGetLastError() { return cudaSuccess; }
inline const char* cudaGetErrorString(cudaError_t e) { return e == cudaSuccess ? "no error" : "fake CUDA error"; }

inline cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned) {
  *e = new fake_cuda::Event();
  return cudaSuccess;
}
inline cudaError_t cudaEventDestroy(cudaEvent_t e) {
  delete e;
  return cudaSuccess;
}
inline cudaError_t cudaEventRecord(cudaEvent_t e, cudaStream_t s) {
  uint64_t seq;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    seq = ++e->recorded;
  }
  s->push([e, seq] {
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->completed < seq) e->completed = seq;
    e->cv.notify_all();
  });
  return cudaSuccess;
}
inline cudaError_t cudaStreamWaitEvent(cudaStream_t s, cudaEvent_t e, unsigned) {
  uint64_t target;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    target = e->recorded;  // the record that is current now; 0: never recorded, no wait
  }
  if (target == 0) return cudaSuccess;
  s->push([e, target] {
    std::unique_lock<std::mutex> lk(e->mu);
    e->cv.wait(lk, [&] { return e->completed >= target; });
  });
  return cudaSuccess;
}
inline cudaError_t cudaEventQuery(cudaEvent_t e) {
  std::lock_guard<std::mutex> lk(e->mu);
  return e->completed >= e->recorded ? cudaSuccess : cudaErrorNotReady;
}
inline cudaError_t cudaEventSynchronize(cudaEvent_t e) {
  std::unique_lock<std::mutex> lk(e->mu);
  const uint64_t target = e->recorded;
  e->cv.wait(lk, [&] { return e->completed >= target; });
  return cudaSuccess;
}
inline cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t n, cudaMemcpyKind, cudaStream_t s) {
  s->push([dst, src, n] { memcpy(dst, src, n); });
  return cudaSuccess;
}
inline cudaError_t cudaMemsetAsync(void* dst, int value, size_t n, cudaStream_t s) {
  s->push([=] { memset(dst, value, n); });
  return cudaSuccess;
}
inline cudaError_t cudaStreamSynchronize(cudaStream_t s) {
  s->drain();
  return cudaSuccess;
}
