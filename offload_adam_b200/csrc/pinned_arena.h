// Pinned host arena: few large NUMA-bound, CUDA-registered regions from which
// every optimizer-state tensor is carved.
//
// The reference allocates one mmap + mbind + memset + cudaHostRegister per
// (parameter, state) pair through ctypes and libnuma
// (reference: src/offload_adam/pinned_alloc.py:177-277), i.e. ~900 registrations
// and a single-threaded first touch of tens of GB for an 8B model.  Here one
// arena packs all tensors into a handful of segments; each segment is mapped
// once, bound with the raw mbind(2) syscall (no libnuma needed), touched by a
// thread pool and registered with one cudaHostRegister call.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace oab {

// Injectable system interface so allocator failures can be exercised on a
// machine without faulting anything: tests swap individual entries for fakes.
struct SysCalls {
  void* (*mmap_fn)(size_t bytes);
  int (*munmap_fn)(void* p, size_t bytes);
  long (*mbind_fn)(void* p, size_t bytes, int node);
  int (*madvise_huge_fn)(void* p, size_t bytes);
  int (*host_register_fn)(void* p, size_t bytes);  // returns cudaError_t
  int (*host_unregister_fn)(void* p);
};
SysCalls& syscalls();          // process-wide table (defaults to the real calls)
void reset_syscalls();         // restore the defaults
// name in {"mmap","mbind","host_register","madvise"}; countdown = number of
// successful calls before the failure fires (0 = next call), -1 disables.
void inject_failure(const std::string& name, int countdown);

struct ArenaOptions {
  int numa_node = -1;          // -1: no binding
  bool register_cuda = true;   // cudaHostRegister each segment
  bool huge_pages = true;      // madvise(MADV_HUGEPAGE) before first touch
  int touch_threads = 0;       // 0: min(16, hardware_concurrency)
  size_t segment_bytes = size_t(4) << 30;
  size_t alignment = 4096;     // per-tensor alignment inside a segment
};

class PinnedArena : public std::enable_shared_from_this<PinnedArena> {
 public:
  // Plans segments for `sizes` (bytes per tensor), maps/binds/touches/registers
  // them.  Throws std::runtime_error with the failing call and errno/cuda code;
  // everything mapped so far is released first.
  PinnedArena(const std::vector<size_t>& sizes, const ArenaOptions& opt);
  ~PinnedArena();
  PinnedArena(const PinnedArena&) = delete;
  PinnedArena& operator=(const PinnedArena&) = delete;

  size_t num_tensors() const { return ptrs_.size(); }
  void* ptr(size_t i) const { return ptrs_[i]; }
  size_t size(size_t i) const { return sizes_[i]; }
  size_t total_bytes() const { return total_bytes_; }
  size_t num_segments() const { return segs_.size(); }
  bool registered() const { return registered_; }
  int numa_node() const { return opt_.numa_node; }
  bool numa_bound() const { return numa_bound_; }
  double seconds_map() const { return t_map_; }
  double seconds_touch() const { return t_touch_; }
  double seconds_register() const { return t_register_; }

 private:
  struct Segment {
    void* base = nullptr;
    size_t bytes = 0;
    bool registered = false;
  };
  void release_all();
  ArenaOptions opt_;
  std::vector<Segment> segs_;
  std::vector<void*> ptrs_;
  std::vector<size_t> sizes_;
  size_t total_bytes_ = 0;
  bool registered_ = false;
  bool numa_bound_ = false;
  double t_map_ = 0, t_touch_ = 0, t_register_ = 0;
};

// NUMA helpers (reference: pinned_alloc.py:113-174).
int gpu_numa_node(int device);                 // -1 when unknown / no CUDA
int64_t numa_node_free_bytes(int node);        // -1 on failure
int64_t numa_node_total_bytes(int node);       // -1 on failure
int numa_num_nodes();                          // count of /sys/devices/system/node/node*
std::string pci_bus_id(int device);            // "" when unavailable

}  // namespace oab
