#include "pinned_arena.h"

#include <cuda_runtime.h>
#include <errno.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <stdexcept>
#include <thread>

namespace oab {
namespace {

constexpr int kMpolPreferred = 1;
constexpr unsigned kMpolMfMove = 1u << 1;

std::atomic<int> g_fail_mmap{-1}, g_fail_mbind{-1}, g_fail_register{-1}, g_fail_madvise{-1};

// true when the injected failure for this call site fires now
bool fire(std::atomic<int>& c) {
  int v = c.load();
  if (v < 0) return false;
  if (v == 0) { c.store(-1); return true; }
  c.store(v - 1);
  return false;
}

void* real_mmap(size_t bytes) {
  if (fire(g_fail_mmap)) { errno = ENOMEM; return MAP_FAILED; }
  return ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
}
int real_munmap(void* p, size_t bytes) { return ::munmap(p, bytes); }
long real_mbind(void* p, size_t bytes, int node) {
  if (fire(g_fail_mbind)) { errno = EINVAL; return -1; }
  // Soft preference: pages land on `node` while it has room and spill to other
  // nodes otherwise, instead of the hard OOM that MPOL_BIND produces.
  constexpr int kWords = 16;
  unsigned long mask[kWords];
  memset(mask, 0, sizeof(mask));
  if (node < 0 || node >= kWords * (int)(8 * sizeof(unsigned long))) { errno = EINVAL; return -1; }
  mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
  return ::syscall(SYS_mbind, p, bytes, kMpolPreferred, mask,
                   (unsigned long)(kWords * 8 * sizeof(unsigned long) + 1), kMpolMfMove);
}
int real_madvise_huge(void* p, size_t bytes) {
  if (fire(g_fail_madvise)) { errno = EINVAL; return -1; }
  return ::madvise(p, bytes, MADV_HUGEPAGE);
}
int real_host_register(void* p, size_t bytes) {
  if (fire(g_fail_register)) return (int)cudaErrorMemoryAllocation;
  return (int)cudaHostRegister(p, bytes, cudaHostRegisterDefault);
}
int real_host_unregister(void* p) { return (int)cudaHostUnregister(p); }

SysCalls make_defaults() {
  return SysCalls{real_mmap, real_munmap, real_mbind, real_madvise_huge, real_host_register,
                  real_host_unregister};
}
SysCalls g_sys = make_defaults();

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int64_t read_meminfo_field(int node, const char* field) {
  // plain stdio: "Node 1 MemFree:   64457228 kB"
  char path[128];
  snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/meminfo", node);
  FILE* f = fopen(path, "r");
  if (!f) return -1;
  char line[256];
  int64_t out = -1;
  while (fgets(line, sizeof(line), f)) {
    const char* hit = strstr(line, field);
    if (!hit) continue;
    long long kb = 0;
    if (sscanf(hit + strlen(field), " %lld", &kb) == 1) out = (int64_t)kb * 1024;
    break;
  }
  fclose(f);
  return out;
}

}  // namespace

SysCalls& syscalls() { return g_sys; }
void reset_syscalls() {
  g_sys = make_defaults();
  g_fail_mmap = g_fail_mbind = g_fail_register = g_fail_madvise = -1;
}
void inject_failure(const std::string& name, int countdown) {
  if (name == "mmap") g_fail_mmap = countdown;
  else if (name == "mbind") g_fail_mbind = countdown;
  else if (name == "host_register") g_fail_register = countdown;
  else if (name == "madvise") g_fail_madvise = countdown;
  else throw std::invalid_argument("inject_failure: unknown call '" + name + "'");
}

PinnedArena::PinnedArena(const std::vector<size_t>& sizes, const ArenaOptions& opt) : opt_(opt) {
  const size_t page = 4096;
  const size_t align = std::max<size_t>(opt_.alignment, 256);
  sizes_ = sizes;
  ptrs_.assign(sizes.size(), nullptr);

  // ---- plan: first-fit in order; a tensor never straddles two segments ----
  struct Plan { size_t bytes = 0; std::vector<std::pair<size_t, size_t>> items; };  // (index, offset)
  std::vector<Plan> plans;
  for (size_t i = 0; i < sizes.size(); ++i) {
    size_t need = round_up(std::max<size_t>(sizes[i], 1), align);
    if (plans.empty() || (plans.back().bytes + need > opt_.segment_bytes && plans.back().bytes > 0)) {
      plans.emplace_back();
    }
    plans.back().items.emplace_back(i, plans.back().bytes);
    plans.back().bytes += need;
  }

  int nthreads = opt_.touch_threads > 0
                     ? opt_.touch_threads
                     : (int)std::min<unsigned>(16u, std::max(1u, std::thread::hardware_concurrency()));

  try {
    for (auto& pl : plans) {
      Segment seg;
      seg.bytes = round_up(pl.bytes, size_t(2) << 20);  // whole 2 MiB pages for THP
      double t0 = now_s();
      void* base = g_sys.mmap_fn(seg.bytes);
      if (base == MAP_FAILED || base == nullptr) {
        int e = errno;
        throw std::runtime_error("PinnedArena: mmap(" + std::to_string(seg.bytes) +
                                 ") failed: " + strerror(e));
      }
      seg.base = base;
      segs_.push_back(seg);
      if (opt_.numa_node >= 0) {
        if (g_sys.mbind_fn(base, seg.bytes, opt_.numa_node) != 0) {
          int e = errno;
          throw std::runtime_error("PinnedArena: mbind(node=" + std::to_string(opt_.numa_node) +
                                   ") failed: " + strerror(e));
        }
        numa_bound_ = true;
      }
      if (opt_.huge_pages) (void)g_sys.madvise_huge_fn(base, seg.bytes);  // best effort
      t_map_ += now_s() - t0;

      // ---- first touch in parallel: commits pages under the bound policy ----
      t0 = now_s();
      {
        size_t per = round_up((seg.bytes + nthreads - 1) / nthreads, size_t(2) << 20);
        std::vector<std::thread> th;
        for (int t = 0; t < nthreads; ++t) {
          size_t lo = (size_t)t * per;
          if (lo >= seg.bytes) break;
          size_t hi = std::min(seg.bytes, lo + per);
          th.emplace_back([base, lo, hi]() { memset((char*)base + lo, 0, hi - lo); });
        }
        for (auto& x : th) x.join();
      }
      t_touch_ += now_s() - t0;

      if (opt_.register_cuda) {
        t0 = now_s();
        int err = g_sys.host_register_fn(base, seg.bytes);
        if (err != 0) {
          throw std::runtime_error(std::string("PinnedArena: cudaHostRegister(") +
                                   std::to_string(seg.bytes) + ") failed: " +
                                   cudaGetErrorString((cudaError_t)err));
        }
        segs_.back().registered = true;
        registered_ = true;
        t_register_ += now_s() - t0;
      }
      for (auto& it : pl.items) ptrs_[it.first] = (char*)base + it.second;
      total_bytes_ += seg.bytes;
      (void)page;
    }
  } catch (...) {
    release_all();
    throw;
  }
}

void PinnedArena::release_all() {
  for (auto& s : segs_) {
    if (s.registered) (void)g_sys.host_unregister_fn(s.base);
    if (s.base) (void)g_sys.munmap_fn(s.base, s.bytes);
  }
  segs_.clear();
}

PinnedArena::~PinnedArena() { release_all(); }

std::string pci_bus_id(int device) {
  char buf[32] = {0};
  if (cudaDeviceGetPCIBusId(buf, sizeof(buf), device) != cudaSuccess) {
    (void)cudaGetLastError();
    return "";
  }
  std::string s(buf);
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  return s;
}

int gpu_numa_node(int device) {
  std::string pci = pci_bus_id(device);
  if (pci.empty()) return -1;
  std::string path = "/sys/bus/pci/devices/" + pci + "/numa_node";
  FILE* f = fopen(path.c_str(), "r");
  if (!f) return -1;
  int node = -1;
  if (fscanf(f, "%d", &node) != 1) node = -1;
  fclose(f);
  return node;
}

int64_t numa_node_free_bytes(int node) { return read_meminfo_field(node, "MemFree:"); }
int64_t numa_node_total_bytes(int node) { return read_meminfo_field(node, "MemTotal:"); }

int numa_num_nodes() {
  int n = 0;
  for (int i = 0; i < 1024; ++i) {
    char path[96];
    snprintf(path, sizeof(path), "/sys/devices/system/node/node%d", i);
    if (access(path, F_OK) == 0) ++n; else if (i > 64) break;
  }
  return n;
}

}  // namespace oab
