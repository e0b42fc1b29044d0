// ZeRO-1 collectives as peer-memory kernels (sm_100a, NVLink 5 through NVSwitch).
//
// The reference issues, per parameter, reduce_scatter_tensor(AVG) / all_reduce(AVG),
// torch.norm, the step kernel and all_gather_into_tensor as separate blocking NCCL
// and Triton launches on the main stream
// (reference: src/offload_adam/distributed_offload_adam.py:61-104, :182-306).
// Here every rank's gradient accumulators and parameters live in symmetric memory
// that each GPU maps; a rank pulls the rows it owns from all replicas with plain
// peer loads, reduces them in fp32 in rank order (bit-identical on every rank) and,
// in the same pass, either feeds Adam and pushes the new bf16 rows into all replicas
// (adam_step.cu, PEERS variant) or stores the reduced slice and its squared norm
// (this file).  Ordering between ranks uses epoch flags written with system-scope
// release stores into the consumers' own memory, so waits spin on local memory.
//
// Every wait is bounded by the global timer: on expiry the kernel records a status
// code and returns; later kernels see the status and do nothing.  No wait can hang a
// GPU, and nothing here traps.
#include "common.cuh"
#include "symm_ops.h"

namespace oab {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool reached(uint32_t v, uint32_t epoch) { return (int32_t)(v - epoch) >= 0; }

// Bounded wait on one flag.  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t t0,
                                          uint64_t timeout_ns) {
  // the iteration cap is a second bound in case the timer misbehaves
  for (uint64_t it = 0; it < (1ull << 34); ++it) {
    if (reached(ld_acquire_sys(flag), epoch)) return true;
    if (global_timer_ns() - t0 > timeout_ns) return false;
    __nanosleep(200);
  }
  return false;
}

struct PeerPtrs {
  const uint16_t* g[kMaxPeers];
  int n;
};

// out = bf16(scale * sum_j peers[j]) or, with `acc`, bf16(acc + that bf16 value): the
// second form accumulates the mean of one micro-batch into a shard-sized accumulator
// with the roundings of a reduce-scatter(AVG) followed by an in-place bf16 add.
template <bool SUMSQ, bool ACC>
__global__ void __launch_bounds__(kThreads)
peer_reduce_kernel(uint16_t* out, const uint16_t* acc_in, PeerPtrs pp, int64_t n, float scale, float* sumsq_out,
                   float* scratch, int vector_ok, const int* abort_flag) {
  __shared__ float red[kThreads / 32];
  __shared__ int is_last;
  if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return;
  float acc = 0.f;
  const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * kThreads;
  int64_t scalar_begin = 0;
  if (vector_ok) {
    const int64_t nvec = n >> 4;
    scalar_begin = nvec << 4;
    for (int64_t vec = tid; vec < nvec; vec += nthreads) {
      V8 in[kMaxPeers];
#pragma unroll
      for (int j = 0; j < kMaxPeers; ++j)
        if (j < pp.n) in[j] = ld32_peer(pp.g[j] + vec * 16);
      V8 prev;
      if (ACC) prev = ld32_stream(acc_in + vec * 16);
      V8 r;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxPeers; ++j)
          if (j < pp.n) {
            lo = __fadd_rn(lo, __uint_as_float(in[j].w[w] << 16));
            hi = __fadd_rn(hi, __uint_as_float(in[j].w[w] & 0xffff0000u));
          }
        uint32_t blo = f32_to_bf16_rne_bits(__fmul_rn(lo, scale));
        uint32_t bhi = f32_to_bf16_rne_bits(__fmul_rn(hi, scale));
        if (ACC) {
          blo = f32_to_bf16_rne_bits(__fadd_rn(__uint_as_float(prev.w[w] << 16), __uint_as_float(blo << 16)));
          bhi = f32_to_bf16_rne_bits(__fadd_rn(__uint_as_float(prev.w[w] & 0xffff0000u), __uint_as_float(bhi << 16)));
        }
        r.w[w] = blo | (bhi << 16);
        if (SUMSQ) {
          const float flo = __uint_as_float(blo << 16), fhi = __uint_as_float(bhi << 16);
          acc = __fadd_rn(acc, __fmul_rn(flo, flo));
          acc = __fadd_rn(acc, __fmul_rn(fhi, fhi));
        }
      }
      st32(out + vec * 16, r);
    }
  }
  for (int64_t i = scalar_begin + tid; i < n; i += nthreads) {
    float s = 0.f;
    for (int j = 0; j < pp.n; ++j) s = __fadd_rn(s, bf16_bits_to_f32(pp.g[j][i]));
    uint32_t b = f32_to_bf16_rne_bits(__fmul_rn(s, scale));
    if (ACC) b = f32_to_bf16_rne_bits(__fadd_rn(bf16_bits_to_f32(acc_in[i]), bf16_bits_to_f32(b)));
    out[i] = (uint16_t)b;
    if (SUMSQ) { const float f = bf16_bits_to_f32(b); acc = __fadd_rn(acc, __fmul_rn(f, f)); }
  }
  if (SUMSQ) grid_sum_to<kThreads>(acc, red, &is_last, scratch, sumsq_out, false);
}

__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t epoch, uint64_t timeout_ns,
                                  int* status, int code) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  const uint64_t t0 = global_timer_ns();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (!wait_flag(flags + i, epoch, t0, timeout_ns)) {
      atomicCAS(status, 0, code);
      __threadfence_system();
      return;
    }
  }
}

struct SignalPtrs {
  uint32_t* p[kMaxPeers];
};
__global__ void signal_kernel(SignalPtrs sp, int n, uint32_t value) {
  // all prior work of this stream has completed (kernel boundary); the fence orders
  // it before the flag for observers on other GPUs
  __threadfence_system();
  if ((int)threadIdx.x < n) st_release_sys(sp.p[threadIdx.x], value);
}

// the same for `count` flag words at base + first + i * stride in every peer's flag array
__global__ void signal_many_kernel(SignalPtrs bases, int n_peers, int first, int stride, int count, uint32_t value) {
  __threadfence_system();
  for (int i = threadIdx.x; i < count; i += blockDim.x)
    for (int j = 0; j < n_peers; ++j) st_release_sys(bases.p[j] + first + (int64_t)i * stride, value);
}

__global__ void mirror_words_kernel(const int* src, int* dst, int n) {
  // plain stores (to mapped host memory): keeps the DMA engines out of it
  if ((int)threadIdx.x < n) dst[threadIdx.x] = src[threadIdx.x];
}

struct ExchangePtrs {
  float* slots[kMaxPeers];
  uint32_t* flags[kMaxPeers];
};
__global__ void scalar_exchange_kernel(const float* my_value, ExchangePtrs ep, const float* local_slots,
                                       const uint32_t* local_flags, int n, int rank, uint32_t epoch,
                                       uint64_t timeout_ns, int* status, float* out, int op_max) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  const int j = threadIdx.x;
  const uint64_t t0 = global_timer_ns();
  if (j < n) {
    const float v = *my_value;
    *reinterpret_cast<volatile float*>(ep.slots[j] + rank) = v;
    __threadfence_system();
    st_release_sys(ep.flags[j] + rank, epoch);
  }
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (j < n && !wait_flag(local_flags + j, epoch, t0, timeout_ns)) failed = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (failed) {
      atomicCAS(status, 0, (int)kSymmTimeoutScalar);
      __threadfence_system();
      return;
    }
    float s = 0.f;
    for (int k = 0; k < n; ++k) {
      const float x = *reinterpret_cast<const volatile float*>(local_slots + k);
      s = op_max ? fmaxf(s, x) : __fadd_rn(s, x);
    }
    *out = s;
  }
}

}  // namespace

cudaError_t launch_peer_reduce(const PeerReduceArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  if (a.n_peers < 1 || a.n_peers > kMaxPeers || a.out == nullptr) return cudaErrorInvalidValue;
  if (a.sumsq_out && !a.scratch) return cudaErrorInvalidValue;
  PeerPtrs pp;
  pp.n = a.n_peers;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  int vector_ok = al(a.out);
  for (int j = 0; j < kMaxPeers; ++j) {
    pp.g[j] = (const uint16_t*)a.peers[j < a.n_peers ? j : 0];
    if (j < a.n_peers) vector_ok = vector_ok && al(a.peers[j]);
  }
  const int64_t nvec = (a.n + 15) / 16;
  int64_t want = (nvec + kThreads - 1) / kThreads;
  int cap = a.max_ctas > 0 ? (a.max_ctas < kMaxPartials ? a.max_ctas : kMaxPartials) : kMaxPartials;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  count_launch();
  const uint16_t* acc = (const uint16_t*)a.acc_in;
  if (acc != nullptr) vector_ok = vector_ok && al(acc);
#define OAB_PR(SQ, AC)                                                                              \
  peer_reduce_kernel<SQ, AC><<<grid, kThreads, 0, stream>>>((uint16_t*)a.out, acc, pp, a.n, a.scale,    \
                                                            (SQ) ? a.sumsq_out : nullptr,               \
                                                            (SQ) ? a.scratch : nullptr, vector_ok, a.abort_flag)
  if (a.sumsq_out) { if (acc) OAB_PR(true, true); else OAB_PR(true, false); }
  else { if (acc) OAB_PR(false, true); else OAB_PR(false, false); }
#undef OAB_PR
  return cudaGetLastError();
}

cudaError_t launch_wait_flags(const uint32_t* flags, int n, uint32_t epoch, uint64_t timeout_ns,
                              int* status, int code, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (status == nullptr) return cudaErrorInvalidValue;
  count_launch();
  int threads = n < 32 ? 32 : (n > 256 ? 256 : (n + 31) / 32 * 32);
  wait_flags_kernel<<<1, threads, 0, stream>>>(flags, n, epoch, timeout_ns, status, code);
  return cudaGetLastError();
}

cudaError_t launch_signal(uint32_t* const* ptrs_host, int n, uint32_t value, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (n > kMaxPeers) return cudaErrorInvalidValue;
  SignalPtrs sp;
  for (int j = 0; j < kMaxPeers; ++j) sp.p[j] = ptrs_host[j < n ? j : 0];
  count_launch();
  signal_kernel<<<1, 32, 0, stream>>>(sp, n, value);
  return cudaGetLastError();
}

cudaError_t launch_signal_many(uint32_t* const* bases_host, int n_peers, int first, int stride, int count,
                               uint32_t value, cudaStream_t stream) {
  if (count <= 0 || n_peers <= 0) return cudaSuccess;
  if (n_peers > kMaxPeers) return cudaErrorInvalidValue;
  SignalPtrs sp;
  for (int j = 0; j < kMaxPeers; ++j) sp.p[j] = bases_host[j < n_peers ? j : 0];
  count_launch();
  signal_many_kernel<<<1, 256, 0, stream>>>(sp, n_peers, first, stride, count, value);
  return cudaGetLastError();
}

cudaError_t launch_mirror_words(const int* src, int* dst, int n, cudaStream_t stream) {
  if (n <= 0 || n > 32) return cudaErrorInvalidValue;
  count_launch();
  mirror_words_kernel<<<1, 32, 0, stream>>>(src, dst, n);
  return cudaGetLastError();
}

cudaError_t launch_scalar_exchange(const ScalarExchangeArgs& a, cudaStream_t stream) {
  if (a.n < 1 || a.n > kMaxPeers || a.status == nullptr) return cudaErrorInvalidValue;
  ExchangePtrs ep;
  for (int j = 0; j < kMaxPeers; ++j) {
    ep.slots[j] = a.peer_slots[j < a.n ? j : 0];
    ep.flags[j] = a.peer_flags[j < a.n ? j : 0];
  }
  count_launch();
  scalar_exchange_kernel<<<1, 32, 0, stream>>>(a.my_value, ep, a.local_slots, a.local_flags, a.n, a.rank,
                                               a.epoch, a.timeout_ns, a.status, a.out, a.op_max ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace oab
