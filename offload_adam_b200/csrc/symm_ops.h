// Host-side launch interface of the symmetric-memory (NVLink peer access) kernels
// that replace the ZeRO-1 collectives (symm_ops.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "adam_step.h"

namespace oab {

// Status codes a bounded wait leaves in the status word (first failure wins).
enum SymmStatus : int {
  kSymmOk = 0,
  kSymmTimeoutGrad = 1,    // a peer never announced its gradient
  kSymmTimeoutParam = 2,   // a peer never announced its updated parameter rows
  kSymmTimeoutScalar = 3,  // a peer never delivered its scalar for the norm exchange
};

// out[i] = bf16(scale * sum_j peers[j][i]) (fp32 sum in index order) and, when
// sumsq_out != nullptr, sumsq_out = sum_i float(out[i])^2 (deterministic order).
// `peers` are pointers into the ranks' replicas (own one included) mapped into this
// device.  Returns without touching memory when *abort_flag != 0.
struct PeerReduceArgs {
  void* out = nullptr;
  // optional: out = bf16(acc_in + bf16(scale * sum)) (acc_in may alias out): one micro-batch's
  // mean added to an accumulator, rounded like reduce-scatter(AVG) + in-place bf16 add
  const void* acc_in = nullptr;
  const void* peers[kMaxPeers] = {};
  int n_peers = 0;
  int64_t n = 0;
  float scale = 1.f;
  float* sumsq_out = nullptr;
  float* scratch = nullptr;
  const int* abort_flag = nullptr;
  int max_ctas = 0;
};
cudaError_t launch_peer_reduce(const PeerReduceArgs& a, cudaStream_t stream);

// Waits until flags[i] >= epoch (wrap-safe) for i in [0, n), giving up after
// timeout_ns: then status (device-visible int) receives `code` unless already set.
// A launch with *status != 0 returns at once.
cudaError_t launch_wait_flags(const uint32_t* flags, int n, uint32_t epoch, uint64_t timeout_ns,
                              int* status, int code, cudaStream_t stream);

// Makes every earlier write of this stream visible system-wide, then stores `value`
// to each of the n addresses (flag words in the peers' memory).
cudaError_t launch_signal(uint32_t* const* ptrs_host, int n, uint32_t value, cudaStream_t stream);

// As launch_signal for many flags at once: word first + i * stride (i < count) of the flag
// array at bases_host[j] on every one of the n_peers ranks receives `value`.
cudaError_t launch_signal_many(uint32_t* const* bases_host, int n_peers, int first, int stride, int count,
                               uint32_t value, cudaStream_t stream);

// dst[i] = src[i] for i < n <= 32, done by a kernel so that a status word can be
// mirrored into mapped host memory without queueing behind bulk DMA copies.
cudaError_t launch_mirror_words(const int* src, int* dst, int n, cudaStream_t stream);

// Single-kernel all-reduce of one fp32 scalar across ranks (SUM in rank order, or MAX of
// non-negative values): stores *my_value into slot[rank] of every peer, raises
// flag[rank] there, waits (bounded) for all local flags and writes the result to *out.
// Consecutive exchanges must alternate between two sets of slots and flags and use
// increasing epochs: a rank can be one exchange ahead of the slowest one, never two.
struct ScalarExchangeArgs {
  const float* my_value = nullptr;
  float* peer_slots[kMaxPeers] = {};     // base of each rank's slot array (n floats)
  uint32_t* peer_flags[kMaxPeers] = {};  // base of each rank's flag array (n words)
  const float* local_slots = nullptr;
  const uint32_t* local_flags = nullptr;
  int n = 0;
  int rank = 0;
  uint32_t epoch = 0;
  uint64_t timeout_ns = 0;
  int* status = nullptr;
  float* out = nullptr;
  bool op_max = false;
};
cudaError_t launch_scalar_exchange(const ScalarExchangeArgs& a, cudaStream_t stream);

}  // namespace oab
