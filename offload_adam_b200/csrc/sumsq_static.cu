// Allocation-free squared-norm entry point (see sumsq_static.h).
//
// A variant of the two-stage reduction in grad_ops.cu: there the caller hands in a
// scratch tensor; here the scratch is a file-scope device array, one slot per block
// of 8192 elements, which is what bounds the input size.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "common.cuh"
#include "sumsq_static.h"

namespace {

constexpr int kThreads = 256;
constexpr int kTile = 8192;  // elements per block: 256 threads x 2 vectors of 16
constexpr int kMaxBlocks = 65536;
constexpr int kMaxDevices = 64;
static_assert((long long)kMaxBlocks * kTile == OAB_SUMSQ_STATIC_MAX_ELEMS, "limit mismatch");

// kMaxBlocks partial sums followed by the ticket counter (kept in its own 256-byte
// line).  In host code this name is only a handle for cudaGetSymbolAddress; it is not
// a device address.
static __device__ __align__(256) float g_static_scratch[kMaxBlocks + 64];

// device address of g_static_scratch per device ordinal, filled on first use
float* g_scratch_addr[kMaxDevices] = {};

__device__ __forceinline__ float sq2(uint32_t w, float acc) {
  const float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
  acc = __fadd_rn(acc, __fmul_rn(lo, lo));
  return __fadd_rn(acc, __fmul_rn(hi, hi));
}

__global__ void __launch_bounds__(kThreads)
sumsq_static_kernel(const uint16_t* __restrict__ x, long long n, float* out, float* scratch,
                    int vector_ok) {
  __shared__ float red[kThreads / 32];
  __shared__ int is_last;
  const long long begin = (long long)blockIdx.x * kTile;
  long long end = begin + kTile;
  if (end > n) end = n;
  float acc = 0.f;
  long long scalar_from = begin;
  if (vector_ok) {
    const long long nvec = (end - begin) >> 4;
    scalar_from = begin + (nvec << 4);
    for (long long v = threadIdx.x; v < nvec; v += kThreads) {
      const oab::V8 r = oab::ld32_stream(x + begin + v * 16);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = sq2(r.w[j], acc);
    }
  }
  for (long long i = scalar_from + threadIdx.x; i < end; i += kThreads) {
    const float f = oab::bf16_bits_to_f32(x[i]);
    acc = __fadd_rn(acc, __fmul_rn(f, f));
  }
  const float bs = oab::block_sum<kThreads>(acc, red);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + kMaxBlocks);
  if (threadIdx.x == 0) {
    scratch[blockIdx.x] = bs;
    __threadfence();
    is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    // the block that finishes last adds the partials in index order
    __threadfence();
    float s = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += kThreads) s += __ldcg(scratch + i);
    const float total = oab::block_sum<kThreads>(s, red);
    if (threadIdx.x == 0) *out = total;
  }
}

int fail(int code, char* err, int err_len, const char* what, cudaError_t e) {
  if (err != nullptr && err_len > 0) {
    if (e != cudaSuccess) snprintf(err, (size_t)err_len, "oab_sumsq_bf16_static: %s: %s", what, cudaGetErrorString(e));
    else snprintf(err, (size_t)err_len, "oab_sumsq_bf16_static: %s", what);
  }
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int oab_sumsq_bf16_static(const void* x, long long n, float* out, void* stream, char* err,
                          int err_len) {
  if (out == nullptr || n < 0 || (x == nullptr && n > 0))
    return fail(OAB_STATIC_BAD_ARGUMENT, err, err_len, "null pointer or negative length", cudaSuccess);
  if (n > OAB_SUMSQ_STATIC_MAX_ELEMS) {
    char msg[160];
    snprintf(msg, sizeof(msg), "n = %lld exceeds the built-in scratch limit of %lld elements; "
             "split the buffer or use the scratch-tensor entry point", n, (long long)OAB_SUMSQ_STATIC_MAX_ELEMS);
    return fail(OAB_STATIC_TOO_LARGE, err, err_len, msg, cudaSuccess);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(OAB_STATIC_CUDA_ERROR, err, err_len, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices)
    return fail(OAB_STATIC_BAD_ARGUMENT, err, err_len, "device ordinal out of range", cudaSuccess);
  if (g_scratch_addr[dev] == nullptr) {
    // once per device, with that device current: translate the symbol into the address
    // the kernel can use
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(OAB_STATIC_CUDA_ERROR, err, err_len, "cudaGetSymbolAddress(scratch)", e);
    g_scratch_addr[dev] = p;
  }
  float* scratch = g_scratch_addr[dev];
  if (n == 0) {
    e = cudaMemsetAsync(out, 0, sizeof(float), st);
    return e == cudaSuccess ? OAB_STATIC_OK : fail(OAB_STATIC_CUDA_ERROR, err, err_len, "cudaMemsetAsync(out)", e);
  }
  // the ticket counter must start at zero whatever the previous call left behind
  e = cudaMemsetAsync(scratch + kMaxBlocks, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) return fail(OAB_STATIC_CUDA_ERROR, err, err_len, "cudaMemsetAsync(ticket)", e);
  const int blocks = (int)((n + kTile - 1) / kTile);
  const int vector_ok = (reinterpret_cast<uintptr_t>(x) & 31u) == 0;
  oab::count_launch();
  sumsq_static_kernel<<<blocks, kThreads, 0, st>>>(static_cast<const uint16_t*>(x), n, out, scratch, vector_ok);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(OAB_STATIC_CUDA_ERROR, err, err_len, "kernel launch", e);
  return OAB_STATIC_OK;
}
