// Shared device helpers for the sm_100a kernels of offload_adam_b200.
//
// Everything here is bit-level arithmetic on bf16/fp32 patterns plus small
// vector load/store wrappers.  The float math uses the explicit round-to-nearest
// intrinsics (__fadd_rn, __fmul_rn, ...) which the compiler never contracts into
// FMAs, so each kernel reproduces an op-by-op fp32 PyTorch restatement of the
// same formula bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oab {

// ----------------------------------------------------------------------------
// launch accounting: every wrapper that launches one of our kernels bumps this
// counter so the benchmark can report how many of our launches ran in a region.
// ----------------------------------------------------------------------------
extern unsigned long long g_launch_count;
inline void count_launch(unsigned long long n = 1) { g_launch_count += n; }

// ----------------------------------------------------------------------------
// bf16 <-> fp32 bit helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) {
  return __uint_as_float(b16 << 16);
}

// round-to-nearest-even fp32 -> bf16 bit pattern (NaN quieted like torch).
__device__ __forceinline__ uint32_t f32_to_bf16_rne_bits(float f) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0u;  // NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return u >> 16;
}

// Two fp32 -> one word of two bf16 (lo in the low half), round to nearest even, with the
// hardware convert.  Identical to f32_to_bf16_rne_bits for every non-NaN input; a NaN
// comes out as 0x7fff instead of 0x7fc0 (still a NaN).
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_rne(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// 16 random bits decide whether the truncated bf16 moves one step away from
// zero: up iff rand16 < low 16 bits of the fp32 pattern.
__device__ __forceinline__ uint32_t f32_to_bf16_sr_bits(float f, uint32_t rand16) {
  uint32_t u = __float_as_uint(f);
  uint32_t frac = u & 0xffffu;
  uint32_t trunc = u & 0xffff0000u;
  uint32_t r = (rand16 < frac) ? (trunc + 0x10000u) : trunc;
  return r >> 16;
}

// ----------------------------------------------------------------------------
// Philox4x32-10: counter = (ctr_lo, ctr_hi, 0, 0), key = (seed_lo, seed_hi).
// One call yields 128 random bits = eight 16-bit words, i.e. the words of eight
// consecutive elements.  The CPU restatement in ops/oracle.py generates the same stream.
// ----------------------------------------------------------------------------
struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint64_t counter, uint64_t seed) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)M0 * c0;
    uint64_t p1 = (uint64_t)M1 * c2;
    uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  Philox4 out{c0, c1, c2, c3};
  return out;
}

// ----------------------------------------------------------------------------
// 32-byte vector I/O (Blackwell 256-bit global loads/stores): one instruction
// moves 16 bf16 or 8 fp32 values per thread, so a warp touches 1 KiB of
// contiguous memory per request.  The *_stream variants are for data touched
// exactly once (optimizer state, gradients): no L1 allocation, evict-first in L2.
// Addresses must be 32-byte aligned.
// ----------------------------------------------------------------------------
struct V8 {
  uint32_t w[8];
};
__device__ __forceinline__ V8 ld32(const void* p) {
  V8 v;
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),
                 "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
__device__ __forceinline__ V8 ld32_stream(const void* p) {
  V8 v;
  asm volatile(
      "ld.global.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
        "=r"(v.w[6]), "=r"(v.w[7])
      : "l"(p));
  return v;
}
__device__ __forceinline__ void st32(void* p, const V8& v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]),
               "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]),
               "r"(v.w[7])
               : "memory");
}
__device__ __forceinline__ void st32_stream(void* p, const V8& v) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p),
               "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]),
               "r"(v.w[6]), "r"(v.w[7])
               : "memory");
}
// Load from another GPU's memory through a peer mapping (NVLink): a plain,
// non-multicast 256-bit load that does not allocate in L1.
__device__ __forceinline__ V8 ld32_peer(const void* p) {
  V8 v;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),
                 "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p)
               : "memory");
  return v;
}
// j-th 16-bit half of a 16 x bf16 vector
__device__ __forceinline__ uint32_t half_of(const V8& q, int j) {
  return (q.w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
}
__device__ __forceinline__ void set_half(V8& q, int j, uint32_t h) {
  uint32_t& w = q.w[j >> 1];
  w = (j & 1) ? ((w & 0x0000ffffu) | (h << 16)) : ((w & 0xffff0000u) | (h & 0xffffu));
}

// block-wide sum in a fixed tree order (deterministic for a given blockDim).
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* smem /* >= THREADS/32 floats */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = 0.f;
  if (warp == 0) {
    r = (lane < THREADS / 32) ? smem[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  __syncthreads();
  return r;  // valid in warp 0 (all lanes)
}

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = 0.f;
  if (warp == 0) {
    r = (lane < THREADS / 32) ? smem[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  }
  __syncthreads();
  return r;
}


// Upper bound on the grid of kernels that reduce through a scratch area: the area
// holds kMaxPartials floats followed by one 32-bit ticket counter (zero at rest).
constexpr int kMaxPartials = 148 * 8;

// Two-stage sum whose result does not depend on block scheduling: every block
// stores one partial, the block drawing the last ticket adds all partials in
// index order.  Must be reached by all threads of all blocks.
template <int THREADS>
__device__ __forceinline__ void grid_sum_to(float acc, float* red, int* is_last_smem, float* scratch,
                                            float* out, bool accumulate) {
  float bs = block_sum<THREADS>(acc, red);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + kMaxPartials);
  if (threadIdx.x == 0) {
    scratch[blockIdx.x] = bs;
    __threadfence();
    unsigned int t = atomicAdd(ticket, 1u);
    *is_last_smem = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (*is_last_smem) {
    __threadfence();
    float s = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += THREADS) s += __ldcg(scratch + i);
    float total = block_sum<THREADS>(s, red);
    if (threadIdx.x == 0) {
      *out = accumulate ? (*out + total) : total;
      *ticket = 0u;  // ready for the next launch on this stream
    }
  }
}

// Number of SMs on a B200; grids are sized as multiples of this.
constexpr int kNumSMs = 148;

// Status codes written by kernels that can give up on a bounded wait.
enum Status : int {
  kStatusOk = 0,
  kStatusTimeout = 1,
  kStatusBadArg = 2,
};

}  // namespace oab
