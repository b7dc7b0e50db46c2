// Shared declarations of the CUDA side: error reporting, device status words,
// small device helpers.  sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

namespace clt {

// ---- host-side error string (one per thread) ---------------------------------
void set_error(const char* fmt, ...);
const char* last_error();

#define CLT_CHECK_ARG(cond, ...)                 \
  do {                                           \
    if (!(cond)) {                               \
      ::clt::set_error(__VA_ARGS__);             \
      return 1;                                  \
    }                                            \
  } while (0)

#define CLT_CHECK_CUDA(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      ::clt::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),      \
                       __FILE__, __LINE__);                                         \
      return 2;                                                                     \
    }                                                                               \
  } while (0)

// ---- device status word --------------------------------------------------------
// Kernels never trap.  A kernel that gives up on a wait or meets an index out of
// range writes one of these codes (first writer wins) and returns; the host
// reads the word at its next synchronisation point.
enum DeviceStatus : int {
  kOk = 0,
  kTimeoutFull = 0x10,       // MMA warp gave up waiting for a TMA stage
  kTimeoutEmpty = 0x11,      // TMA warp gave up waiting for a free stage
  kTimeoutTmemFull = 0x12,   // epilogue gave up waiting for the accumulator
  kTimeoutTmemEmpty = 0x13,  // MMA warp gave up waiting for the epilogue
  kBadIndex = 0x20,          // an index read from memory was out of range
  kOverflow = 0x21,          // a fixed-capacity list overflowed
};

__device__ __forceinline__ void report_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ---- small device helpers -----------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <class T>
struct ToFloat;
template <>
struct ToFloat<float> {
  __device__ static __forceinline__ float get(float v) { return v; }
};
template <>
struct ToFloat<__nv_bfloat16> {
  __device__ static __forceinline__ float get(__nv_bfloat16 v) { return __bfloat162float(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Column sums over the 32 rows held by one warp.  Each lane holds 32 values
// (one row, 32 consecutive columns); on return lane j holds the sum over all
// lanes of column j.  Recursive halving: 31 shuffles for 32 columns.
__device__ __forceinline__ float warp_colsum32(float (&v)[32]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      float send = upper ? v[i] : v[i + off];
      float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

}  // namespace clt
