// Batch ingestion from the reference's activation store (crosslayer_transcoder/data/shared_memory.py:168-214:
// `get_activations` gathers `batch_size` random valid rows of the `[buffer_size, 2, L, D]` host buffer with
// one CPU thread and returns a pageable copy, which the trainer then uploads).  Here the store's host
// mapping is registered with the CUDA driver once and the GPU gathers the chosen rows itself over PCIe,
// straight into the device batch the step reads: no CPU copy of the 147 MB (C3) batch at all.
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {
namespace {

constexpr int kGatherThreads = 256;
constexpr int kGatherUnroll = 4;     // 16-byte loads in flight per thread: PCIe reads need depth, not width

// dst[i, :] = src[rows[i], :] for rows of `row_vec` 16-byte vectors.  `src` may be host memory mapped into
// the device's address space.  A CTA copies one row chunk of kGatherThreads * kGatherUnroll vectors at a time.
__global__ void __launch_bounds__(kGatherThreads) gather_batch_rows_kernel(const uint4* __restrict__ src,
                                                                     const long long* __restrict__ rows,
                                                                     uint4* __restrict__ dst, long long row_vec,
                                                                     int n_rows, long long n_src_rows, int* status) {
  const long long chunk = (long long)kGatherThreads * kGatherUnroll;
  const long long chunks_per_row = (row_vec + chunk - 1) / chunk;
  const long long total = chunks_per_row * n_rows;
  for (long long c = blockIdx.x; c < total; c += gridDim.x) {
    const int i = (int)(c / chunks_per_row);
    const long long v0 = (c - (long long)i * chunks_per_row) * chunk + threadIdx.x;
    const long long r = rows[i];
    if (r < 0 || r >= n_src_rows) {
      if (threadIdx.x == 0) report_status(status, kBadIndex);
      continue;
    }
    const uint4* s = src + r * row_vec;
    uint4* d = dst + (long long)i * row_vec;
    uint4 buf[kGatherUnroll];
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const long long v = v0 + (long long)u * kGatherThreads;
      if (v < row_vec) buf[u] = s[v];
    }
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const long long v = v0 + (long long)u * kGatherThreads;
      if (v < row_vec) d[v] = buf[u];
    }
  }
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_host_register(void* host_ptr, int64_t bytes, void** device_ptr) {
  CLT_CHECK_ARG(host_ptr && bytes > 0 && device_ptr, "host_register: bad arguments");
  CLT_CHECK_CUDA(cudaHostRegister(host_ptr, (size_t)bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, host_ptr, 0);
  if (e != cudaSuccess) {
    cudaHostUnregister(host_ptr);
    CLT_CHECK_CUDA(e);
  }
  *device_ptr = d;
  return 0;
}

int clt_host_unregister(void* host_ptr) {
  CLT_CHECK_ARG(host_ptr, "host_unregister: bad arguments");
  CLT_CHECK_CUDA(cudaHostUnregister(host_ptr));
  return 0;
}

int clt_gather_batch_rows(const void* src, const int64_t* rows, void* dst, int64_t row_bytes, int n_rows,
                          int64_t n_src_rows, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(src && rows && dst && n_rows > 0 && n_src_rows > 0, "gather_batch_rows: bad arguments");
  CLT_CHECK_ARG(row_bytes > 0 && row_bytes % 16 == 0, "gather_batch_rows: rows must be a multiple of 16 bytes");
  CLT_CHECK_ARG(((uintptr_t)src | (uintptr_t)dst) % 16 == 0, "gather_batch_rows: buffers must be 16-byte aligned");
  const long long row_vec = row_bytes / 16;
  const long long chunk = (long long)kGatherThreads * kGatherUnroll;
  const long long total = ((row_vec + chunk - 1) / chunk) * n_rows;
  const long long cap = (long long)device_sm_count() * 8;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  gather_batch_rows_kernel<<<grid, kGatherThreads, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, (const long long*)rows, (uint4*)dst, row_vec, n_rows, (long long)n_src_rows, status);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
