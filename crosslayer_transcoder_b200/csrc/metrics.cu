// Training metrics computed on the device from buffers the step already holds, so that
// logging needs no copy of the [B, L, F] features to the host:
//   recon_stats   per (layer, dim) sums over the tokens from which the fraction of variance
//                 unexplained, the per-layer MSE and the rescaled MSE follow
//   count_active  per-layer number of positive entries (L0) of a dense feature tensor or of
//                 a sparse value list
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {
namespace {

template <class T>
__device__ __forceinline__ float as_float(T v);
template <>
__device__ __forceinline__ float as_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

constexpr int kStatRows = 64;  // tokens per CTA

// out[c, 0..5] += sum over the CTA's tokens of
//   yn, yn^2, (yn - r)^2, (y - (r sd + mu))^2, r, r^2     with yn = (y - mu) / sd, c = l * D + d
template <class TIn>
__global__ void __launch_bounds__(256)
recon_stats_kernel(const float* __restrict__ recon, const TIn* __restrict__ batch, const float* __restrict__ mu,
                   const float* __restrict__ sd, float* __restrict__ out, int b_lo, int n, int LD) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= LD) return;
  const int r0 = blockIdx.y * kStatRows, r1 = min(n, r0 + kStatRows);
  const float m = mu[c], s = sd[c];
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f;
  for (int i = r0; i < r1; ++i) {
    const float r = recon[(size_t)i * LD + c];
    const float y = as_float<TIn>(batch[((size_t)(b_lo + i) * 2 + 1) * LD + c]);
    const float yn = (y - m) / s;
    const float e = yn - r, e2 = y - fmaf(r, s, m);
    a0 += yn, a1 = fmaf(yn, yn, a1), a2 = fmaf(e, e, a2), a3 = fmaf(e2, e2, a3), a4 += r, a5 = fmaf(r, r, a5);
  }
  float* o = out + (size_t)c * 6;
  atomicAdd(o + 0, a0), atomicAdd(o + 1, a1), atomicAdd(o + 2, a2);
  atomicAdd(o + 3, a3), atomicAdd(o + 4, a4), atomicAdd(o + 5, a5);
}

template <class T>
__global__ void __launch_bounds__(256)
count_active_kernel(const T* __restrict__ x, long long n_per_layer, unsigned long long* __restrict__ out) {
  const int l = blockIdx.y;
  const T* xl = x + (size_t)l * n_per_layer;
  int cnt = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_per_layer;
       i += (long long)gridDim.x * blockDim.x)
    cnt += as_float<T>(xl[i]) > 0.f ? 1 : 0;
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  __shared__ int wsum[8];
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < 8; ++w) t += wsum[w];
    if (t) atomicAdd(out + l, (unsigned long long)t);
  }
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_recon_stats(const float* recon_rows, const void* batch, int in_dtype, const float* mu_out, const float* sd_out,
                    float* out, int b_lo, int n_rows, int L, int D, clt_stream_t stream) {
  CLT_CHECK_ARG(recon_rows && batch && mu_out && sd_out && out, "recon_stats: null pointer");
  CLT_CHECK_ARG(L > 0 && D > 0 && b_lo >= 0 && n_rows >= 0, "recon_stats: bad dims");
  if (n_rows == 0) return 0;
  const int LD = L * D;
  dim3 grid((LD + 255) / 256, (n_rows + kStatRows - 1) / kStatRows);
  CLT_CHECK_ARG(grid.y <= 65535, "recon_stats: too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  switch (in_dtype) {
    case 0:
      recon_stats_kernel<float><<<grid, 256, 0, s>>>(recon_rows, (const float*)batch, mu_out, sd_out, out, b_lo,
                                                     n_rows, LD);
      break;
    case 1:
      recon_stats_kernel<__half><<<grid, 256, 0, s>>>(recon_rows, (const __half*)batch, mu_out, sd_out, out, b_lo,
                                                      n_rows, LD);
      break;
    case 2:
      recon_stats_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(recon_rows, (const __nv_bfloat16*)batch, mu_out, sd_out,
                                                             out, b_lo, n_rows, LD);
      break;
    default:
      set_error("recon_stats: unknown input dtype %d", in_dtype);
      return 1;
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_count_active(const void* x, int dtype, int64_t n_per_layer, int L, uint64_t* out, clt_stream_t stream) {
  CLT_CHECK_ARG(x && out && L > 0 && n_per_layer >= 0, "count_active: bad arguments");
  CLT_CHECK_ARG(L <= 65535, "count_active: too many layers");
  if (n_per_layer == 0) return 0;
  const long long want = (n_per_layer + 255) / 256;
  dim3 grid((unsigned)(want < 148 * 4 ? want : 148 * 4), L);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned long long* o = reinterpret_cast<unsigned long long*>(out);
  switch (dtype) {
    case 0: count_active_kernel<float><<<grid, 256, 0, s>>>((const float*)x, n_per_layer, o); break;
    case 1: count_active_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, n_per_layer, o); break;
    case 2: count_active_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, n_per_layer, o); break;
    default:
      set_error("count_active: unknown dtype %d", dtype);
      return 1;
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
