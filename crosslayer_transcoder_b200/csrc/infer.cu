// Element-wise kernels of the inference forward (CrossLayerTranscoder.forward and the per-layer
// forward_layer calls of the reference, crosslayer_transcoder/model/clt.py:134-145, 216-231, 304-317,
// 403-425): layout changes between the token-major tensors of the module surface and the layer-major
// operands of the contraction kernels, with the bias / statistics applied on the way.
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {
namespace {

template <class T>
__device__ __forceinline__ float cvt_in(T v);
template <>
__device__ __forceinline__ float cvt_in<float>(float v) { return v; }
template <>
__device__ __forceinline__ float cvt_in<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out[b, l, f] = src[l, b, f] (+ bias[l, f])     layer-major T -> token-major fp32
template <class T>
__global__ void export_blf_kernel(const T* __restrict__ src, const float* __restrict__ bias, float* __restrict__ out,
                                  int B, int L, long long F) {
  const long long total = (long long)B * L * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long f = i % F;
    const long long r = i / F;
    const int l = (int)(r % L);
    const long long b = r / L;
    float v = cvt_in<T>(src[((long long)l * B + b) * F + f]);
    if (bias != nullptr) v += __ldg(bias + (long long)l * F + f);
    out[i] = v;
  }
}

// dst[l, b, f] = T(src[b, l, f])                  token-major fp32 -> layer-major T
template <class T>
__global__ void import_blf_kernel(const float* __restrict__ src, T* __restrict__ dst, int B, int L, long long F) {
  const long long total = (long long)B * L * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long f = i % F;
    const long long r = i / F;
    const int l = (int)(r % L);
    const long long b = r / L;
    const float v = src[i];
    if constexpr (sizeof(T) == 2)
      dst[((long long)l * B + b) * F + f] = __float2bfloat16_rn(v);
    else
      dst[((long long)l * B + b) * F + f] = v;
  }
}

// out[b, l, d] = recon[b, l, d] * sd[l, d] + mu[l, d]
__global__ void destandardize_kernel(const float* __restrict__ recon, const float* __restrict__ mu,
                                     const float* __restrict__ sd, float* __restrict__ out, long long total, int LD) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % LD);
    out[i] = fmaf(recon[i], __ldg(sd + c), __ldg(mu + c));
  }
}

// dense[token, l, idx] = val for every valid entry of the per-layer lists idx / val [L, npl]; the token of
// entry e is etok[e], or e / k for the fixed-slot lists of the per-row selection (npl = B k)
__global__ void scatter_features_kernel(const int* __restrict__ idx, const float* __restrict__ val,
                                        const int* __restrict__ etok, float* __restrict__ dense, int B, int L, int F,
                                        int k, long long npl, int* status) {
  const long long total = (long long)L * npl;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = val[i];
    if (v == 0.f) continue;
    const int f = idx[i];
    const int l = (int)(i / npl);
    const long long b = etok != nullptr ? (long long)etok[i] : (i - (long long)l * npl) / k;
    if (f < 0 || f >= F || b < 0 || b >= B) {
      report_status(status, kBadIndex);
      continue;
    }
    dense[(b * L + l) * (long long)F + f] = v;
  }
}

inline unsigned grid_for(long long total) {
  const long long want = (total + 255) / 256;
  return (unsigned)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_prep_acts(const void* acts, int in_dtype, const float* mu, const float* sd, void* xn, int bf16, int B, int L,
                  int D, clt_stream_t stream) {
  CLT_CHECK_ARG(acts && xn && B > 0 && L > 0 && D > 0, "prep_acts: bad arguments");
  CLT_CHECK_ARG((mu == nullptr) == (sd == nullptr), "prep_acts: mean and std go together");
  return prep_input(acts, in_dtype, mu, sd, xn, bf16, B, L, D, 1, (cudaStream_t)stream);
}

int clt_export_blf(const void* src, const float* bias, float* out, int B, int L, int64_t F, int bf16,
                   clt_stream_t stream) {
  CLT_CHECK_ARG(src && out && B > 0 && L > 0 && F > 0, "export_blf: bad arguments");
  const long long total = (long long)B * L * F;
  cudaStream_t s = (cudaStream_t)stream;
  if (bf16)
    export_blf_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>((const __nv_bfloat16*)src, bias, out, B, L, F);
  else
    export_blf_kernel<float><<<grid_for(total), 256, 0, s>>>((const float*)src, bias, out, B, L, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_import_blf(const float* src, void* dst, int B, int L, int64_t F, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(src && dst && B > 0 && L > 0 && F > 0, "import_blf: bad arguments");
  const long long total = (long long)B * L * F;
  cudaStream_t s = (cudaStream_t)stream;
  if (bf16)
    import_blf_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(src, (__nv_bfloat16*)dst, B, L, F);
  else
    import_blf_kernel<float><<<grid_for(total), 256, 0, s>>>(src, (float*)dst, B, L, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_destandardize(const float* recon, const float* mu, const float* sd, float* out, int B, int L, int D,
                      clt_stream_t stream) {
  CLT_CHECK_ARG(recon && mu && sd && out && B > 0 && L > 0 && D > 0, "destandardize: bad arguments");
  const long long total = (long long)B * L * D;
  destandardize_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(recon, mu, sd, out, total, L * D);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_scatter_features(const int* idx, const float* val, const int* etok, float* dense, int B, int L, int F, int k,
                         int64_t npl, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(idx && val && dense && B > 0 && L > 0 && F > 0 && k > 0 && npl > 0, "scatter_features: bad arguments");
  CLT_CHECK_ARG(etok != nullptr || npl == (int64_t)B * k, "scatter_features: fixed slots need npl = B*k");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(dense, 0, sizeof(float) * (size_t)B * L * F, s));
  scatter_features_kernel<<<grid_for((long long)L * npl), 256, 0, s>>>(idx, val, etok, dense, B, L, F, k, npl, status);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
