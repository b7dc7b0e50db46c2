// HBM-bound kernels of the training step that are not contractions:
// standardise + cast of the input batch, reconstruction loss forward and
// backward, decoder row norms, the dead-feature counters and the fused Adam step.
#include "adam.cuh"
#include "common.cuh"
#include "kernels.h"

namespace clt {

template <class T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---------------------------------------------------------------------------------
// Input preparation: xn[l, b, d] = (batch[b, 0, l, d] - mu[l, d]) / sd[l, d], cast to TOut.
// The layer-major output makes every layer's [B, D] matrix one contiguous GEMM operand.
// ---------------------------------------------------------------------------------
template <class TIn, class TOut>
__global__ void prep_input_kernel(const TIn* __restrict__ batch, const float* __restrict__ mu,
                                  const float* __restrict__ sd, TOut* __restrict__ xn, int B, int L, int D,
                                  int halves) {
  const long long total = (long long)B * L * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const long long r = i / D;
    const int l = (int)(r % L);
    const long long b = r / L;
    const float x = to_float<TIn>(batch[((b * halves + 0) * L + l) * D + d]);
    const float v = mu != nullptr ? (x - mu[l * D + d]) / sd[l * D + d] : x;
    xn[((long long)l * B + b) * D + d] = from_float<TOut>(v);
  }
}

// ---- 8-element vector I/O for the streaming kernels -------------------------------------
template <class T>
__device__ __forceinline__ void load8(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&o)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&o)[8]) {
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(h[j]);
    o[2 * j] = f.x, o[2 * j + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    o[2 * j] = __uint_as_float(w[j] << 16);
    o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}
template <class T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 t;
  t.x = pack_bf16x2(v[0], v[1]), t.y = pack_bf16x2(v[2], v[3]);
  t.z = pack_bf16x2(v[4], v[5]), t.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = t;
}

// same as prep_input_kernel, 8 consecutive d per thread (needs D % 8 == 0).  One warp per (token, layer) row:
// the 64-bit index arithmetic is done once per row, not once per 16 bytes (which made this copy-like kernel
// run at half the copy rate).
template <class TIn, class TOut>
__global__ void prep_input_vec_kernel(const TIn* __restrict__ batch, const float* __restrict__ mu,
                                      const float* __restrict__ sd, TOut* __restrict__ xn, int B, int L, int D,
                                      int halves) {
  const int dv = D / 8;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)B * L;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; r < rows; r += nwarps) {
    const int l = (int)(r % L);
    const long long b = r / L;
    const TIn* src = batch + ((b * halves + 0) * L + l) * (long long)D;
    TOut* dst = xn + ((long long)l * B + b) * D;
    const float* ml = mu != nullptr ? mu + (long long)l * D : nullptr;
    const float* sl = mu != nullptr ? sd + (long long)l * D : nullptr;
#pragma unroll 4
    for (int c = lane; c < dv; c += 32) {
      float x[8];
      load8<TIn>(src + 8 * c, x);
      if (ml != nullptr) {
        float m[8], s[8];
        load8<float>(ml + 8 * c, m);
        load8<float>(sl + 8 * c, s);
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = (x[q] - m[q]) / s[q];
      }
      store8<TOut>(dst + 8 * c, x);
    }
  }
}

template <class TIn, class TOut>
static int prep_input_t(const void* batch, const float* mu, const float* sd, void* xn, int B, int L, int D,
                        int halves, cudaStream_t s) {
  const int threads = 256;
  if (D % 8 == 0 && ((uintptr_t)batch | (uintptr_t)xn | (uintptr_t)mu | (uintptr_t)sd) % 16 == 0) {  // (NULL statistics pass)
    const long long rows = (long long)B * L;                       // one warp per row, 8 warps per CTA
    const int blocks = (int)min((rows + 7) / 8, (long long)148 * 16);
    prep_input_vec_kernel<TIn, TOut><<<blocks, threads, 0, s>>>((const TIn*)batch, mu, sd, (TOut*)xn, B, L, D, halves);
  } else {
    const long long total = (long long)B * L * D;
    const int blocks = (int)min((total + threads - 1) / threads, (long long)148 * 16);
    prep_input_kernel<TIn, TOut><<<blocks, threads, 0, s>>>((const TIn*)batch, mu, sd, (TOut*)xn, B, L, D, halves);
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int prep_input(const void* batch, int in_dtype, const float* mu, const float* sd, void* xn, int out_bf16, int B, int L,
               int D, int halves, cudaStream_t s) {
  if (B <= 0) return 0;
  switch (in_dtype * 2 + (out_bf16 ? 1 : 0)) {
    case 0: return prep_input_t<float, float>(batch, mu, sd, xn, B, L, D, halves, s);
    case 1: return prep_input_t<float, __nv_bfloat16>(batch, mu, sd, xn, B, L, D, halves, s);
    case 2: return prep_input_t<__half, float>(batch, mu, sd, xn, B, L, D, halves, s);
    case 3: return prep_input_t<__half, __nv_bfloat16>(batch, mu, sd, xn, B, L, D, halves, s);
    case 4: return prep_input_t<__nv_bfloat16, float>(batch, mu, sd, xn, B, L, D, halves, s);
    case 5: return prep_input_t<__nv_bfloat16, __nv_bfloat16>(batch, mu, sd, xn, B, L, D, halves, s);
  }
  set_error("prep_input: unknown input dtype %d", in_dtype);
  return 1;
}

// ---------------------------------------------------------------------------------
// Reconstruction loss.
//   diff[b,l,d] = recon[b,l,d] - (batch[b,1,l,d] - mu_o[l,d]) / sd_o[l,d]
// forward : acc[0] += sum diff^2
// backward: drecon[l,b,d] = 2 diff * gscale / (B L D)   (cast to TOut, layer-major)
//           db_dec[l,d]  += sum_b of the same (fp32)
// A CTA owns a strip of 32 consecutive (l, d) columns and walks the batch, so the
// bias gradient needs one atomic per column per CTA.
// With aux != null (TopK auxiliary loss) the residual target is err = -diff and
//   adiff = aux[b,l,d] - err = aux + diff ;  acc[1] += sum adiff^2  (NaNs count as 0)
//   d recon = 2 diff gs/(BLD) + 2 adiff a_scale gs/(BLD) ; d aux = 2 adiff a_scale gs/(BLD)
// ---------------------------------------------------------------------------------
template <class TIn>
__global__ void loss_fwd_kernel(const float* __restrict__ recon, const float* __restrict__ aux,
                                const TIn* __restrict__ batch, const float* __restrict__ mu,
                                const float* __restrict__ sd, float* __restrict__ acc, int B, int L, int D) {
  const long long total = (long long)B * L * D;
  float s0 = 0.f, s1 = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % ((long long)L * D));
    const long long b = i / ((long long)L * D);
    const float y = (to_float<TIn>(batch[(b * 2 + 1) * L * D + c]) - mu[c]) / sd[c];
    const float diff = recon[i] - y;
    s0 += diff * diff;
    if (aux != nullptr) {
      const float ad = aux[i] + diff;
      const float sq = ad * ad;
      s1 += (sq == sq) ? sq : 0.f;
    }
  }
  s0 = warp_sum(s0);
  s1 = warp_sum(s1);
  __shared__ float sh[2][32];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[0][w] = s0, sh[1][w] = s1;
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    s0 = warp_sum(lane < nw ? sh[0][lane] : 0.f);
    s1 = warp_sum(lane < nw ? sh[1][lane] : 0.f);
    if (lane == 0) {
      atomicAdd(acc + 0, s0);
      if (aux != nullptr) atomicAdd(acc + 1, s1);
    }
  }
}

// same sums, 8 consecutive (l, d) columns per thread (needs L*D % 8 == 0)
template <class TIn>
__global__ void loss_fwd_vec_kernel(const float* __restrict__ recon, const float* __restrict__ aux,
                                    const TIn* __restrict__ batch, const float* __restrict__ mu,
                                    const float* __restrict__ sd, float* __restrict__ acc, int B, int L, int D) {
  const long long LD = (long long)L * D;
  const long long total = (long long)B * LD / 8;
  float s0 = 0.f, s1 = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 8;
    const long long c = e % LD, b = e / LD;
    float y[8], m[8], sdv[8], r[8];
    load8<TIn>(batch + (b * 2 + 1) * LD + c, y);
    load8<float>(mu + c, m);
    load8<float>(sd + c, sdv);
    load8<float>(recon + e, r);
    float diff[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      diff[q] = r[q] - (y[q] - m[q]) / sdv[q];
      s0 = fmaf(diff[q], diff[q], s0);
    }
    if (aux != nullptr) {
      float a[8];
      load8<float>(aux + e, a);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float ad = a[q] + diff[q];
        const float sq = ad * ad;
        s1 += (sq == sq) ? sq : 0.f;
      }
    }
  }
  s0 = warp_sum(s0);
  s1 = warp_sum(s1);
  __shared__ float sh[2][32];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[0][w] = s0, sh[1][w] = s1;
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    s0 = warp_sum(lane < nw ? sh[0][lane] : 0.f);
    s1 = warp_sum(lane < nw ? sh[1][lane] : 0.f);
    if (lane == 0) {
      atomicAdd(acc + 0, s0);
      if (aux != nullptr) atomicAdd(acc + 1, s1);
    }
  }
}

int loss_fwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu, const float* sd,
             float* acc, int B, int L, int D, cudaStream_t s) {
  if (B <= 0) return 0;
  const long long total = (long long)B * L * D;
  const int threads = 256;
  const bool vec = ((long long)L * D) % 8 == 0 &&
                   ((uintptr_t)recon | (uintptr_t)aux | (uintptr_t)batch | (uintptr_t)mu | (uintptr_t)sd) % 16 == 0;
  const long long work = vec ? total / 8 : total;
  const int blocks = (int)min((work + threads - 1) / threads, (long long)148 * 8);
#define CLT_LF(TI)                                                                                               \
  if (vec)                                                                                                       \
    loss_fwd_vec_kernel<TI><<<blocks, threads, 0, s>>>(recon, aux, (const TI*)batch, mu, sd, acc, B, L, D);      \
  else                                                                                                           \
    loss_fwd_kernel<TI><<<blocks, threads, 0, s>>>(recon, aux, (const TI*)batch, mu, sd, acc, B, L, D)
  if (in_dtype == 0) {
    CLT_LF(float);
  } else if (in_dtype == 1) {
    CLT_LF(__half);
  } else {
    CLT_LF(__nv_bfloat16);
  }
#undef CLT_LF
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <class TIn, class TOut>
__global__ void loss_bwd_kernel(const float* __restrict__ recon, const float* __restrict__ aux,
                                const TIn* __restrict__ batch, const float* __restrict__ mu,
                                const float* __restrict__ sd, const float* __restrict__ gscale, float aux_scale,
                                TOut* __restrict__ drecon, TOut* __restrict__ daux, float* __restrict__ db_dec, int B,
                                int L, int D, int rows_per_cta) {
  // blockDim = (32, 8): x walks 32 columns of the flattened (l, d) axis, y walks batch rows
  const int LD = L * D;
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int b0 = blockIdx.y * rows_per_cta;
  const int b1 = min(B, b0 + rows_per_cta);
  const float gs = (gscale != nullptr ? *gscale : 1.f) / ((float)B * (float)L * (float)D);
  float colsum = 0.f;
  if (c < LD) {
    const int l = c / D, d = c % D;
    const float m = mu[c], sdv = sd[c];
    for (int b = b0 + threadIdx.y; b < b1; b += blockDim.y) {
      const long long i = (long long)b * LD + c;
      const float y = (to_float<TIn>(batch[((long long)b * 2 + 1) * LD + c]) - m) / sdv;
      const float diff = recon[i] - y;
      float g = 2.f * diff * gs;
      const long long o = ((long long)l * B + b) * D + d;
      if (aux != nullptr) {
        const float ad = aux[i] + diff;
        float ga = 2.f * ad * aux_scale * gs;
        if (!(ad * ad == ad * ad)) ga = 0.f;  // nan_to_num on the squared error
        g += ga;
        daux[o] = from_float<TOut>(ga);
        colsum += ga;  // the auxiliary reconstruction carries the decoder bias too
      }
      drecon[o] = from_float<TOut>(g);
      colsum += g;
    }
  }
  __shared__ float sh[8][33];
  sh[threadIdx.y][threadIdx.x] = colsum;
  __syncthreads();
  if (threadIdx.y == 0 && c < LD) {
    float t = 0.f;
    for (int j = 0; j < (int)blockDim.y; ++j) t += sh[j][threadIdx.x];
    if (t != 0.f) atomicAdd(db_dec + c, t);
  }
}

// same computation, 4 consecutive columns per thread (needs D % 4 == 0): blockDim (32, 8) covers
// 128 columns; 16-byte loads of the reconstruction, 8-byte loads/stores of the 16-bit tensors
template <class TIn, class TOut>
__global__ void loss_bwd_vec_kernel(const float* __restrict__ recon, const float* __restrict__ aux,
                                    const TIn* __restrict__ batch, const float* __restrict__ mu,
                                    const float* __restrict__ sd, const float* __restrict__ gscale, float aux_scale,
                                    TOut* __restrict__ drecon, TOut* __restrict__ daux, float* __restrict__ db_dec,
                                    int B, int L, int D, int rows_per_cta) {
  const int LD = L * D;
  const int c = (blockIdx.x * 32 + threadIdx.x) * 4;
  const int b0 = blockIdx.y * rows_per_cta;
  const int b1 = min(B, b0 + rows_per_cta);
  const float gs = (gscale != nullptr ? *gscale : 1.f) / ((float)B * (float)L * (float)D);
  float cs[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < LD) {
    const int l = c / D, d = c % D;
    const float4 m = *reinterpret_cast<const float4*>(mu + c), sv = *reinterpret_cast<const float4*>(sd + c);
    const float mm[4] = {m.x, m.y, m.z, m.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
    for (int b = b0 + threadIdx.y; b < b1; b += blockDim.y) {
      const long long i = (long long)b * LD + c;
      const TIn* yp = batch + ((long long)b * 2 + 1) * LD + c;
      const float4 r4 = *reinterpret_cast<const float4*>(recon + i);
      const float rr[4] = {r4.x, r4.y, r4.z, r4.w};
      float aa[4] = {0.f, 0.f, 0.f, 0.f};
      if (aux != nullptr) {
        const float4 a4 = *reinterpret_cast<const float4*>(aux + i);
        aa[0] = a4.x, aa[1] = a4.y, aa[2] = a4.z, aa[3] = a4.w;
      }
      float g[4], ga[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float y = (to_float<TIn>(yp[q]) - mm[q]) / ss[q];
        const float diff = rr[q] - y;
        g[q] = 2.f * diff * gs;
        ga[q] = 0.f;
        if (aux != nullptr) {
          const float ad = aa[q] + diff;
          ga[q] = (ad * ad == ad * ad) ? 2.f * ad * aux_scale * gs : 0.f;
          g[q] += ga[q];
          cs[q] += ga[q];
        }
        cs[q] += g[q];
      }
      const long long o = ((long long)l * B + b) * D + d;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        drecon[o + q] = from_float<TOut>(g[q]);
        if (aux != nullptr) daux[o + q] = from_float<TOut>(ga[q]);
      }
    }
  }
  __shared__ float sh[8][32][4];
#pragma unroll
  for (int q = 0; q < 4; ++q) sh[threadIdx.y][threadIdx.x][q] = cs[q];
  __syncthreads();
  if (threadIdx.y == 0 && c < LD) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float t = 0.f;
      for (int j = 0; j < (int)blockDim.y; ++j) t += sh[j][threadIdx.x][q];
      if (t != 0.f) atomicAdd(db_dec + c + q, t);
    }
  }
}

// Loss backward for the token rows this rank owns, with the all-gather fused in: the rank holds the
// summed reconstructions of rows [b_lo, b_lo + b_cnt) as [b_cnt, L, D]; the gradient rows it derives
// are written straight into every rank's [L, B, D] gradient buffer (16/8-byte stores over NVLink for
// the peers), so no collective has to move them afterwards.  db_dec receives this rank's partial
// column sums.  Same arithmetic as loss_bwd_vec_kernel.
// out[i] = sum over slots of slots[s * n + i]: the owner's local reduction of the partial rows that the
// ranks stored into its slots.  n % 4 == 0.
__global__ void sum_slots_kernel(const float4* __restrict__ slots, float4* __restrict__ out, int n_slots, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 a = __ldcs(slots + i);
    for (int s = 1; s < n_slots; ++s) {
      const float4 b = __ldcs(slots + (long long)s * n4 + i);
      a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
    }
    out[i] = a;
  }
}

// same with bf16 slots: 8 values per thread
__global__ void sum_slots_bf16_kernel(const uint4* __restrict__ slots, float4* __restrict__ out, int n_slots,
                                      long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_slots; ++s) {
      const uint4 t = __ldcs(slots + (long long)s * n8 + i);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a[2 * j] += __uint_as_float(w[j] << 16);
        a[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    out[2 * i] = make_float4(a[0], a[1], a[2], a[3]);
    out[2 * i + 1] = make_float4(a[4], a[5], a[6], a[7]);
  }
}

int sum_slots(const void* slots, float* out, int n_slots, long long n, int slots_bf16, cudaStream_t s) {
  if (n <= 0) return 0;
  if (slots_bf16) {
    const long long n8 = n / 8;
    const int blocks = (int)min((n8 + 255) / 256, (long long)148 * 16);
    sum_slots_bf16_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const uint4*>(slots), reinterpret_cast<float4*>(out),
                                                 n_slots, n8);
    CLT_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  const long long n4 = n / 4;
  const int blocks = (int)min((n4 + 255) / 256, (long long)148 * 16);
  sum_slots_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(slots), reinterpret_cast<float4*>(out),
                                          n_slots, n4);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

constexpr int kMaxPushRanks = 16;
struct PushPtrs {
  unsigned long long drecon[kMaxPushRanks];
  unsigned long long daux[kMaxPushRanks];
  int n;
};

template <class TOut>
__device__ __forceinline__ void store8_as(TOut* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8_as<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8_as<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  uint4 t;
  t.x = *reinterpret_cast<unsigned*>(&a), t.y = *reinterpret_cast<unsigned*>(&b);
  t.z = *reinterpret_cast<unsigned*>(&c), t.w = *reinterpret_cast<unsigned*>(&d);
  *reinterpret_cast<uint4*>(p) = t;
}

// 8 consecutive columns per thread (blockDim (32, 8) covers 256 columns): the gradient rows leave as
// 16-byte stores, which is what the NVLink path to the peers' buffers wants.  Needs D % 8 == 0.
template <class TIn, class TOut>
__global__ void loss_bwd_push_kernel(const float* __restrict__ recon, const float* __restrict__ aux,
                                     const TIn* __restrict__ batch, const float* __restrict__ mu,
                                     const float* __restrict__ sd, const float* __restrict__ gscale, float aux_scale,
                                     PushPtrs dst, float* __restrict__ db_dec, int B, int b_lo, int b_cnt, int L,
                                     int D, int rows_per_cta) {
  const int LD = L * D;
  const int c = (blockIdx.x * 32 + threadIdx.x) * 8;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(b_cnt, r0 + rows_per_cta);
  const float gs = (gscale != nullptr ? *gscale : 1.f) / ((float)B * (float)L * (float)D);
  float cs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < LD) {
    const int l = c / D, d = c % D;
    float mm[8], ss[8];
    load8<float>(mu + c, mm);
    load8<float>(sd + c, ss);
    for (int r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      const int b = b_lo + r;
      const long long i = (long long)r * LD + c;
      float y[8], rr[8], aa[8];
      load8<TIn>(batch + ((long long)b * 2 + 1) * LD + c, y);
      load8<float>(recon + i, rr);
      if (aux != nullptr) load8<float>(aux + i, aa);
      float g[8], ga[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float diff = rr[q] - (y[q] - mm[q]) / ss[q];
        g[q] = 2.f * diff * gs;
        ga[q] = 0.f;
        if (aux != nullptr) {
          const float ad = aa[q] + diff;
          ga[q] = (ad * ad == ad * ad) ? 2.f * ad * aux_scale * gs : 0.f;
          g[q] += ga[q];
          cs[q] += ga[q];
        }
        cs[q] += g[q];
      }
      const long long o = ((long long)l * B + b) * D + d;
      for (int k = 0; k < dst.n; ++k) {
        store8_as<TOut>(reinterpret_cast<TOut*>(dst.drecon[k]) + o, g);
        if (aux != nullptr) store8_as<TOut>(reinterpret_cast<TOut*>(dst.daux[k]) + o, ga);
      }
    }
  }
  __shared__ float sh[8][32][9];
#pragma unroll
  for (int q = 0; q < 8; ++q) sh[threadIdx.y][threadIdx.x][q] = cs[q];
  __syncthreads();
  if (threadIdx.y == 0 && c < LD) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float t = 0.f;
      for (int j = 0; j < (int)blockDim.y; ++j) t += sh[j][threadIdx.x][q];
      if (t != 0.f) atomicAdd(db_dec + c + q, t);
    }
  }
}

int loss_bwd_push(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu,
                  const float* sd, const float* gscale, float aux_scale, const unsigned long long* drecon_ptrs,
                  const unsigned long long* daux_ptrs, int n_ranks, int out_bf16, float* db_dec, int B, int b_lo,
                  int b_cnt, int L, int D, cudaStream_t s) {
  if (b_cnt <= 0) return 0;
  if (n_ranks > kMaxPushRanks) {
    set_error("loss_bwd_push: %d ranks, at most %d", n_ranks, kMaxPushRanks);
    return 1;
  }
  PushPtrs dst;
  dst.n = n_ranks;
  for (int k = 0; k < n_ranks; ++k) dst.drecon[k] = drecon_ptrs[k], dst.daux[k] = daux_ptrs ? daux_ptrs[k] : 0ull;
  const int LD = L * D;
  const int rows_per_cta = 64;
  dim3 grid((LD / 8 + 31) / 32, (b_cnt + rows_per_cta - 1) / rows_per_cta), block(32, 8);
#define CLT_LBP(TI, TO)                                                                                            \
  loss_bwd_push_kernel<TI, TO><<<grid, block, 0, s>>>(recon, aux, (const TI*)batch, mu, sd, gscale, aux_scale, dst, \
                                                      db_dec, B, b_lo, b_cnt, L, D, rows_per_cta)
  switch (in_dtype * 2 + (out_bf16 ? 1 : 0)) {
    case 0: CLT_LBP(float, float); break;
    case 1: CLT_LBP(float, __nv_bfloat16); break;
    case 2: CLT_LBP(__half, float); break;
    case 3: CLT_LBP(__half, __nv_bfloat16); break;
    case 4: CLT_LBP(__nv_bfloat16, float); break;
    case 5: CLT_LBP(__nv_bfloat16, __nv_bfloat16); break;
    default: set_error("loss_bwd_push: unknown input dtype %d", in_dtype); return 1;
  }
#undef CLT_LBP
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int loss_bwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu, const float* sd,
             const float* gscale, float aux_scale, void* drecon, void* daux, int out_bf16, float* db_dec, int B, int L,
             int D, cudaStream_t s) {
  if (B <= 0) return 0;
  const int LD = L * D;
  const int rows_per_cta = 256;
  const bool vec = D % 4 == 0 && ((uintptr_t)recon | (uintptr_t)aux | (uintptr_t)mu | (uintptr_t)sd) % 16 == 0;
  dim3 grid(vec ? (LD / 4 + 31) / 32 : (LD + 31) / 32, (B + rows_per_cta - 1) / rows_per_cta), block(32, 8);
#define CLT_LB(TI, TO)                                                                                            \
  if (vec)                                                                                                        \
    loss_bwd_vec_kernel<TI, TO><<<grid, block, 0, s>>>(recon, aux, (const TI*)batch, mu, sd, gscale, aux_scale,   \
                                                       (TO*)drecon, (TO*)daux, db_dec, B, L, D, rows_per_cta);    \
  else                                                                                                            \
    loss_bwd_kernel<TI, TO><<<grid, block, 0, s>>>(recon, aux, (const TI*)batch, mu, sd, gscale, aux_scale,       \
                                                   (TO*)drecon, (TO*)daux, db_dec, B, L, D, rows_per_cta)
  switch (in_dtype * 2 + (out_bf16 ? 1 : 0)) {
    case 0: CLT_LB(float, float); break;
    case 1: CLT_LB(float, __nv_bfloat16); break;
    case 2: CLT_LB(__half, float); break;
    case 3: CLT_LB(__half, __nv_bfloat16); break;
    case 4: CLT_LB(__nv_bfloat16, float); break;
    case 5: CLT_LB(__nv_bfloat16, __nv_bfloat16); break;
    default: set_error("loss_bwd: unknown input dtype %d", in_dtype); return 1;
  }
#undef CLT_LB
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------
// (Jump)ReLU forward / backward as streaming kernels over z [L, B, F].
// When the contraction length is short (d_acts of a few hundred) the tensor-core main loop of a
// tile is shorter than a fused activation epilogue, so the encoder contraction only stores z and
// these kernels do the rest at HBM speed; for long contractions the fused epilogues are used.
// A thread owns 8 consecutive features: their bias / threshold / norm live in registers, the
// per-feature sums accumulate in registers over the CTA's rows and leave with one atomic each.
//
// forward : feat = pre [pre > theta, pre > 0], pre = z + b;  loss_acc[0] += sum relu(-pre),
//           loss_acc[1] += sum tanh(feat n c) (or the product);  fired bits
// backward: dpre, dtheta, db_enc, d dec_norm from g = dL/dfeat exactly as csrc/epilogues.cuh states
// ---------------------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(128)
act_fwd_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, const float* __restrict__ theta,
               const float* __restrict__ dec_norm, T* __restrict__ feat, unsigned* __restrict__ fired_bits,
               float* __restrict__ loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int F,
               int rows_per_cta) {
  const int l = blockIdx.z;
  const int f0 = (blockIdx.x * 128 + threadIdx.x) * 8;
  const int r0 = blockIdx.y * rows_per_cta, r1 = min(B, r0 + rows_per_cta);
  float s_pre = 0.f, s_sp = 0.f;
  if (f0 < F) {
    float bb[8], tt[8], nn[8];
    load8<float>(b_enc + (size_t)l * F + f0, bb);
#pragma unroll
    for (int q = 0; q < 8; ++q) tt[q] = 0.f, nn[q] = 0.f;
    if (theta != nullptr) load8<float>(theta + (size_t)l * F + f0, tt);
    const bool sp = dec_norm != nullptr;
    if (sp) {
      load8<float>(dec_norm + (size_t)l * F + f0, nn);
#pragma unroll
      for (int q = 0; q < 8; ++q) nn[q] *= c_sparsity;
    }
    unsigned mask = 0u;
    for (int r = r0; r < r1; ++r) {
      const size_t o = ((size_t)l * B + r) * F + f0;
      float zv[8], fv[8];
      load8<T>(z + o, zv);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float pre = zv[q] + bb[q];
        const float f = (pre > tt[q] && pre > 0.f) ? pre : 0.f;
        fv[q] = f;
        mask |= (f > 0.f) ? (1u << q) : 0u;
        if (want_pre) s_pre += fmaxf(-pre, 0.f);
        if (sp) {
          const float w = f * nn[q];
          s_sp += use_tanh ? tanhf(w) : w;
        }
      }
      store8<T>(feat + o, fv);
    }
    if (fired_bits != nullptr && mask != 0u)
      atomicOr(fired_bits + (size_t)l * ((F + 31) / 32) + f0 / 32, mask << (f0 & 31));
  }
  s_pre = warp_sum(s_pre);
  s_sp = warp_sum(s_sp);
  if ((threadIdx.x & 31) == 0) {
    if (s_pre != 0.f) atomicAdd(loss_acc + 0, s_pre);
    if (s_sp != 0.f) atomicAdd(loss_acc + 1, s_sp);
  }
}

template <class T>
__global__ void __launch_bounds__(128)
act_bwd_kernel(const T* __restrict__ g, const T* __restrict__ z, const float* __restrict__ b_enc,
               const float* __restrict__ theta, const float* __restrict__ dec_norm, T* __restrict__ dpre,
               float* __restrict__ dtheta, float* __restrict__ dbenc, float* __restrict__ dnorm, float bandwidth,
               float lam_, float c_sparsity, float pal_, int use_tanh, const float* __restrict__ gscale, int B, int F,
               int rows_per_cta) {
  const int l = blockIdx.z;
  const int f0 = (blockIdx.x * 128 + threadIdx.x) * 8;
  if (f0 >= F) return;
  const int r0 = blockIdx.y * rows_per_cta, r1 = min(B, r0 + rows_per_cta);
  const float gsc = gscale != nullptr ? __ldg(gscale) : 1.f;
  const float lam = lam_ * gsc, pal = pal_ * gsc;
  const float hb = 0.5f * bandwidth;
  const bool relu = theta == nullptr;
  const bool sp = dec_norm != nullptr;
  const float pass_lim = relu ? 0.f : -1.0e-45f;   // JumpReLU passes pre >= 0, ReLU pre > 0
  float bb[8], tt[8], nn[8], cc[8];
  load8<float>(b_enc + (size_t)l * F + f0, bb);
#pragma unroll
  for (int q = 0; q < 8; ++q) tt[q] = 0.f, nn[q] = 0.f, cc[q] = 0.f;
  if (!relu) {
    load8<float>(theta + (size_t)l * F + f0, tt);
#pragma unroll
    for (int q = 0; q < 8; ++q) cc[q] = -tt[q] / bandwidth;
  }
  if (sp) {
    load8<float>(dec_norm + (size_t)l * F + f0, nn);
#pragma unroll
    for (int q = 0; q < 8; ++q) nn[q] *= c_sparsity;
  }
  float sb[8], st[8], sn[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) sb[q] = 0.f, st[q] = 0.f, sn[q] = 0.f;
  for (int r = r0; r < r1; ++r) {
    const size_t o = ((size_t)l * B + r) * F + f0;
    float gv[8], zv[8], dp[8];
    load8<T>(g + o, gv);
    load8<T>(z + o, zv);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float th = tt[q];
      const float pre = zv[q] + bb[q];
      float gs = gv[q];
      if (sp) {
        const float f = (pre > th && pre > 0.f) ? pre : 0.f;
        float d1 = 1.f;
        if (use_tanh) {
          const float tw = tanhf(f * nn[q]);
          d1 = 1.f - tw * tw;
        }
        gs = fmaf(lam * d1, nn[q], gs);
        sn[q] = fmaf(lam * d1 * c_sparsity, f, sn[q]);
      }
      const float d = pre - th;
      const bool rect = (d > -hb) && !(d > hb);
      float x = (pre > pass_lim) ? gs : 0.f;
      x = (pre < 0.f) ? x - pal : x;
      dp[q] = x;
      sb[q] += x;
      st[q] += rect ? cc[q] * gs : 0.f;
    }
    store8<T>(dpre + o, dp);
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const size_t i = (size_t)l * F + f0 + q;
    if (sb[q] != 0.f) atomicAdd(dbenc + i, sb[q]);
    if (dtheta != nullptr && st[q] != 0.f) atomicAdd(dtheta + i, st[q]);
    if (dnorm != nullptr && sn[q] != 0.f) atomicAdd(dnorm + i, sn[q]);
  }
}

static int act_rows_per_cta(int B) { return B >= 2048 ? 250 : (B >= 256 ? 64 : 16); }

int act_fwd(const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* feat,
            unsigned* fired_bits, float* loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int L, int F,
            int bf16, cudaStream_t s) {
  if (B <= 0) return 0;
  CLT_CHECK_ARG(F % 8 == 0, "act_fwd: d_features=%d must be a multiple of 8", F);
  const int rpc = act_rows_per_cta(B);
  dim3 grid((F / 8 + 127) / 128, (B + rpc - 1) / rpc, L);
  CLT_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "act_fwd: grid too large");
  if (bf16)
    act_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((const __nv_bfloat16*)z, b_enc, theta, dec_norm,
                                                       (__nv_bfloat16*)feat, fired_bits, loss_acc, c_sparsity, use_tanh,
                                                       want_pre, B, F, rpc);
  else
    act_fwd_kernel<float><<<grid, 128, 0, s>>>((const float*)z, b_enc, theta, dec_norm, (float*)feat, fired_bits,
                                               loss_acc, c_sparsity, use_tanh, want_pre, B, F, rpc);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int act_bwd(const void* g, const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* dpre,
            float* dtheta, float* dbenc, float* dnorm, float bandwidth, float lam, float c_sparsity, float pal,
            int use_tanh, const float* gscale, int B, int L, int F, int bf16, cudaStream_t s) {
  if (B <= 0) return 0;
  CLT_CHECK_ARG(F % 8 == 0, "act_bwd: d_features=%d must be a multiple of 8", F);
  CLT_CHECK_ARG(bandwidth > 0.f, "act_bwd: bandwidth must be positive");
  const int rpc = act_rows_per_cta(B);
  dim3 grid((F / 8 + 127) / 128, (B + rpc - 1) / rpc, L);
  CLT_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "act_bwd: grid too large");
  if (bf16)
    act_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)z, b_enc, theta,
                                                       dec_norm, (__nv_bfloat16*)dpre, dtheta, dbenc, dnorm, bandwidth,
                                                       lam, c_sparsity, pal, use_tanh, gscale, B, F, rpc);
  else
    act_bwd_kernel<float><<<grid, 128, 0, s>>>((const float*)g, (const float*)z, b_enc, theta, dec_norm, (float*)dpre,
                                               dtheta, dbenc, dnorm, bandwidth, lam, c_sparsity, pal, use_tanh, gscale,
                                               B, F, rpc);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------
// Decoder row norms  n[s, f] = sqrt( sum over blocks (t, s) of |W[pair(t,s), f, :]|^2 ).
// crosslayer = 0: one block per layer (per-layer decoder), n[l, f] = |W[l, f, :]|.
// One warp per (s, f).
// ---------------------------------------------------------------------------------
__global__ void dec_norm_kernel(const float* __restrict__ W, float* __restrict__ out, int L, int F, int D,
                                int crosslayer) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= L * F) return;
  const int s = warp / F, f = warp % F;
  float acc = 0.f;
  const int t_end = crosslayer ? L : s + 1;
  for (int t = s; t < t_end; ++t) {
    const long long p = crosslayer ? (long long)t * (t + 1) / 2 + s : s;
    const float* row = W + (p * F + f) * D;
    for (int d = lane; d < D; d += 32) {
      const float w = row[d];
      acc = fmaf(w, w, acc);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[warp] = sqrtf(acc);
}

int dec_norms(const float* W, float* out, int L, int F, int D, int crosslayer, cudaStream_t s) {
  const long long warps = (long long)L * F;
  if (warps <= 0) return 0;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  dec_norm_kernel<<<(unsigned)blocks, threads, 0, s>>>(W, out, L, F, D, crosslayer);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// rowcoef[s, f] = dnorm[s, f] / n[s, f]  (0 where the norm is 0)
__global__ void norm_coef_kernel(const float* dnorm, const float* n, float* out, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = n[i] > 0.f ? dnorm[i] / n[i] : 0.f;
}
int norm_coef(const float* dnorm, const float* n, float* out, int count, cudaStream_t s) {
  if (count <= 0) return 0;
  norm_coef_kernel<<<(count + 255) / 256, 256, 0, s>>>(dnorm, n, out, count);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------
// Dead-feature counters: last_active[fired] = 0; last_active += B; dead = last_active > limit.
// fired_bits holds one bit per feature ([L, ceil(F/32)] words, set by the encoder or
// selection kernels); the words are cleared here for the next step.
// ---------------------------------------------------------------------------------
__global__ void dead_update_kernel(long long* last_active, unsigned* fired_bits, unsigned char* dead, long long B,
                                   long long limit, int F, int* dead_count, int* soon_dead) {
  const int l = blockIdx.y;
  const int f = blockIdx.x * blockDim.x + threadIdx.x;  // a warp covers one 32-feature word
  const int words = (F + 31) / 32;
  unsigned word = 0u;
  if (f < F) word = fired_bits[(size_t)l * words + f / 32];
  __syncwarp();
  bool is_dead = false, is_soon = false;
  if (f < F) {
    const size_t i = (size_t)l * F + f;
    long long v = ((word >> (f & 31)) & 1u) ? 0 : last_active[i];
    v += B;
    last_active[i] = v;
    is_dead = v > limit;
    is_soon = v + 2 * B > limit;   // dead within the next two steps unless it fires
    if (dead != nullptr) dead[i] = is_dead ? 1 : 0;
    if ((f & 31) == 0) fired_bits[(size_t)l * words + f / 32] = 0u;
  }
  if (dead_count != nullptr) {
    const int n = __popc(__ballot_sync(0xffffffffu, is_dead));
    if ((threadIdx.x & 31) == 0 && n) atomicAdd(dead_count, n);
  }
  if (soon_dead != nullptr) {
    const int n = __popc(__ballot_sync(0xffffffffu, is_soon));
    if ((threadIdx.x & 31) == 0 && n) atomicAdd(soon_dead + l, n);
  }
}
int dead_update(long long* last_active, unsigned* fired_bits, unsigned char* dead, long long B, long long limit, int L,
                int F, int* dead_count, int* soon_dead, cudaStream_t s) {
  if (L <= 0 || F <= 0) return 0;
  if (dead_count != nullptr) CLT_CHECK_CUDA(cudaMemsetAsync(dead_count, 0, sizeof(int), s));
  if (soon_dead != nullptr) CLT_CHECK_CUDA(cudaMemsetAsync(soon_dead, 0, sizeof(int) * L, s));
  dim3 grid((F + 255) / 256, L);
  dead_update_kernel<<<grid, 256, 0, s>>>(last_active, fired_bits, dead, B, limit, F, dead_count, soon_dead);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------
// Fused Adam over one flat fp32 buffer, optionally refreshing the bf16 copy that
// the tensor-core kernels read.  28 bytes of traffic per parameter (+2 for the copy).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                   float* __restrict__ m, float* __restrict__ v,
                                                   __nv_bfloat16* __restrict__ shadow, long long n, AdamScalars a) {
  const long long n4 = n / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = __ldcs(reinterpret_cast<const float4*>(g) + i);
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    adam_one(pp.x, gg.x, mm.x, vv.x, a);
    adam_one(pp.y, gg.y, mm.y, vv.y, a);
    adam_one(pp.z, gg.z, mm.z, vv.z, a);
    adam_one(pp.w, gg.w, mm.w, vv.w, a);
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (shadow != nullptr) {
      uint2 s;
      s.x = pack_bf16x2(pp.x, pp.y);
      s.y = pack_bf16x2(pp.z, pp.w);
      reinterpret_cast<uint2*>(shadow)[i] = s;
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float pp = p[i], mm = m[i], vv = v[i];
    adam_one(pp, g[i], mm, vv, a);
    p[i] = pp, m[i] = mm, v[i] = vv;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(pp);
  }
}

int adam_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float beta1,
              float beta2, float eps, float weight_decay, int decoupled, long long step, int num_sms, cudaStream_t s) {
  if (n <= 0) return 0;
  CLT_CHECK_ARG(step >= 1, "adam_step: step counts from 1 (got %lld)", step);
  CLT_CHECK_ARG(((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) % 16 == 0,
                "adam_step: buffers must be 16-byte aligned");
  const AdamScalars a = make_adam_scalars(lr, beta1, beta2, eps, weight_decay, decoupled, step);
  const int threads = 256;
  const long long want = (n / 4 + threads - 1) / threads + 1;
  const long long cap = (long long)num_sms * 8;
  adam_kernel<<<(unsigned)(want < cap ? want : cap), threads, 0, s>>>(p, g, m, v, (__nv_bfloat16*)shadow_bf16, n, a);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// fp32 -> bf16 copy (initial shadows, and after a state-dict load)
__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}
int cast_bf16(const float* src, void* dst, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  cast_bf16_kernel<<<(unsigned)(want < 148 * 16 ? want : 148 * 16), 256, 0, s>>>(src, (__nv_bfloat16*)dst, n);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------
// Scalar loss assembly on the device (no host round trip):
//   loss = acc[0] / (B L D) + lam * acc_sp / B + pal * acc_pre / (B L) + aux_scale * acc[1] / (B L D)
// terms[0..3] receive the four summands.
// ---------------------------------------------------------------------------------
__global__ void finalize_loss_kernel(const float* mse_acc, const float* enc_acc, float* loss, float* terms, float inv_bld,
                                     float lam_over_b, float pal_over_bl, float aux_scale) {
  const float mse = mse_acc[0] * inv_bld;
  const float aux = aux_scale != 0.f ? aux_scale * mse_acc[1] * inv_bld : 0.f;
  const float pre = enc_acc != nullptr ? pal_over_bl * enc_acc[0] : 0.f;
  const float sp = enc_acc != nullptr ? lam_over_b * enc_acc[1] : 0.f;
  terms[0] = mse, terms[1] = sp, terms[2] = pre, terms[3] = aux;
  loss[0] = mse + sp + pre + aux;
}
int finalize_loss(const float* mse_acc, const float* enc_acc, float* loss, float* terms, float inv_bld, float lam_over_b,
                  float pal_over_bl, float aux_scale, cudaStream_t s) {
  finalize_loss_kernel<<<1, 1, 0, s>>>(mse_acc, enc_acc, loss, terms, inv_bld, lam_over_b, pal_over_bl, aux_scale);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace clt
