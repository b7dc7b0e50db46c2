// Decoder backward of the sparse (TopK / BatchTopK) step with the optimizer applied in the same pass.
//
// The plain pair of kernels moves every decoder parameter three times per step: the feature-major
// backward reads the bf16 operand row and writes the fp32 gradient row (6 B/parameter), then the Adam
// kernel reads parameter, gradient and both moments and writes parameter, moments and the bf16 copy
// (30 B/parameter).  Here one warp owns a 256-column part of a decoder row from the first load to the
// last store:
//
//   p, m, v   <- the part's master weights and moments           (12 B/parameter read)
//   g          = sum over the tokens that selected the feature of val * drecon[t, token, :]
//                (+ the row of the auxiliary dead-feature gradient, if the feature is dead)
//   dval      += bf16(p) . drecon[t, token, :]     (bf16(p) IS the operand copy the forward used)
//   Adam(p, g, m, v);  store p, m, v and the refreshed bf16 copy  (14 B/parameter written)
//
// so the gradient never exists in memory and the operand copy is never read: 26 B/parameter.  Rows of
// features nobody selected still get their moment decay and parameter step (g = 0), which keeps the
// result equal to torch.optim.Adam on the dense gradient.
//
// Work unit = (8 consecutive features of one decoder block) x (one 256-column part): the features'
// entries are contiguous in the feature-major list, so a unit reads 9 column pointers and walks its
// entries once; the parts of a row meet in dval by atomic adds of their partial dot products.  With 8
// values of p, m, v and g per lane the kernel needs 80 registers, so 24 warps are resident per SM; wider
// parts (24 values per lane, 8 warps per SM) left every warp waiting for its own loads at 0.60 of the
// HBM roofline, and a variant that streamed p, m, v through shared memory with cp.async.bulk and
// mbarriers was bound by the instruction issue of its few consumer warps (0.43 - 0.65).  The update
// uses sqrt.approx / div.approx (adam_fast): at this occupancy the instruction count per element,
// not the memory system, is the limit.
#include "../../include/clt_b200.h"
#include "adam.cuh"
#include "common.cuh"
#include "gemm.cuh"
#include "kernels.h"

namespace clt {
namespace {

struct F8 {
  float4 a, b;
};
__device__ __forceinline__ F8 ld_f8(const float* p) {
  F8 r;
  r.a = *reinterpret_cast<const float4*>(p);
  r.b = *(reinterpret_cast<const float4*>(p) + 1);
  return r;
}
__device__ __forceinline__ F8 ldg_f8(const float* p) {
  F8 r;
  r.a = __ldg(reinterpret_cast<const float4*>(p));
  r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  return r;
}
__device__ __forceinline__ F8 zero_f8() {
  F8 r;
  r.a = make_float4(0.f, 0.f, 0.f, 0.f);
  r.b = r.a;
  return r;
}
__device__ __forceinline__ void unpack(const F8& r, float (&o)[8]) {
  o[0] = r.a.x, o[1] = r.a.y, o[2] = r.a.z, o[3] = r.a.w, o[4] = r.b.x, o[5] = r.b.y, o[6] = r.b.z, o[7] = r.b.w;
}
__device__ __forceinline__ void st_f8(float* p, const float (&v)[8]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(v[4], v[5], v[6], v[7]));
}

// a chunk of 8 reconstruction-gradient values in its storage format
template <class T>
struct Row8;
template <>
struct Row8<__nv_bfloat16> {
  using Raw = uint4;
  __device__ static __forceinline__ Raw load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ static __forceinline__ Raw zero() { return make_uint4(0, 0, 0, 0); }
  __device__ static __forceinline__ void unpack(const Raw& r, float (&o)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = __uint_as_float(w[j] << 16);
      o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  // the operand the forward contraction read for a master weight
  __device__ static __forceinline__ float operand(float w) { return bf16_round(w); }
};
template <>
struct Row8<float> {
  using Raw = F8;
  __device__ static __forceinline__ Raw load(const float* p) { return ldg_f8(p); }
  __device__ static __forceinline__ Raw zero() { return zero_f8(); }
  __device__ static __forceinline__ void unpack(const Raw& r, float (&o)[8]) { clt::unpack(r, o); }
  __device__ static __forceinline__ float operand(float w) { return w; }
};

template <class T, int VPL>
__global__ void __launch_bounds__(128, 6)
sparse_bwd_dec_adam_kernel(const int* __restrict__ col_ptr, const int* __restrict__ ent, const float* __restrict__ val,
                           const int* __restrict__ etok, long long npl_, float* __restrict__ Wm, float* __restrict__ Mo,
                           float* __restrict__ Vo, __nv_bfloat16* __restrict__ shadow, const T* __restrict__ drecon,
                           float* __restrict__ dval, const float* __restrict__ dW_c, const int* __restrict__ dead_pos,
                           int nd_pad, int B, int L, int D, int F, int k, int crosslayer, long long n_units, int nseg,
                           AdamScalars adam) {
  const long long unit = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (unit >= n_units) return;
  const long long gid = unit / nseg;
  const int seg = (int)(unit % nseg);
  const int gpf = F / 8;
  const int p = (int)(gid / gpf), f0 = (int)(gid % gpf) * 8;
  int s = p, t = p;
  if (crosslayer) pair_split(p, t, s);
  const int nvec = D / 8;
  const int cbase = seg * 32 * VPL;  // first 8-column chunk of this segment
  const size_t npl = (size_t)npl_;
  using R = Row8<T>;
  const int cpv = lane < 9 ? __ldg(col_ptr + (size_t)s * (F + 1) + f0 + lane) : 0;
  const int dpos_l = (dead_pos != nullptr && lane < 8) ? __ldg(dead_pos + (size_t)s * F + f0 + lane) : -1;
  const size_t row0 = ((size_t)p * F + f0) * D;
  // entry metadata, 32 entries at a time
  int base = __shfl_sync(0xffffffffu, cpv, 0);
  const int e_end = __shfl_sync(0xffffffffu, cpv, 8);
  int my_slot = 0, my_tok = 0;
  float my_val = 0.f;
  auto load_chunk = [&](int b0) {
    my_slot = 0, my_tok = 0, my_val = 0.f;
    if (b0 + lane < e_end) {
      my_slot = __ldg(ent + (size_t)s * npl + b0 + lane);
      my_val = __ldg(val + (size_t)s * npl + my_slot);
      my_tok = etok != nullptr ? __ldg(etok + (size_t)s * npl + my_slot) : my_slot / k;
    }
  };
  if (e_end > base) load_chunk(base);
  F8 w_cur[VPL], w_next[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = cbase + lane + 32 * i;
    w_cur[i] = c < nvec ? ld_f8(Wm + row0 + 8 * c) : zero_f8();
    w_next[i] = zero_f8();
  }
#pragma unroll 1
  for (int fi = 0; fi < 8; ++fi) {
    const size_t row = row0 + (size_t)fi * D;
    // this row's moments and the next row's weights: in flight while the entries are processed
    F8 m_r[VPL], v_r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = cbase + lane + 32 * i;
      m_r[i] = c < nvec ? ld_f8(Mo + row + 8 * c) : zero_f8();
      v_r[i] = c < nvec ? ld_f8(Vo + row + 8 * c) : zero_f8();
      if (fi < 7 && c < nvec) w_next[i] = ld_f8(Wm + row + D + 8 * c);
    }
    float g[VPL][8];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int q = 0; q < 8; ++q) g[i][q] = 0.f;
    const int eb = __shfl_sync(0xffffffffu, cpv, fi), ee = __shfl_sync(0xffffffffu, cpv, fi + 1);
    for (int e = eb; e < ee; e += 2) {
      const bool two = e + 1 < ee;
      if (e + 1 - base >= 32) {  // both entries of the pair must lie inside the loaded chunk
        base = e;
        load_chunk(base);
      }
      const int j0 = e - base, j1 = two ? j0 + 1 : j0;
      const int slot0 = __shfl_sync(0xffffffffu, my_slot, j0), slot1 = __shfl_sync(0xffffffffu, my_slot, j1);
      const float v0 = __shfl_sync(0xffffffffu, my_val, j0);
      const float v1 = two ? __shfl_sync(0xffffffffu, my_val, j1) : 0.f;
      const T* dr0 = drecon + ((size_t)t * B + __shfl_sync(0xffffffffu, my_tok, j0)) * D;
      const T* dr1 = drecon + ((size_t)t * B + __shfl_sync(0xffffffffu, my_tok, j1)) * D;
      typename R::Raw x0[VPL], x1[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = cbase + lane + 32 * i;
        x0[i] = c < nvec ? R::load(dr0 + 8 * c) : R::zero();
        x1[i] = (two && c < nvec) ? R::load(dr1 + 8 * c) : R::zero();
      }
      float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float wf[8], xf[8];
        unpack(w_cur[i], wf);
#pragma unroll
        for (int q = 0; q < 8; ++q) wf[q] = R::operand(wf[q]);
        R::unpack(x0[i], xf);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          dot0 = fmaf(wf[q], xf[q], dot0);
          g[i][q] = fmaf(v0, xf[q], g[i][q]);
        }
        R::unpack(x1[i], xf);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          dot1 = fmaf(wf[q], xf[q], dot1);
          g[i][q] = fmaf(v1, xf[q], g[i][q]);
        }
      }
      // both dot products in one butterfly: the lower half-warp ends with dot0, the upper with dot1
      const bool lower = lane < 16;
      float r = (lower ? dot0 : dot1) + __shfl_xor_sync(0xffffffffu, lower ? dot1 : dot0, 16);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
      if (lane == 0) atomicAdd(dval + (size_t)s * npl + slot0, r);
      if (lane == 16 && two) atomicAdd(dval + (size_t)s * npl + slot1, r);
    }
    // gradient of the auxiliary dead-feature loss for this row (dense contraction over the dead features)
    const int dpos = __shfl_sync(0xffffffffu, dpos_l, fi);
    if (dpos >= 0 && dW_c != nullptr) {
      const float* ar = dW_c + ((size_t)p * nd_pad + dpos) * D;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = cbase + lane + 32 * i;
        if (c < nvec) {
          float af[8];
          unpack(ldg_f8(ar + 8 * c), af);
#pragma unroll
          for (int q = 0; q < 8; ++q) g[i][q] += af[q];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = cbase + lane + 32 * i;
      if (c < nvec) {
        float pf[8], mf[8], vf[8];
        unpack(w_cur[i], pf);
        unpack(m_r[i], mf);
        unpack(v_r[i], vf);
#pragma unroll
        for (int q = 0; q < 8; ++q) adam_fast(pf[q], g[i][q], mf[q], vf[q], adam);
        st_f8(Wm + row + 8 * c, pf);
        st_f8(Mo + row + 8 * c, mf);
        st_f8(Vo + row + 8 * c, vf);
        if (shadow != nullptr) {
          uint4 sh;
          sh.x = pack_bf16x2(pf[0], pf[1]), sh.y = pack_bf16x2(pf[2], pf[3]);
          sh.z = pack_bf16x2(pf[4], pf[5]), sh.w = pack_bf16x2(pf[6], pf[7]);
          __stcs(reinterpret_cast<uint4*>(shadow + row + 8 * c), sh);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) w_cur[i] = w_next[i];
  }
}

template <class T>
int launch(const int* col_ptr, const int* ent, const float* val, const int* etok, long long npl, float* W, float* M,
           float* V, void* shadow, const void* drecon, float* dval, const float* dW_c, const int* dead_pos, int nd_pad,
           int B, int L, int D, int F, int k, int crosslayer, const AdamScalars& a, cudaStream_t s) {
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  const int nvec = D / 8;
  const int nseg = (nvec + 31) / 32;   // column parts of 256 columns, one warp each
  const long long n_units = (long long)P * (F / 8) * nseg;
  const long long blocks = (n_units + 3) / 4;
  CLT_CHECK_ARG(blocks < (1ll << 31), "sparse_bwd_dec_adam: too many rows");
  sparse_bwd_dec_adam_kernel<T, 1><<<(unsigned)blocks, 128, 0, s>>>(
      col_ptr, ent, val, etok, npl, W, M, V, (__nv_bfloat16*)shadow, (const T*)drecon, dval, dW_c, dead_pos, nd_pad, B,
      L, D, F, k, crosslayer, n_units, nseg, a);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// dead_pos[l, f] = position of feature f in dead_list[l] (j < n_dead[l]), -1 for live features
__global__ void dead_pos_kernel(const int* __restrict__ dead_list, const int* __restrict__ n_dead,
                                int* __restrict__ dead_pos, int F, int nd_pad) {
  const int l = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < min(n_dead[l], nd_pad)) {
    const int f = dead_list[(size_t)l * F + j];
    if (f >= 0 && f < F) dead_pos[(size_t)l * F + f] = j;
  }
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_dead_positions(const int* dead_list, const int* n_dead, int* dead_pos, int L, int F, int nd_pad,
                       clt_stream_t stream) {
  CLT_CHECK_ARG(dead_list && n_dead && dead_pos && L > 0 && F > 0 && nd_pad > 0, "dead_positions: bad arguments");
  CLT_CHECK_ARG(L <= 65535, "dead_positions: too many layers");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(dead_pos, 0xff, sizeof(int) * (size_t)L * F, s));
  dim3 grid((F + 255) / 256, L);
  dead_pos_kernel<<<grid, 256, 0, s>>>(dead_list, n_dead, dead_pos, F, nd_pad);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_sparse_bwd_dec_adam(const int* col_ptr, const int* ent, const float* val, const int* etok, int64_t npl,
                            float* W_master, float* exp_avg, float* exp_avg_sq, void* shadow_bf16, const void* drecon,
                            float* dval, const float* dW_aux, const int* dead_pos, int nd_pad, int B, int L, int D,
                            int F, int k, int crosslayer, int bf16, float lr, float beta1, float beta2, float eps,
                            float weight_decay, int decoupled, int64_t step, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && F > 0 && k > 0 && npl > 0, "sparse_bwd_dec_adam: bad dims");
  CLT_CHECK_ARG(D % 8 == 0 && F % 8 == 0, "sparse_bwd_dec_adam: d_acts=%d and d_features=%d must be multiples of 8", D,
                F);
  CLT_CHECK_ARG(col_ptr && ent && val && W_master && exp_avg && exp_avg_sq && drecon && dval,
                "sparse_bwd_dec_adam: null pointer");
  CLT_CHECK_ARG((dW_aux == nullptr) == (dead_pos == nullptr), "sparse_bwd_dec_adam: dW_aux and dead_pos go together");
  CLT_CHECK_ARG(dW_aux == nullptr || nd_pad > 0, "sparse_bwd_dec_adam: nd_pad=%d", nd_pad);
  CLT_CHECK_ARG(bf16 == 0 || shadow_bf16 != nullptr, "sparse_bwd_dec_adam: the bf16 path needs the operand copy");
  CLT_CHECK_ARG(step >= 1, "sparse_bwd_dec_adam: step counts from 1 (got %lld)", (long long)step);
  CLT_CHECK_ARG(((uintptr_t)W_master | (uintptr_t)exp_avg | (uintptr_t)exp_avg_sq | (uintptr_t)shadow_bf16 |
                 (uintptr_t)drecon | (uintptr_t)dW_aux) % 16 == 0,
                "sparse_bwd_dec_adam: buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(dval, 0, sizeof(float) * (size_t)L * npl, s));
  const AdamScalars a = make_adam_scalars(lr, beta1, beta2, eps, weight_decay, decoupled, step);
  if (bf16)
    return launch<__nv_bfloat16>(col_ptr, ent, val, etok, npl, W_master, exp_avg, exp_avg_sq, shadow_bf16, drecon, dval,
                                 dW_aux, dead_pos, nd_pad, B, L, D, F, k, crosslayer, a, s);
  return launch<float>(col_ptr, ent, val, etok, npl, W_master, exp_avg, exp_avg_sq, nullptr, drecon, dval, dW_aux,
                       dead_pos, nd_pad, B, L, D, F, k, crosslayer, a, s);
}

}  // extern "C"
