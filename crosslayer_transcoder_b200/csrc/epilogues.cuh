// Epilogue functors of the contraction kernels.
//
// Both contraction kernels (fp32 SIMT, bf16 tcgen05) hand their accumulators to
// the epilogue in the same shape: a warp holds 32 consecutive rows of the output
// tile, each lane one row, and passes 32 consecutive columns of that row at a
// time.  Column reductions over the batch axis are therefore warp shuffles.
//
//   struct Epi {
//     struct Params;                      // pointers and scalars, passed by value
//     struct State;                       // per-thread registers living for the whole kernel
//     static void init(State&);
//     static void apply(const Params&, State&, int z, int row, bool row_ok,
//                       int n0, int M, int N, float (&v)[32]);
//     static void finish(const Params&, State&);   // once per thread, warp-converged
//   };
#pragma once

#include "common.cuh"
#include "gemm.cuh"

namespace clt {
namespace epi {

// ---- 32-wide row segment I/O ------------------------------------------------------
template <class T>
__device__ __forceinline__ void load32(const T* p, int nvalid, bool vec, float (&o)[32]);

template <>
__device__ __forceinline__ void load32<float>(const float* p, int nvalid, bool vec, float (&o)[32]) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 t = reinterpret_cast<const float4*>(p)[i];
      o[4 * i] = t.x, o[4 * i + 1] = t.y, o[4 * i + 2] = t.z, o[4 * i + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = i < nvalid ? p[i] : 0.f;
  }
}

template <>
__device__ __forceinline__ void load32<__nv_bfloat16>(const __nv_bfloat16* p, int nvalid, bool vec, float (&o)[32]) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 t = reinterpret_cast<const uint4*>(p)[i];
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        o[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = i < nvalid ? __bfloat162float(p[i]) : 0.f;
  }
}

template <class T>
__device__ __forceinline__ void store32(T* p, int nvalid, bool vec, const float (&v)[32]);

template <>
__device__ __forceinline__ void store32<float>(float* p, int nvalid, bool vec, const float (&v)[32]) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) p[i] = v[i];
  }
}

template <>
__device__ __forceinline__ void store32<__nv_bfloat16>(__nv_bfloat16* p, int nvalid, bool vec, const float (&v)[32]) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 t;
      t.x = pack_bf16x2(v[8 * i], v[8 * i + 1]);
      t.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
      t.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
      t.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      reinterpret_cast<uint4*>(p)[i] = t;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nvalid) p[i] = __float2bfloat16_rn(v[i]);
  }
}

template <class T>
__device__ __forceinline__ float round_to(float x);
template <>
__device__ __forceinline__ float round_to<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return bf16_round(x); }

template <class T>
__device__ __forceinline__ bool can_vec(int n0, int N) {
  return (n0 + 32 <= N) && (N % (16 / (int)sizeof(T)) == 0);
}

// lane j adds its column total to dst[n0 + j]
__device__ __forceinline__ void col_atomic_add(float* dst, int n0, int N, float colsum) {
  const int lane = threadIdx.x & 31;
  if (n0 + lane < N && colsum != 0.f) atomicAdd(dst + n0 + lane, colsum);
}

// =====================================================================================
// Plain stores
// =====================================================================================
// out[z, row, n] = acc rounded to T   (pre-activations without bias, for the selection kernels)
template <class T>
struct StoreZ {
  struct Params {
    T* out;  // [nz, M, N]
  };
  struct State {};
  __device__ static void init(State&) {}
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32]) {
    if (!row_ok) return;
    T* dst = p.out + ((size_t)z * M + row) * N + n0;
    store32<T>(dst, N - n0, can_vec<T>(n0, N), v);
  }
  __device__ static void finish(const Params&, State&) {}
};

// Decoder forward: out[row, z, n] = acc + bias[z, n]  (fp32, row stride ld, slab stride zstride)
struct DecOut {
  struct Params {
    float* out;
    const float* bias;  // [nz, N] or null
    long long ld, zstride;
  };
  struct State {};
  __device__ static void init(State&) {}
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32]) {
    if (!row_ok) return;
    if (p.bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n0 + i < N) v[i] += __ldg(p.bias + (size_t)z * N + n0 + i);
    }
    float* dst = p.out + (size_t)row * p.ld + (size_t)z * p.zstride + n0;
    const bool vec = (n0 + 32 <= N) && (p.ld % 4 == 0) && (p.zstride % 4 == 0);
    store32<float>(dst, N - n0, vec, v);
  }
  __device__ static void finish(const Params&, State&) {}
};

// Weight gradient: out[z, row, n] = acc (+ rowcoef[zc, row] * w[z, row, n]).
// The optional second term is the gradient of the decoder-norm factor of the
// sparsity penalty: d|W[s,f,:]| / dW = W / |W|, scaled per feature row.
struct GradOut {
  struct Params {
    float* out;            // [nz, M, N]
    const float* rowcoef;  // [n_src, M] or null
    const float* w;        // [nz, M, N] master weights (read only when rowcoef != null)
    int coef_by_source;    // 1: z is a (target, source) pair and rowcoef is indexed by its source layer
  };
  struct State {};
  __device__ static void init(State&) {}
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32]) {
    if (!row_ok) return;
    const size_t off = ((size_t)z * M + row) * N + n0;
    const bool vec = can_vec<float>(n0, N);
    if (p.rowcoef != nullptr) {
      int zc = z;
      if (p.coef_by_source) {
        int t;
        pair_split(z, t, zc);
      }
      const float c = __ldg(p.rowcoef + (size_t)zc * M + row);
      float w[32];
      load32<float>(p.w + off, N - n0, vec, w);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = fmaf(c, w[i], v[i]);
    }
    store32<float>(p.out + off, N - n0, vec, v);
  }
  __device__ static void finish(const Params&, State&) {}
};

// =====================================================================================
// Encoder forward with the (Jump)ReLU fused
// =====================================================================================
// acc -> z = round_T(acc); pre = z + b; feat = pre * [pre > theta and pre > 0].
// Stores z and feat, marks columns that fired, and accumulates the two scalar
// loss terms that depend on every pre-activation:
//   sum relu(-pre)                       (pre-activation loss)
//   sum tanh(feat * dec_norm * c)        (sparsity penalty; without tanh: the product itself)
template <class T>
struct EncJumpReLU {
  struct Params {
    const float* b_enc;     // [nz, N]
    const float* theta;     // [nz, N] or null (plain ReLU)
    const float* dec_norm;  // [nz, N] or null (no sparsity term)
    T* z_out;               // [nz, M, N]
    T* feat_out;            // [nz, M, N]
    int* fired;             // [nz, N] or null
    float* loss_acc;        // [0] += sum relu(-pre), [1] += sum of the sparsity summand
    float c_sparsity;
    int use_tanh;
  };
  struct State {
    float s_pre, s_sp;
  };
  __device__ static void init(State& s) { s.s_pre = 0.f, s.s_sp = 0.f; }
  __device__ static void apply(const Params& p, State& st, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32]) {
    const int lane = threadIdx.x & 31;
    const size_t cz = (size_t)z * N + n0;
    float feat[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const bool ok = row_ok && (n0 + i < N);
      const float zr = round_to<T>(v[i]);
      const float b = ok ? __ldg(p.b_enc + cz + i) : 0.f;
      const float th = (ok && p.theta != nullptr) ? __ldg(p.theta + cz + i) : 0.f;
      const float pre = zr + b;
      const float f = (ok && pre > th && pre > 0.f) ? pre : 0.f;
      v[i] = zr;
      feat[i] = f;
      if (ok) {
        st.s_pre += fmaxf(-pre, 0.f);
        if (p.dec_norm != nullptr) {
          const float w = f * __ldg(p.dec_norm + cz + i) * p.c_sparsity;
          st.s_sp += p.use_tanh ? tanhf(w) : w;
        }
      }
    }
    if (p.fired != nullptr) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const unsigned any = __ballot_sync(0xffffffffu, feat[i] > 0.f);
        if (lane == i && any != 0u && n0 + i < N) p.fired[cz + i] = 1;
      }
    }
    if (!row_ok) return;
    const size_t off = ((size_t)z * M + row) * N + n0;
    const bool vec = can_vec<T>(n0, N);
    store32<T>(p.z_out + off, N - n0, vec, v);
    store32<T>(p.feat_out + off, N - n0, vec, feat);
  }
  __device__ static void finish(const Params& p, State& st) {
    const float a = warp_sum(st.s_pre), b = warp_sum(st.s_sp);
    if ((threadIdx.x & 31) == 0) {
      if (a != 0.f) atomicAdd(p.loss_acc + 0, a);
      if (b != 0.f) atomicAdd(p.loss_acc + 1, b);
    }
  }
};

// =====================================================================================
// Feature gradient with the (Jump)ReLU backward fused
// =====================================================================================
// acc = dL/dfeat from the decoder.  With pre = z + b recomputed from the stored z:
//   gs      = acc + lam * (1 - tanh^2(w)) * n * c          w = feat * n * c   (sparsity term)
//   dtheta += -(theta/bw) * rect((pre - theta)/bw) * gs     rect(u) = [u > -1/2] - [u > 1/2]
//   dpre    = gs * [pre >= 0]  -  pal * [pre < 0]           (JumpReLU passes 0 <= pre <= theta)
//           = gs * [pre >  0]  -  pal * [pre < 0]           (plain ReLU)
//   dnorm  += lam * (1 - tanh^2(w)) * feat * c
//   db_enc += dpre
// dpre is stored rounded to T (the operand type of the encoder weight-gradient contraction).
template <class T>
struct DFeatJumpReLU {
  struct Params {
    const T* z_in;          // [nz, M, N]
    const float* b_enc;     // [nz, N]
    const float* theta;     // [nz, N] or null (plain ReLU)
    const float* dec_norm;  // [nz, N] or null
    T* dpre_out;            // [nz, M, N]
    float* dtheta;          // [nz, N] or null
    float* dbenc;           // [nz, N]
    float* dnorm;           // [nz, N] or null
    float bandwidth;
    float lam;  // lambda / B
    float c_sparsity;
    float pal;  // pre_actv_loss / (B * L)
    int use_tanh;
    const float* gscale;  // device scalar: gradient of the loss w.r.t. itself (null = 1)
  };
  struct State {};
  __device__ static void init(State&) {}
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32]) {
    const size_t cz = (size_t)z * N + n0;
    const size_t off = ((size_t)z * M + (row_ok ? row : 0)) * N + n0;
    const bool vec = can_vec<T>(n0, N);
    float zv[32];
    load32<T>(p.z_in + off, row_ok ? N - n0 : 0, vec && row_ok, zv);
    float dth[32], dnr[32];
    const bool relu = p.theta == nullptr;
    const bool sp = p.dec_norm != nullptr;
    const float gsc = p.gscale != nullptr ? __ldg(p.gscale) : 1.f;
    const float lam = p.lam * gsc, pal = p.pal * gsc;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const bool ok = row_ok && (n0 + i < N);
      const float b = ok ? __ldg(p.b_enc + cz + i) : 0.f;
      const float th = (ok && !relu) ? __ldg(p.theta + cz + i) : 0.f;
      const float pre = zv[i] + b;
      const float f = (pre > th && pre > 0.f) ? pre : 0.f;
      float gs = v[i];
      float dn = 0.f;
      if (sp) {
        const float n = ok ? __ldg(p.dec_norm + cz + i) : 0.f;
        const float w = f * n * p.c_sparsity;
        float d1 = 1.f;
        if (p.use_tanh) {
          const float tw = tanhf(w);
          d1 = 1.f - tw * tw;
        }
        gs += lam * d1 * n * p.c_sparsity;
        dn = lam * d1 * f * p.c_sparsity;
      }
      const float u = (pre - th) / p.bandwidth;
      const float rect = ((u + 0.5f > 0.f) ? 1.f : 0.f) - ((u - 0.5f > 0.f) ? 1.f : 0.f);
      const bool pass = relu ? (pre > 0.f) : !(pre < 0.f);
      float dp = pass ? gs : 0.f;
      if (pre < 0.f) dp -= pal;
      dp = ok ? dp : 0.f;
      dth[i] = ok ? -(th / p.bandwidth) * rect * gs : 0.f;
      dnr[i] = ok ? dn : 0.f;
      v[i] = dp;
    }
    if (row_ok) store32<T>(p.dpre_out + off, N - n0, vec, v);
    col_atomic_add(p.dbenc + (size_t)z * N, n0, N, warp_colsum32(v));
    if (p.dtheta != nullptr) col_atomic_add(p.dtheta + (size_t)z * N, n0, N, warp_colsum32(dth));
    if (p.dnorm != nullptr) col_atomic_add(p.dnorm + (size_t)z * N, n0, N, warp_colsum32(dnr));
  }
  __device__ static void finish(const Params&, State&) {}
};

}  // namespace epi
}  // namespace clt
