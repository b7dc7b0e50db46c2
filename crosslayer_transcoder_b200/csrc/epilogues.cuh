// Epilogue functors of the contraction kernels.
//
// Both contraction kernels (fp32 SIMT, bf16 tcgen05) hand their accumulators to
// the epilogue in the same shape: a warp holds 32 consecutive rows of the output
// tile, each lane one row, and passes 32 consecutive columns of that row at a
// time.  Column reductions over the batch axis are therefore warp shuffles.
//
// Per-column parameters (biases, thresholds, norms) are staged by the kernel in
// shared memory once per tile and read by every row as broadcasts.
//
//   struct Epi {
//     struct Params;                      // pointers and scalars, passed by value
//     struct State;                       // per-thread registers living for the whole kernel
//     static constexpr int kColArrays;    // per-column parameter arrays to stage
//     static constexpr bool kPrefetch;    // registers allow reading the next accumulator chunk early
//     static float col_value(const Params&, int arr, int z, int n, int N);   // array arr at column n < N
//     static void init(State&);
//     template <int CS>                   // CS = stride between staged arrays (columns per tile)
//     static void apply(const Params&, State&, int z, int row, bool row_ok, int n0, int M, int N,
//                       float (&v)[32], const float* colp,    // colp[arr * CS + i], i = 0..31
//                       unsigned char* stage);                // per-warp staging buffer (kStageBytes)
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

// tanh at the accuracy the activation type needs: the exact routine beside fp32 activations, the
// hardware approximation (relative error about 2^-11, below the 2^-9 rounding step of bf16) beside bf16
// ones, where the routine's instruction count would otherwise outweigh the rest of the epilogue.
template <class T>
__device__ __forceinline__ float tanh_as(float x) { return tanhf(x); }
template <>
__device__ __forceinline__ float tanh_as<__nv_bfloat16>(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <class T>
__device__ __forceinline__ bool can_vec(int n0, int N) {
  return (n0 + 32 <= N) && (N % (16 / (int)sizeof(T)) == 0);
}

// ---- coalesced store of a warp's 32 x 32 sub-tile ------------------------------------------------
// Each lane holds one row (32 consecutive columns).  Writing that straight to global memory makes
// every store instruction touch 32 different rows, 16 bytes each.  Instead the sub-tile goes through
// a per-warp shared-memory buffer (kStageBytes, rows padded to 80 bytes: conflict-free 16-byte
// accesses) and is written out with 4 lanes per row segment, so an instruction covers 8 rows x 64
// contiguous bytes (full 32-byte sectors).  fp32 tiles go in two halves of 16 columns.
// `base` points at (first row of the warp, column n0); `rows_valid` rows of the 32 exist.
constexpr int kStageRow = 80;
constexpr int kStageBytes = 32 * kStageRow;

template <class T>
__device__ __forceinline__ void store_rows32(unsigned char* stage, T* base, size_t ld, int rows_valid,
                                             const float (&v)[32]);

template <>
__device__ __forceinline__ void store_rows32<__nv_bfloat16>(unsigned char* stage, __nv_bfloat16* base, size_t ld,
                                                            int rows_valid, const float (&v)[32]) {
  const int lane = threadIdx.x & 31;
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * kStageRow);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 t;
    t.x = pack_bf16x2(v[8 * i], v[8 * i + 1]);
    t.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
    t.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
    t.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
    mine[i] = t;
  }
  __syncwarp();
  const int piece = lane & 3;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 8 + (lane >> 2);
    const uint4 t = *reinterpret_cast<const uint4*>(stage + r * kStageRow + piece * 16);
    if (r < rows_valid) *reinterpret_cast<uint4*>(base + (size_t)r * ld + piece * 8) = t;
  }
  __syncwarp();
}

template <>
__device__ __forceinline__ void store_rows32<float>(unsigned char* stage, float* base, size_t ld, int rows_valid,
                                                    const float (&v)[32]) {
  const int lane = threadIdx.x & 31;
  float4* mine = reinterpret_cast<float4*>(stage + lane * kStageRow);
  const int piece = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      mine[i] = make_float4(v[16 * h + 4 * i], v[16 * h + 4 * i + 1], v[16 * h + 4 * i + 2], v[16 * h + 4 * i + 3]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = it * 8 + (lane >> 2);
      const float4 t = *reinterpret_cast<const float4*>(stage + r * kStageRow + piece * 16);
      if (r < rows_valid) *reinterpret_cast<float4*>(base + (size_t)r * ld + 16 * h + piece * 4) = t;
    }
    __syncwarp();
  }
}

// Store a warp's sub-tile: coalesced through `stage` when the 32 columns are all inside the matrix
// and rows are 16-byte aligned, else lane by lane with guards.  `row0` is the warp's first row.
template <class T>
__device__ __forceinline__ void store_tile(unsigned char* stage, T* mat, size_t ld, int row0, int row, bool row_ok,
                                           int M, int n0, int N, bool aligned, const float (&v)[32]) {
  if (aligned && n0 + 32 <= N) {
    store_rows32<T>(stage, mat + (size_t)row0 * ld + n0, ld, M - row0, v);
  } else if (row_ok) {
    store32<T>(mat + (size_t)row * ld + n0, N - n0, false, v);
  }
}

// Coalesced load of a warp's 32 x 32 sub-tile (the mirror image of store_rows32): 4 lanes fetch one
// row's 64-byte segment, the tile is parked in the staging buffer, every lane then reads its own row.
// Rows beyond rows_valid read as 0.
template <class T>
__device__ __forceinline__ void load_rows32(unsigned char* stage, const T* base, size_t ld, int rows_valid,
                                            float (&o)[32]);

template <>
__device__ __forceinline__ void load_rows32<__nv_bfloat16>(unsigned char* stage, const __nv_bfloat16* base, size_t ld,
                                                           int rows_valid, float (&o)[32]) {
  const int lane = threadIdx.x & 31;
  const int piece = lane & 3;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 8 + (lane >> 2);
    uint4 t = make_uint4(0, 0, 0, 0);
    if (r < rows_valid) t = *reinterpret_cast<const uint4*>(base + (size_t)r * ld + piece * 8);
    *reinterpret_cast<uint4*>(stage + r * kStageRow + piece * 16) = t;
  }
  __syncwarp();
  const uint4* mine = reinterpret_cast<const uint4*>(stage + lane * kStageRow);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 t = mine[i];
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
      o[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  __syncwarp();
}

template <>
__device__ __forceinline__ void load_rows32<float>(unsigned char* stage, const float* base, size_t ld, int rows_valid,
                                                   float (&o)[32]) {
  const int lane = threadIdx.x & 31;
  const int piece = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = it * 8 + (lane >> 2);
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < rows_valid) t = *reinterpret_cast<const float4*>(base + (size_t)r * ld + 16 * h + piece * 4);
      *reinterpret_cast<float4*>(stage + r * kStageRow + piece * 16) = t;
    }
    __syncwarp();
    const float4* mine = reinterpret_cast<const float4*>(stage + lane * kStageRow);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 t = mine[i];
      o[16 * h + 4 * i] = t.x, o[16 * h + 4 * i + 1] = t.y, o[16 * h + 4 * i + 2] = t.z, o[16 * h + 4 * i + 3] = t.w;
    }
    __syncwarp();
  }
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
  static constexpr int kColArrays = 0;
  static constexpr bool kPrefetch = true;
  __device__ static float col_value(const Params&, int, int, int, int) { return 0.f; }
  __device__ static void init(State&) {}
  template <int CS>
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float*, unsigned char* stage) {
    const int row0 = row - (threadIdx.x & 31);
    store_tile<T>(stage, p.out + (size_t)z * M * N, (size_t)N, row0, row, row_ok, M, n0, N,
                  N % (16 / (int)sizeof(T)) == 0, v);
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
  static constexpr int kColArrays = 1;
  static constexpr bool kPrefetch = true;
  __device__ static float col_value(const Params& p, int, int z, int n, int N) {
    return p.bias != nullptr ? __ldg(p.bias + (size_t)z * N + n) : 0.f;
  }
  __device__ static void init(State&) {}
  template <int CS>
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float* colp, unsigned char* stage) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += colp[i];
    const int row0 = row - (threadIdx.x & 31);
    store_tile<float>(stage, p.out + (size_t)z * p.zstride, (size_t)p.ld, row0, row, row_ok, M, n0, N,
                      (p.ld % 4 == 0) && (p.zstride % 4 == 0), v);
  }
  __device__ static void finish(const Params&, State&) {}
};

// Decoder forward with the exchange over feature-shard ranks fused in.  The token axis is split over
// the ranks (rank o owns rows [o * rows_per_rank, (o+1) * rows_per_rank) and holds, in a buffer every
// rank has mapped, one slot per source rank: [n_ranks, rows_per_rank, nz, N] fp32); acc + bias is STORED
// into this rank's slot of the owner's buffer (16-byte stores, over NVLink for the peers' buffers),
// tile by tile while the main loop of the next tile runs; the owner adds the slots afterwards.
// Sub-tiles go through the staging buffer so that an instruction covers 8 rows x 64 contiguous bytes.
constexpr int kMaxPushRanks = 16;
struct DecOutPush {
  struct Params {
    unsigned long long bases[kMaxPushRanks];  // address of each rank's buffer
    const float* bias;                        // [nz, N] or null
    int rows_per_rank;
    long long ld, zstride;                    // row and slab strides inside a slot
    long long slot_offset;                    // this rank's slot, in elements
    int slot_bf16;                            // slots hold bf16 partial sums (half the bytes over NVLink)
  };
  struct State {};
  static constexpr int kColArrays = 1;
  static constexpr bool kPrefetch = true;
  __device__ static float col_value(const Params& p, int, int z, int n, int N) {
    return p.bias != nullptr ? __ldg(p.bias + (size_t)z * N + n) : 0.f;
  }
  __device__ static void init(State&) {}
  // element offset of (row, slab z) inside the owner's buffer, and the owner's base address
  __device__ static __forceinline__ size_t row_off(const Params& p, int row, int z, unsigned long long& base) {
    const int o = row / p.rows_per_rank;
    base = p.bases[o];
    return (size_t)p.slot_offset + (size_t)(row - o * p.rows_per_rank) * p.ld + (size_t)z * p.zstride;
  }
  __device__ static __forceinline__ float* row_ptr(const Params& p, int row, int z) {
    unsigned long long base;
    const size_t off = row_off(p, row, z, base);
    return reinterpret_cast<float*>(base) + off;
  }
  __device__ static __forceinline__ __nv_bfloat16* row_ptr_bf16(const Params& p, int row, int z) {
    unsigned long long base;
    const size_t off = row_off(p, row, z, base);
    return reinterpret_cast<__nv_bfloat16*>(base) + off;
  }
  template <int CS>
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float* colp, unsigned char* stage) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += colp[i];
    const int lane = threadIdx.x & 31;
    const int row0 = row - lane;
    if (p.slot_bf16) {
      if (n0 + 32 <= N && p.ld % 8 == 0 && p.zstride % 8 == 0 && N % 8 == 0) {
        // 32 values of a row = 64 bytes of bf16: one pass through the staging buffer, 8 rows x 64 bytes per store
        uint4* mine = reinterpret_cast<uint4*>(stage + lane * kStageRow);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 t;
          t.x = pack_bf16x2(v[8 * i], v[8 * i + 1]), t.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
          t.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), t.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
          mine[i] = t;
        }
        __syncwarp();
        const int piece = lane & 3;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + (lane >> 2);
          const uint4 t = *reinterpret_cast<const uint4*>(stage + r * kStageRow + piece * 16);
          if (row0 + r < M) *reinterpret_cast<uint4*>(row_ptr_bf16(p, row0 + r, z) + n0 + piece * 8) = t;
        }
        __syncwarp();
      } else if (row_ok) {
        __nv_bfloat16* o = row_ptr_bf16(p, row, z) + n0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (n0 + i < N) o[i] = __float2bfloat16_rn(v[i]);
      }
      return;
    }
    if (n0 + 32 <= N && p.ld % 4 == 0 && p.zstride % 4 == 0 && N % 4 == 0) {
      float4* mine = reinterpret_cast<float4*>(stage + lane * kStageRow);
      const int piece = lane & 3;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          mine[i] = make_float4(v[16 * h + 4 * i], v[16 * h + 4 * i + 1], v[16 * h + 4 * i + 2], v[16 * h + 4 * i + 3]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + (lane >> 2);
          const float4 t = *reinterpret_cast<const float4*>(stage + r * kStageRow + piece * 16);
          if (row0 + r < M) *reinterpret_cast<float4*>(row_ptr(p, row0 + r, z) + n0 + 16 * h + piece * 4) = t;
        }
        __syncwarp();
      }
    } else if (row_ok) {
      float* o = row_ptr(p, row, z) + n0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n0 + i < N) o[i] = v[i];
    }
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
  static constexpr int kColArrays = 0;
  static constexpr bool kPrefetch = true;
  __device__ static float col_value(const Params&, int, int, int, int) { return 0.f; }
  __device__ static void init(State&) {}
  template <int CS>
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float*, unsigned char* stage) {
    const size_t off = ((size_t)z * M + (row_ok ? row : 0)) * N + n0;
    const bool vec = can_vec<float>(n0, N);
    if (p.rowcoef != nullptr && row_ok) {
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
    const int row0 = row - (threadIdx.x & 31);
    store_tile<float>(stage, p.out + (size_t)z * M * N, (size_t)N, row0, row, row_ok, M, n0, N, N % 4 == 0, v);
  }
  __device__ static void finish(const Params&, State&) {}
};

// =====================================================================================
// Encoder forward with the (Jump)ReLU fused
// =====================================================================================
// acc -> z = round_T(acc); pre = z + b; feat = pre * [pre > theta and pre > 0].
// Stores z and feat, marks (one bit per column) the columns that fired, and
// accumulates the two scalar loss terms that depend on every pre-activation:
//   sum relu(-pre)                       (pre-activation loss; skipped when want_pre == 0)
//   sum tanh(feat * dec_norm * c)        (sparsity penalty; without tanh: the product itself)
// Staged columns: 0 = b, 1 = theta (0 for ReLU), 2 = dec_norm * c.
template <class T>
struct EncJumpReLU {
  struct Params {
    const float* b_enc;     // [nz, N]
    const float* theta;     // [nz, N] or null (plain ReLU)
    const float* dec_norm;  // [nz, N] or null (no sparsity term)
    T* z_out;               // [nz, M, N]
    T* feat_out;            // [nz, M, N]
    unsigned* fired_bits;   // [nz, ceil(N/32)] packed flags, or null
    float* loss_acc;        // [0] += sum relu(-pre), [1] += sum of the sparsity summand
    float c_sparsity;
    int use_tanh;
    int want_pre;           // accumulate sum relu(-pre)
  };
  struct State {
    float s_pre, s_sp;
  };
  static constexpr int kColArrays = 3;
  static constexpr bool kPrefetch = false;
  __device__ static float col_value(const Params& p, int arr, int z, int n, int N) {
    const size_t i = (size_t)z * N + n;
    if (arr == 0) return __ldg(p.b_enc + i);
    if (arr == 1) return p.theta != nullptr ? __ldg(p.theta + i) : 0.f;
    return p.dec_norm != nullptr ? __ldg(p.dec_norm + i) * p.c_sparsity : 0.f;
  }
  __device__ static void init(State& s) { s.s_pre = 0.f, s.s_sp = 0.f; }
  // The element loop, specialised on the launch-constant options so that it carries no branches:
  // kPre (pre-activation sum wanted), kSp (sparsity sum wanted), kEdge (tile edge: per-element guards).
  template <int CS, bool kPre, bool kSp, bool kEdge>
  __device__ static __forceinline__ void body(const Params& p, State& st, bool row_ok, int n0, int N, float (&v)[32],
                                              float (&feat)[32], unsigned& mask, const float* colp) {
    float s_pre = 0.f, s_sp = 0.f;
#pragma unroll
    for (int i4 = 0; i4 < 8; ++i4) {
      const float4 b4 = *reinterpret_cast<const float4*>(colp + 4 * i4);
      const float4 t4 = *reinterpret_cast<const float4*>(colp + CS + 4 * i4);
      const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, tt[4] = {t4.x, t4.y, t4.z, t4.w};
      float nn[4] = {0.f, 0.f, 0.f, 0.f};
      if (kSp) {
        const float4 n4 = *reinterpret_cast<const float4*>(colp + 2 * CS + 4 * i4);
        nn[0] = n4.x, nn[1] = n4.y, nn[2] = n4.z, nn[3] = n4.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * i4 + j;
        const float zr = round_to<T>(v[i]);
        const float pre = zr + bb[j];
        float f = (pre > tt[j] && pre > 0.f) ? pre : 0.f;
        bool ok = true;
        if (kEdge) {
          ok = row_ok && (n0 + i < N);
          f = ok ? f : 0.f;
        }
        v[i] = zr;
        feat[i] = f;
        mask |= (f > 0.f) ? (1u << i) : 0u;
        if (kPre) s_pre += ok ? fmaxf(-pre, 0.f) : 0.f;
        if (kSp) {
          const float w = f * nn[j];
          s_sp += p.use_tanh ? tanh_as<T>(w) : w;
        }
      }
    }
    st.s_pre += s_pre, st.s_sp += s_sp;
  }

  template <int CS>
  __device__ static void apply(const Params& p, State& st, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float* colp, unsigned char* stage) {
    const bool edge = (n0 + 32 > N) || __any_sync(0xffffffffu, !row_ok);
    const bool sp = p.dec_norm != nullptr;
    float feat[32];
    unsigned mask = 0u;
    const int sel = (p.want_pre ? 1 : 0) | (sp ? 2 : 0) | (edge ? 4 : 0);
    switch (sel) {
      case 0: body<CS, false, false, false>(p, st, row_ok, n0, N, v, feat, mask, colp); break;
      case 1: body<CS, true, false, false>(p, st, row_ok, n0, N, v, feat, mask, colp); break;
      case 2: body<CS, false, true, false>(p, st, row_ok, n0, N, v, feat, mask, colp); break;
      case 3: body<CS, true, true, false>(p, st, row_ok, n0, N, v, feat, mask, colp); break;
      default: body<CS, true, true, true>(p, st, row_ok, n0, N, v, feat, mask, colp); break;
    }
    if (p.fired_bits != nullptr) {
      mask = __reduce_or_sync(0xffffffffu, mask);
      if ((threadIdx.x & 31) == 0 && mask != 0u) atomicOr(p.fired_bits + (size_t)z * ((N + 31) / 32) + n0 / 32, mask);
    }
    const int row0 = row - (threadIdx.x & 31);
    const bool al = N % (16 / (int)sizeof(T)) == 0;
    store_tile<T>(stage, p.z_out + (size_t)z * M * N, (size_t)N, row0, row, row_ok, M, n0, N, al, v);
    store_tile<T>(stage, p.feat_out + (size_t)z * M * N, (size_t)N, row0, row, row_ok, M, n0, N, al, feat);
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
// Staged columns: 0 = b, 1 = theta (0 for ReLU), 2 = dec_norm * c.
// rect is evaluated as -bw/2 < pre - theta <= bw/2, the same set without the division.
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
  static constexpr int kColArrays = 3;
  static constexpr bool kPrefetch = false;
  __device__ static float col_value(const Params& p, int arr, int z, int n, int N) {
    const size_t i = (size_t)z * N + n;
    if (arr == 0) return __ldg(p.b_enc + i);
    if (arr == 1) return p.theta != nullptr ? __ldg(p.theta + i) : 0.f;
    return p.dec_norm != nullptr ? __ldg(p.dec_norm + i) * p.c_sparsity : 0.f;
  }
  __device__ static void init(State&) {}
  template <int CS>
  __device__ static void apply(const Params& p, State&, int z, int row, bool row_ok, int n0, int M, int N,
                               float (&v)[32], const float* colp, unsigned char* stage) {
    const bool edge = (n0 + 32 > N) || __any_sync(0xffffffffu, !row_ok);
    const bool al = N % (16 / (int)sizeof(T)) == 0;
    const int row0 = row - (threadIdx.x & 31);
    float zv[32];
    if (al && n0 + 32 <= N) {
      load_rows32<T>(stage, p.z_in + ((size_t)z * M + row0) * N + n0, (size_t)N, M - row0, zv);
    } else {
      const size_t off = ((size_t)z * M + (row_ok ? row : 0)) * N + n0;
      load32<T>(p.z_in + off, row_ok ? N - n0 : 0, false, zv);
    }
    float dth[32], dnr[32];
    const bool sp = p.dec_norm != nullptr;
    if (sp) {
      if (edge) body<CS, true, true>(p, row_ok, n0, N, v, zv, dth, dnr, colp);
      else body<CS, true, false>(p, row_ok, n0, N, v, zv, dth, dnr, colp);
    } else {
      if (edge) body<CS, false, true>(p, row_ok, n0, N, v, zv, dth, dnr, colp);
      else body<CS, false, false>(p, row_ok, n0, N, v, zv, dth, dnr, colp);
    }
    store_tile<T>(stage, p.dpre_out + (size_t)z * M * N, (size_t)N, row0, row, row_ok, M, n0, N, al, v);
    col_atomic_add(p.dbenc + (size_t)z * N, n0, N, warp_colsum32(v));
    if (p.dtheta != nullptr) col_atomic_add(p.dtheta + (size_t)z * N, n0, N, warp_colsum32(dth));
    if (sp && p.dnorm != nullptr) col_atomic_add(p.dnorm + (size_t)z * N, n0, N, warp_colsum32(dnr));
  }

  // The element loop, specialised on kSp (sparsity gradient present) and kEdge (tile edge guards).
  template <int CS, bool kSp, bool kEdge>
  __device__ static __forceinline__ void body(const Params& p, bool row_ok, int n0, int N, float (&v)[32],
                                              const float (&zv)[32], float (&dth)[32], float (&dnr)[32],
                                              const float* colp) {
    const bool relu = p.theta == nullptr;
    const float gsc = p.gscale != nullptr ? __ldg(p.gscale) : 1.f;
    const float lam = p.lam * gsc, pal = p.pal * gsc;
    const float hb = 0.5f * p.bandwidth, ninv_bw = -1.f / p.bandwidth;
    // JumpReLU passes the gradient for pre >= 0, plain ReLU for pre > 0
    const float pass_lim = relu ? 0.f : -1.0e-45f;
#pragma unroll
    for (int i4 = 0; i4 < 8; ++i4) {
      const float4 b4 = *reinterpret_cast<const float4*>(colp + 4 * i4);
      const float4 t4 = *reinterpret_cast<const float4*>(colp + CS + 4 * i4);
      const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, tt[4] = {t4.x, t4.y, t4.z, t4.w};
      float nn[4] = {0.f, 0.f, 0.f, 0.f};
      if (kSp) {
        const float4 n4 = *reinterpret_cast<const float4*>(colp + 2 * CS + 4 * i4);
        nn[0] = n4.x, nn[1] = n4.y, nn[2] = n4.z, nn[3] = n4.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * i4 + j;
        const float th = tt[j];
        const float pre = zv[i] + bb[j];
        float gs = v[i];
        float dn = 0.f;
        if (kSp) {
          const float f = (pre > th && pre > 0.f) ? pre : 0.f;
          const float nc = nn[j];
          float d1 = 1.f;
          if (p.use_tanh) {
            const float tw = tanh_as<T>(f * nc);
            d1 = 1.f - tw * tw;
          }
          gs = fmaf(lam * d1, nc, gs);
          dn = lam * d1 * f * p.c_sparsity;
        }
        const float d = pre - th;
        const bool rect = (d > -hb) && !(d > hb);
        float dp = (pre > pass_lim) ? gs : 0.f;
        dp = (pre < 0.f) ? dp - pal : dp;
        float dt = rect ? (th * ninv_bw) * gs : 0.f;
        if (kEdge) {
          const bool ok = row_ok && (n0 + i < N);
          dp = ok ? dp : 0.f;
          dt = ok ? dt : 0.f;
          dn = ok ? dn : 0.f;
        }
        v[i] = dp;
        dth[i] = dt;
        if (kSp) dnr[i] = dn;
      }
    }
  }
  __device__ static void finish(const Params&, State&) {}
};

}  // namespace epi
}  // namespace clt
