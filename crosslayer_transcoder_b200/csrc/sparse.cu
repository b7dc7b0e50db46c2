// Sparse half of the TopK training step (HBM / L2 bound, no tensor cores).
//
// The selection leaves k (index, value) pairs per (layer, token) row.  The decoder
// forward gathers decoder rows token by token; the backward works feature by feature
// from a transposed (feature-major) copy of the selection so that every decoder row is
// read once, every gradient row is written once and no pre-zeroing or atomics on the
// large gradient buffers are needed.
//
// Layouts: idx / val / dval [L, B, k];  col_ptr [L, F+1];  ent [L, B*k] (slot = b*k + j);
//          W_dec flat [P, F, D];  recon [B, L, D];  drecon, xn [L, B, D].
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "gemm.cuh"
#include "kernels.h"

namespace clt {
namespace {

// ---- 8-wide row chunks ------------------------------------------------------------------
// load_raw keeps a chunk in its storage format (4 registers for bf16); unpack widens it to fp32
// at the point of use, which keeps rows that are in flight cheap in registers.
template <class T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  struct Raw {
    uint4 v;
  };
  __device__ static __forceinline__ Raw load_raw(const __nv_bfloat16* p) {
    Raw r;
    r.v = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
  }
  __device__ static __forceinline__ Raw zero() {
    Raw r;
    r.v = make_uint4(0, 0, 0, 0);
    return r;
  }
  __device__ static __forceinline__ void unpack(const Raw& r, float (&o)[8]) {
    const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = __uint_as_float(w[j] << 16);
      o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) { unpack(load_raw(p), o); }
};
template <>
struct Vec8<float> {
  struct Raw {
    float4 a, b;
  };
  __device__ static __forceinline__ Raw load_raw(const float* p) {
    Raw r;
    r.a = __ldg(reinterpret_cast<const float4*>(p));
    r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    return r;
  }
  __device__ static __forceinline__ Raw zero() {
    Raw r;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
    return r;
  }
  __device__ static __forceinline__ void unpack(const Raw& r, float (&o)[8]) {
    o[0] = r.a.x, o[1] = r.a.y, o[2] = r.a.z, o[3] = r.a.w, o[4] = r.b.x, o[5] = r.b.y, o[6] = r.b.z, o[7] = r.b.w;
  }
  __device__ static __forceinline__ void load(const float* p, float (&o)[8]) { unpack(load_raw(p), o); }
};

// Where a reconstruction row goes.  On one GPU, or when the partial reconstructions are summed by a
// library collective afterwards, the row is stored to `recon` [B, L, D].  With the exchange fused
// into this kernel the token axis is split over the ranks: rank o owns tokens
// [o * rows_per_rank, (o+1) * rows_per_rank) and holds, in a buffer that every rank has mapped, one
// slot per source rank: [n_ranks, rows_per_rank, L, D].  Every rank STORES its partial row into its
// own slot of the owner's buffer (16-byte stores, over NVLink for the peers' buffers), so that the
// transfer overlaps the gather row by row; the owner adds the slots from its local memory afterwards
// (clt_sum_slots).  Plain stores, because 16-byte reductions over NVLink ran at a third of the
// stores' rate.
constexpr int kMaxPushRanks = 16;
struct PushDst {
  unsigned long long bases[kMaxPushRanks];  // address of each rank's buffer
  int rows_per_rank;                        // 0 = plain store to `recon`
  long long slot_offset;                    // this rank's slot: slot * rows_per_rank * L * D elements
  int slot_bf16;                            // slots hold bf16 partial sums (half the bytes over NVLink)
};

__device__ __forceinline__ float* push_row(const PushDst& p, float* recon, int b, int t, int L, int D) {
  if (p.rows_per_rank == 0) return recon + ((size_t)b * L + t) * D;
  const int o = b / p.rows_per_rank;
  return reinterpret_cast<float*>(p.bases[o]) + p.slot_offset + ((size_t)(b - o * p.rows_per_rank) * L + t) * D;
}
__device__ __forceinline__ __nv_bfloat16* push_row_bf16(const PushDst& p, int b, int t, int L, int D) {
  const int o = b / p.rows_per_rank;
  return reinterpret_cast<__nv_bfloat16*>(p.bases[o]) + p.slot_offset +
         ((size_t)(b - o * p.rows_per_rank) * L + t) * D;
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* o, const float (&v)[8]) {
  uint4 t;
  t.x = pack_bf16x2(v[0], v[1]), t.y = pack_bf16x2(v[2], v[3]);
  t.z = pack_bf16x2(v[4], v[5]), t.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(o) = t;
}

// =========================================================================================
// Decoder forward, token-major gather.  One CTA per (token b, target layer t):
//   recon[b, t, :] = b_dec[t] + sum_{s <= t} sum_j val[s,b,j] * W[pair(t,s), idx[s,b,j], :]
// Each of the 4 warps takes every 4th selected row; lanes hold D/8/32 chunks of 8 columns.
// =========================================================================================
template <class T, int VPL>
__global__ void __launch_bounds__(128)
sparse_dec_fwd_kernel(const int* __restrict__ idx, const float* __restrict__ val, const int* __restrict__ row_start,
                      const int* __restrict__ row_cnt, long long npl, const T* __restrict__ W,
                      const float* __restrict__ b_dec, float* __restrict__ recon, int B, int L, int D, int F, int k,
                      int crosslayer, int* status, PushDst push) {
  extern __shared__ float red[];  // [4][D]
  const int b = blockIdx.x, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D / 8;
  float acc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  const int s_lo = crosslayer ? 0 : t;
  for (int s = s_lo; s <= t; ++s) {
    const size_t p = crosslayer ? (size_t)pair_index(t, s) : (size_t)t;
    // the row's entries: k fixed slots (valid ones first), or a (start, count) segment of the layer's list
    size_t e0 = ((size_t)s * B + b) * k;
    int n = k;
    if (row_start != nullptr) {
      e0 = (size_t)s * npl + __ldg(row_start + (size_t)s * B + b);
      n = __ldg(row_cnt + (size_t)s * B + b);
    }
    for (int j = warp; j < n; j += 4) {
      const float v = __ldg(val + e0 + j);
      if (v == 0.f) break;  // valid slots come first
      const int f = __ldg(idx + e0 + j);
      if (f < 0 || f >= F) {
        report_status(status, kBadIndex);
        continue;
      }
      const T* row = W + (p * F + f) * D;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
          float w[8];
          Vec8<T>::load(row + 8 * c, w);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][q] = fmaf(v, w[q], acc[i][q]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
#pragma unroll
      for (int q = 0; q < 8; ++q) red[warp * D + 8 * c + q] = acc[i][q];
    }
  }
  __syncthreads();
  if (push.rows_per_rank != 0 && push.slot_bf16) {  // bf16 slots: 8 columns = one 16-byte store (D % 8 == 0)
    __nv_bfloat16* ob = push_row_bf16(push, b, t, L, D);
    for (int d = 8 * threadIdx.x; d < D; d += 8 * 128) {
      float sum[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        sum[q] = red[d + q] + red[D + d + q] + red[2 * D + d + q] + red[3 * D + d + q];
        if (b_dec != nullptr) sum[q] += __ldg(b_dec + (size_t)t * D + d + q);
      }
      store8_bf16(ob + d, sum);
    }
    return;
  }
  float* out = push_row(push, recon, b, t, L, D);
  if (D % 4 == 0) {  // 16-byte stores (always the case for pushed rows: D % 8 == 0 there)
    for (int d = 4 * threadIdx.x; d < D; d += 4 * 128) {
      float4 sum;
      sum.x = red[d] + red[D + d] + red[2 * D + d] + red[3 * D + d];
      sum.y = red[d + 1] + red[D + d + 1] + red[2 * D + d + 1] + red[3 * D + d + 1];
      sum.z = red[d + 2] + red[D + d + 2] + red[2 * D + d + 2] + red[3 * D + d + 2];
      sum.w = red[d + 3] + red[D + d + 3] + red[2 * D + d + 3] + red[3 * D + d + 3];
      if (b_dec != nullptr) {
        const float4 bb = __ldg(reinterpret_cast<const float4*>(b_dec + (size_t)t * D + d));
        sum.x += bb.x, sum.y += bb.y, sum.z += bb.z, sum.w += bb.w;
      }
      *reinterpret_cast<float4*>(out + d) = sum;
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += 128) {
    float sum = red[d] + red[D + d] + red[2 * D + d] + red[3 * D + d];
    if (b_dec != nullptr) sum += __ldg(b_dec + (size_t)t * D + d);
    out[d] = sum;
  }
}

// Measured effects of order on this gather (12-layer, 32768-feature, k = 32 workload unless said otherwise):
// target layers in ascending order, tokens fastest (below) 1.99 ms, longest target layers first 2.26 ms; one
// warp per (token, layer) 1.99 ms, one CTA 2.34 ms (four times fewer tokens in flight per decoder block);
// entry lists in feature order or, for the short ragged lists of the batch-wide selection, in value order cost
// 10 % (16-layer BatchTopK workload: 3.6 ms against 3.2-3.3 ms in arrival or scrambled order).  Two variants of
// the warp form were measured and dropped: four rows in flight per warp instead of two (2.29 ms against
// 1.99 ms: fewer resident warps), and the columns of a wide row (D = 2048) split over two warps (4.6 ms against
// 3.3 ms: the halves of a decoder row are then fetched at different times).
//
// Same computation with one WARP per (token, target layer) and no shared-memory reduction: for
// short entry lists (a feature shard keeps only a few of a row's k slots) the per-CTA overhead of
// the kernel above dominates.  Entries are fetched 32 at a time, rows two at a time.
template <class T, int VPL>
__global__ void __launch_bounds__(128)
sparse_dec_fwd_warp_kernel(const int* __restrict__ idx, const float* __restrict__ val,
                           const int* __restrict__ row_start, const int* __restrict__ row_cnt, long long npl,
                           const T* __restrict__ W, const float* __restrict__ b_dec, float* __restrict__ recon, int B,
                           int L, int D, int F, int k, int crosslayer, int* status, PushDst push) {
  const long long pair = blockIdx.x * 4ll + (threadIdx.x >> 5);
  if (pair >= (long long)B * L) return;
  const int b = (int)(pair % B), t = (int)(pair / B);
  const int lane = threadIdx.x & 31;
  const int nvec = D / 8;
  using V = Vec8<T>;
  float acc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  const int s_lo = crosslayer ? 0 : t;
  for (int s = s_lo; s <= t; ++s) {
    const size_t p = crosslayer ? (size_t)pair_index(t, s) : (size_t)t;
    size_t e0 = ((size_t)s * B + b) * k;
    int n = k;
    if (row_start != nullptr) {
      e0 = (size_t)s * npl + __ldg(row_start + (size_t)s * B + b);
      n = __ldg(row_cnt + (size_t)s * B + b);
    }
    for (int j0 = 0; j0 < n; j0 += 32) {
      const int m = min(32, n - j0);
      float my_v = 0.f;
      int my_f = 0;
      if (lane < m) {
        my_v = __ldg(val + e0 + j0 + lane);
        my_f = __ldg(idx + e0 + j0 + lane);
      }
      const int valid = __popc(__ballot_sync(0xffffffffu, my_v != 0.f));  // valid slots come first
      if (my_v != 0.f && (my_f < 0 || my_f >= F)) {  // skip this entry only: it contributes 0 * row 0
        report_status(status, kBadIndex);
        my_v = 0.f, my_f = 0;
      }
      for (int j = 0; j < valid; j += 2) {
        const bool two = j + 1 < valid;
        const float v0 = __shfl_sync(0xffffffffu, my_v, j);
        const float v1 = two ? __shfl_sync(0xffffffffu, my_v, j + 1) : 0.f;
        const T* r0 = W + (p * F + __shfl_sync(0xffffffffu, my_f, j)) * D;
        const T* r1 = W + (p * F + __shfl_sync(0xffffffffu, my_f, two ? j + 1 : j)) * D;
        typename V::Raw x0[VPL], x1[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          const int c = lane + 32 * i;
          x0[i] = c < nvec ? V::load_raw(r0 + 8 * c) : V::zero();
          x1[i] = (two && c < nvec) ? V::load_raw(r1 + 8 * c) : V::zero();
        }
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          float w[8];
          V::unpack(x0[i], w);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][q] = fmaf(v0, w[q], acc[i][q]);
          V::unpack(x1[i], w);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][q] = fmaf(v1, w[q], acc[i][q]);
        }
      }
      if (valid < m) break;
    }
  }
  if (push.rows_per_rank != 0 && push.slot_bf16) {
    __nv_bfloat16* ob = push_row_bf16(push, b, t, L, D);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float bb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (b_dec != nullptr) Vec8<float>::load(b_dec + (size_t)t * D + 8 * c, bb);
        float o8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) o8[q] = acc[i][q] + bb[q];
        store8_bf16(ob + 8 * c, o8);
      }
    }
    return;
  }
  float* out = push_row(push, recon, b, t, L, D);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float bb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (b_dec != nullptr) Vec8<float>::load(b_dec + (size_t)t * D + 8 * c, bb);
      float4* o = reinterpret_cast<float4*>(out + 8 * c);
      const float4 lo = make_float4(acc[i][0] + bb[0], acc[i][1] + bb[1], acc[i][2] + bb[2], acc[i][3] + bb[3]);
      const float4 hi = make_float4(acc[i][4] + bb[4], acc[i][5] + bb[5], acc[i][6] + bb[6], acc[i][7] + bb[7]);
      o[0] = lo;
      o[1] = hi;
    }
  }
}

// =========================================================================================
// Feature-major copy of the selection (counting sort per layer).
// =========================================================================================
// Scratch of the allocation-free variant of the counting sort (clt_csc_build_static): the
// per-feature write cursors.  It lives in the library image, so every GPU that loads the
// library holds these 4 MiB until the process exits.
constexpr long long kStaticCursorCap = 1ll << 20;  // layers x features this rank may hold
static __device__ __align__(256) int g_static_cursor[kStaticCursorCap];

__global__ void csc_count_kernel(const int* __restrict__ idx, const float* __restrict__ val, int* __restrict__ count,
                                 long long n_per_layer, int F, int L, int* status) {
  const long long total = n_per_layer * L;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    if (val[i] == 0.f) continue;
    const int l = (int)(i / n_per_layer);
    const int f = idx[i];
    if (f < 0 || f >= F) {
      report_status(status, kBadIndex);
      continue;
    }
    atomicAdd(count + (size_t)l * (F + 1) + f, 1);
  }
}

// exclusive scan of count[l, 0..F) in place -> col_ptr[l, 0..F]; cursor[l, f] = col_ptr[l, f]
__global__ void csc_scan_kernel(int* __restrict__ col_ptr, int* __restrict__ cursor, int F) {
  const int l = blockIdx.x;
  int* cp = col_ptr + (size_t)l * (F + 1);
  int* cur = cursor + (size_t)l * F;
  __shared__ int wsum[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int f0 = 0; f0 < F; f0 += blockDim.x) {
    const int f = f0 + threadIdx.x;
    const int c = f < F ? cp[f] : 0;
    int x = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) wsum[w] = x;
    __syncthreads();
    int woff = 0;
    for (int j = 0; j < w; ++j) woff += wsum[j];
    const int excl = carry + woff + x - c;
    __syncthreads();
    if (f < F) cp[f] = excl, cur[f] = excl;
    if (threadIdx.x == blockDim.x - 1) carry = excl + c;
    __syncthreads();
  }
  if (threadIdx.x == 0) cp[F] = carry;
}

__global__ void csc_fill_kernel(const int* __restrict__ idx, const float* __restrict__ val, int* __restrict__ cursor,
                                int* __restrict__ ent, long long n_per_layer, int F, int L) {
  const long long total = n_per_layer * L;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    if (val[i] == 0.f) continue;
    const int l = (int)(i / n_per_layer);
    const int f = idx[i];
    if (f < 0 || f >= F) continue;
    const int pos = atomicAdd(cursor + (size_t)l * F + f, 1);
    ent[(size_t)l * n_per_layer + pos] = (int)(i - (long long)l * n_per_layer);
  }
}

// =========================================================================================
// Decoder backward, feature-major.  One warp per decoder row (block p = (target t, source s),
// feature f):   w = W[p, f, :]
//   for every token b that selected feature f of layer s:
//       dval[s,b,j] += w . drecon[t,b,:]            (one atomic per token and target)
//       g           += val[s,b,j] * drecon[t,b,:]
//   dW[p, f, :] = g                                 (zeros when nobody selected f)
// The reconstruction gradient (tens of MB) stays resident in L2; W is read once and dW
// written once.
// =========================================================================================
template <class T, int VPL>
__global__ void __launch_bounds__(128)
sparse_bwd_dec_kernel(const int* __restrict__ col_ptr, const int* __restrict__ ent, const float* __restrict__ val,
                      const int* __restrict__ etok, long long npl_, const T* __restrict__ W,
                      const T* __restrict__ drecon, float* __restrict__ dW, float* __restrict__ dval, int B, int L,
                      int D, int F, int k, int crosslayer, long long n_rows) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= n_rows) return;
  const int p = (int)(wid / F), f = (int)(wid % F);
  int s = p, t = p;
  if (crosslayer) pair_split(p, t, s);
  const int nvec = D / 8;
  const int* cp = col_ptr + (size_t)s * (F + 1);
  const int e0 = __ldg(cp + f), e1 = __ldg(cp + f + 1);
  const size_t npl = (size_t)npl_;
  const size_t roff = ((size_t)p * F + f) * D;
  using V = Vec8<T>;
  constexpr bool kTwo = VPL <= 4;  // two rows in flight while the register budget allows it
  typename V::Raw w[VPL];
  float g[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
#pragma unroll
    for (int q = 0; q < 8; ++q) g[i][q] = 0.f;
    w[i] = (e1 > e0 && c < nvec) ? V::load_raw(W + roff + 8 * c) : V::zero();
  }
  // entries in groups of 32: one coalesced load of the group's slots and values, then the rows
  // (two at a time where possible, so that two independent row fetches are in flight per warp)
  for (int eb = e0; eb < e1; eb += 32) {
    const int n = min(32, e1 - eb);
    int my_slot = 0, my_tok = 0;
    float my_val = 0.f;
    if (lane < n) {
      my_slot = __ldg(ent + (size_t)s * npl + eb + lane);
      my_val = __ldg(val + (size_t)s * npl + my_slot);
      my_tok = etok != nullptr ? __ldg(etok + (size_t)s * npl + my_slot) : my_slot / k;
    }
    for (int j = 0; j < n; j += (kTwo ? 2 : 1)) {
      const bool two = kTwo && (j + 1 < n);
      const int slot0 = __shfl_sync(0xffffffffu, my_slot, j);
      const int slot1 = __shfl_sync(0xffffffffu, my_slot, two ? j + 1 : j);
      const float v0 = __shfl_sync(0xffffffffu, my_val, j);
      const float v1 = two ? __shfl_sync(0xffffffffu, my_val, j + 1) : 0.f;
      const int tok0 = __shfl_sync(0xffffffffu, my_tok, j);
      const int tok1 = __shfl_sync(0xffffffffu, my_tok, two ? j + 1 : j);
      const T* dr0 = drecon + ((size_t)t * B + tok0) * D;
      const T* dr1 = drecon + ((size_t)t * B + tok1) * D;
      typename V::Raw x0[VPL], x1[kTwo ? VPL : 1];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        x0[i] = c < nvec ? V::load_raw(dr0 + 8 * c) : V::zero();
        if (kTwo) x1[i] = (two && c < nvec) ? V::load_raw(dr1 + 8 * c) : V::zero();
      }
      float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float wf[8], xf[8];
        V::unpack(w[i], wf);
        V::unpack(x0[i], xf);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          dot0 = fmaf(wf[q], xf[q], dot0);
          g[i][q] = fmaf(v0, xf[q], g[i][q]);
        }
        if (kTwo) {
          V::unpack(x1[i], xf);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            dot1 = fmaf(wf[q], xf[q], dot1);
            g[i][q] = fmaf(v1, xf[q], g[i][q]);
          }
        }
      }
      dot0 = warp_sum(dot0);
      if (kTwo) dot1 = warp_sum(dot1);
      if (lane == 0) {
        atomicAdd(dval + (size_t)s * npl + slot0, dot0);
        if (two) atomicAdd(dval + (size_t)s * npl + slot1, dot1);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float4* o = reinterpret_cast<float4*>(dW + roff + 8 * c);
      __stcs(o, make_float4(g[i][0], g[i][1], g[i][2], g[i][3]));
      __stcs(o + 1, make_float4(g[i][4], g[i][5], g[i][6], g[i][7]));
    }
  }
}

// Same computation with one warp per GROUP of 8 consecutive features of a block (needs F % 8 == 0).
// The features' entries are contiguous in the feature-major list, so the group needs one read of 9
// column pointers and coalesced reads of the entries' slots / values / tokens (32 at a time); the
// decoder row of the next non-empty feature is fetched while the current one is processed; rows of
// features nobody selected are zero-filled without touching W.  This removes most of the dependent
// round trips (pointer -> entry -> token -> row) that bound the one-row-per-warp kernel above.
template <class T, int VPL>
__global__ void __launch_bounds__(128, 5)
sparse_bwd_dec_group_kernel(const int* __restrict__ col_ptr, const int* __restrict__ ent,
                            const float* __restrict__ val, const int* __restrict__ etok, long long npl_,
                            const T* __restrict__ W, const T* __restrict__ drecon, float* __restrict__ dW,
                            float* __restrict__ dval, int B, int L, int D, int F, int k, int crosslayer,
                            long long n_groups) {
  const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gid >= n_groups) return;
  const int gpf = F / 8;
  const int p = (int)(gid / gpf), f0 = (int)(gid % gpf) * 8;
  int s = p, t = p;
  if (crosslayer) pair_split(p, t, s);
  const int nvec = D / 8;
  const size_t npl = (size_t)npl_;
  using V = Vec8<T>;
  const int cpv = lane < 9 ? __ldg(col_ptr + (size_t)s * (F + 1) + f0 + lane) : 0;
  const int cpn = __shfl_down_sync(0xffffffffu, cpv, 1);
  unsigned mask = __ballot_sync(0xffffffffu, lane < 8 && cpn > cpv) & 0xffu;   // features with entries
  const size_t row0 = ((size_t)p * F + f0) * D;
  // rows of features without entries are zero
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (!((mask >> j) & 1u)) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
          float4* o = reinterpret_cast<float4*>(dW + row0 + (size_t)j * D + 8 * c);
          __stcs(o, make_float4(0.f, 0.f, 0.f, 0.f));
          __stcs(o + 1, make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
    }
  }
  if (mask == 0u) return;
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
  load_chunk(base);
  int fi = __ffs(mask) - 1;
  typename V::Raw w_cur[VPL], w_next[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    w_cur[i] = c < nvec ? V::load_raw(W + row0 + (size_t)fi * D + 8 * c) : V::zero();
    w_next[i] = V::zero();
  }
  for (;;) {
    const unsigned rest = mask >> (fi + 1);
    const bool has_next = rest != 0u;
    const int fn = fi + __ffs(rest);   // index of the next feature with entries (valid when has_next)
    if (has_next) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) w_next[i] = V::load_raw(W + row0 + (size_t)fn * D + 8 * c);
      }
    }
    float g[VPL][8];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int q = 0; q < 8; ++q) g[i][q] = 0.f;
    const int eb = __shfl_sync(0xffffffffu, cpv, fi), ee = __shfl_sync(0xffffffffu, cpv, fi + 1);
    for (int e = eb; e < ee; e += 2) {
      const bool two = e + 1 < ee;
      if (e + 1 - base >= 32) {   // both entries of the pair must lie inside the loaded chunk
        base = e;
        load_chunk(base);
      }
      const int j0 = e - base, j1 = two ? j0 + 1 : j0;
      const int slot0 = __shfl_sync(0xffffffffu, my_slot, j0), slot1 = __shfl_sync(0xffffffffu, my_slot, j1);
      const float v0 = __shfl_sync(0xffffffffu, my_val, j0);
      const float v1 = two ? __shfl_sync(0xffffffffu, my_val, j1) : 0.f;
      const T* dr0 = drecon + ((size_t)t * B + __shfl_sync(0xffffffffu, my_tok, j0)) * D;
      const T* dr1 = drecon + ((size_t)t * B + __shfl_sync(0xffffffffu, my_tok, j1)) * D;
      typename V::Raw x0[VPL], x1[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        x0[i] = c < nvec ? V::load_raw(dr0 + 8 * c) : V::zero();
        x1[i] = (two && c < nvec) ? V::load_raw(dr1 + 8 * c) : V::zero();
      }
      float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float wf[8], xf[8];
        V::unpack(w_cur[i], wf);
        V::unpack(x0[i], xf);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          dot0 = fmaf(wf[q], xf[q], dot0);
          g[i][q] = fmaf(v0, xf[q], g[i][q]);
        }
        V::unpack(x1[i], xf);
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
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float4* o = reinterpret_cast<float4*>(dW + row0 + (size_t)fi * D + 8 * c);
        __stcs(o, make_float4(g[i][0], g[i][1], g[i][2], g[i][3]));
        __stcs(o + 1, make_float4(g[i][4], g[i][5], g[i][6], g[i][7]));
      }
    }
    if (!has_next) break;
    fi = fn;
#pragma unroll
    for (int i = 0; i < VPL; ++i) w_cur[i] = w_next[i];
  }
}

// =========================================================================================
// Encoder backward, feature-major.  One CTA per (layer l, 8 features, 768 input dims):
//   dW_enc[l, d, f] = sum over tokens b that selected f of dval[l,b,j] * xn[l,b,d]
//   db_enc[l, f]    = sum of the same dval
// Thread t owns dims d0 + t, d0 + t + 256, d0 + t + 512 and the 8 features of the block, so every
// store is a full 32-byte sector of the F-contiguous gradient; the small register footprint
// keeps many CTAs resident to hide the latency of the dependent entry -> row loads.
// =========================================================================================
constexpr int kEncFB = 8;

template <class T>
__global__ void __launch_bounds__(256)
sparse_bwd_enc_kernel(const int* __restrict__ col_ptr, const int* __restrict__ ent, const float* __restrict__ dval,
                      const int* __restrict__ etok, long long npl_, const T* __restrict__ xn, float* __restrict__ dW,
                      float* __restrict__ db, int B, int D, int F, int k, const float* __restrict__ dW_aux,
                      const float* __restrict__ db_aux, const int* __restrict__ dead_pos, int nd_pad) {
  const int l = blockIdx.y, f0 = blockIdx.x * kEncFB, d0 = blockIdx.z * 768;
  const int* cp = col_ptr + (size_t)l * (F + 1);
  const size_t npl = (size_t)npl_;
  // the block's entries (all 8 features' lists are contiguous): gradient and token, staged once
  constexpr int kCap = 512;
  __shared__ float s_g[kCap];
  __shared__ int s_tok[kCap];
  __shared__ int s_cp[kEncFB + 1];
  if (threadIdx.x <= kEncFB) s_cp[threadIdx.x] = __ldg(cp + min(f0 + (int)threadIdx.x, F));
  __syncthreads();
  const int e_begin = s_cp[0], e_end = s_cp[kEncFB];
  float acc[3][kEncFB];
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int q = 0; q < kEncFB; ++q) acc[i][q] = 0.f;
  float bsum = 0.f;
  const T* xl = xn + (size_t)l * B * D;
  for (int c0 = e_begin; c0 < e_end; c0 += kCap) {
    const int c1 = min(e_end, c0 + kCap);
    __syncthreads();
    for (int e = c0 + threadIdx.x; e < c1; e += 256) {
      const int slot = __ldg(ent + (size_t)l * npl + e);
      s_g[e - c0] = __ldg(dval + (size_t)l * npl + slot);
      s_tok[e - c0] = etok != nullptr ? __ldg(etok + (size_t)l * npl + slot) : slot / k;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kEncFB; ++q) {
      const int eb = max(s_cp[q], c0), ee = min(s_cp[q + 1], c1);
      float bs = 0.f;
      int e = eb;
      for (; e + 1 < ee; e += 2) {  // two rows of x in flight
        const float g0 = s_g[e - c0], g1 = s_g[e + 1 - c0];
        const T* x0 = xl + (size_t)s_tok[e - c0] * D;
        const T* x1 = xl + (size_t)s_tok[e + 1 - c0] * D;
        float a0[3], a1[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const int d = d0 + threadIdx.x + 256 * i;
          a0[i] = d < D ? ToFloat<T>::get(x0[d]) : 0.f;
          a1[i] = d < D ? ToFloat<T>::get(x1[d]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 3; ++i) acc[i][q] = fmaf(g1, a1[i], fmaf(g0, a0[i], acc[i][q]));
        bs += g0 + g1;
      }
      if (e < ee) {
        const float g0 = s_g[e - c0];
        const T* x0 = xl + (size_t)s_tok[e - c0] * D;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const int d = d0 + threadIdx.x + 256 * i;
          if (d < D) acc[i][q] = fmaf(g0, ToFloat<T>::get(x0[d]), acc[i][q]);
        }
        bs += g0;
      }
      if ((int)threadIdx.x == q) bsum += bs;
    }
  }
  // gradient of the auxiliary dead-feature loss (dense contraction over the compact dead features): added
  // here, so that no separate read-modify-write pass over the scattered columns is needed
  if (dW_aux != nullptr) {
#pragma unroll
    for (int q = 0; q < kEncFB; ++q) {
      const int pos = f0 + q < F ? __ldg(dead_pos + (size_t)l * F + f0 + q) : -1;   // CTA-uniform
      if (pos < 0) continue;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int d = d0 + threadIdx.x + 256 * i;
        if (d < D) acc[i][q] += __ldg(dW_aux + ((size_t)l * D + d) * nd_pad + pos);
      }
      if ((int)threadIdx.x == q) bsum += __ldg(db_aux + (size_t)l * nd_pad + pos);
    }
  }
  const bool vec = (F % 4 == 0) && (f0 + kEncFB <= F);
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int d = d0 + threadIdx.x + 256 * i;
    if (d >= D) continue;
    float* o = dW + ((size_t)l * D + d) * F + f0;
    if (vec) {
#pragma unroll
      for (int q = 0; q < kEncFB / 4; ++q)
        __stcs(reinterpret_cast<float4*>(o) + q,
               make_float4(acc[i][4 * q], acc[i][4 * q + 1], acc[i][4 * q + 2], acc[i][4 * q + 3]));
    } else {
#pragma unroll
      for (int q = 0; q < kEncFB; ++q)
        if (f0 + q < F) o[q] = acc[i][q];
    }
  }
  if (blockIdx.z == 0 && threadIdx.x < kEncFB && f0 + (int)threadIdx.x < F)
    db[(size_t)l * F + f0 + threadIdx.x] = bsum;
}

// =========================================================================================
// Compaction helpers of the auxiliary (dead-feature) path.
// =========================================================================================
// out[p, j, :] = W[p, dead_list[s(p)][j], :] for j < n_dead[s(p)], else 0
// Compact encoder operands of the dead features, for the auxiliary path's own small contraction:
//   Wc[l, d, j] = W_enc[l, d, dead_list[l][j]],  bc[l, j] = b_enc[l, dead_list[l][j]]     (j < n_dead[l])
// Padding columns (j >= n_dead[l]) get weight 0 and bias -1: their pre-activation is -1, never positive.
// The same computation with 16-byte loads: a thread owns 8 consecutive input dimensions (one 16-byte chunk of an
// x row) and all kEncFB features of the CTA, 128 threads cover 1024 dimensions (blockIdx.z takes the next 1024).
// An 8th of the load instructions of the kernel above for the same rows; needs D % 8 == 0.
template <class T>
__global__ void __launch_bounds__(128)
sparse_bwd_enc_vec_kernel(const int* __restrict__ col_ptr, const int* __restrict__ ent, const float* __restrict__ dval,
                          const int* __restrict__ etok, long long npl_, const T* __restrict__ xn,
                          float* __restrict__ dW, float* __restrict__ db, int B, int D, int F, int k,
                          const float* __restrict__ dW_aux, const float* __restrict__ db_aux,
                          const int* __restrict__ dead_pos, int nd_pad) {
  using V = Vec8<T>;
  const int l = blockIdx.y, f0 = blockIdx.x * kEncFB;
  const int d = (blockIdx.z * 128 + threadIdx.x) * 8;      // this thread's first input dimension
  const bool on = d < D;
  const int* cp = col_ptr + (size_t)l * (F + 1);
  const size_t npl = (size_t)npl_;
  constexpr int kCap = 512;
  __shared__ float s_g[kCap];
  __shared__ int s_tok[kCap];
  __shared__ int s_cp[kEncFB + 1];
  if (threadIdx.x <= kEncFB) s_cp[threadIdx.x] = __ldg(cp + min(f0 + (int)threadIdx.x, F));
  __syncthreads();
  const int e_begin = s_cp[0], e_end = s_cp[kEncFB];
  float acc[kEncFB][8];
#pragma unroll
  for (int q = 0; q < kEncFB; ++q)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[q][i] = 0.f;
  float bsum = 0.f;
  const T* xl = xn + (size_t)l * B * D + d;
  for (int c0 = e_begin; c0 < e_end; c0 += kCap) {
    const int c1 = min(e_end, c0 + kCap);
    __syncthreads();
    for (int e = c0 + threadIdx.x; e < c1; e += 128) {
      const int slot = __ldg(ent + (size_t)l * npl + e);
      s_g[e - c0] = __ldg(dval + (size_t)l * npl + slot);
      s_tok[e - c0] = etok != nullptr ? __ldg(etok + (size_t)l * npl + slot) : slot / k;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kEncFB; ++q) {
      const int eb = max(s_cp[q], c0), ee = min(s_cp[q + 1], c1);
      float bs = 0.f;
      for (int e = eb; e < ee; e += 2) {  // two rows of x in flight
        const bool two = e + 1 < ee;
        const float g0 = s_g[e - c0], g1 = two ? s_g[e + 1 - c0] : 0.f;
        typename V::Raw r0 = V::zero(), r1 = V::zero();
        if (on) {
          r0 = V::load_raw(xl + (size_t)s_tok[e - c0] * D);
          if (two) r1 = V::load_raw(xl + (size_t)s_tok[e + 1 - c0] * D);
        }
        float x0[8], x1[8];
        V::unpack(r0, x0);
        V::unpack(r1, x1);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[q][i] = fmaf(g1, x1[i], fmaf(g0, x0[i], acc[q][i]));
        bs += g0 + g1;
      }
      if ((int)threadIdx.x == q) bsum += bs;
    }
  }
  if (dW_aux != nullptr) {   // the auxiliary loss's compact gradient, for the dead features among these 8
#pragma unroll
    for (int q = 0; q < kEncFB; ++q) {
      const int pos = f0 + q < F ? __ldg(dead_pos + (size_t)l * F + f0 + q) : -1;   // CTA-uniform
      if (pos < 0) continue;
      if (on) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[q][i] += __ldg(dW_aux + ((size_t)l * D + d + i) * nd_pad + pos);
      }
      if ((int)threadIdx.x == q) bsum += __ldg(db_aux + (size_t)l * nd_pad + pos);
    }
  }
  if (on) {
    const bool vec = (F % 4 == 0) && (f0 + kEncFB <= F);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float* o = dW + ((size_t)l * D + d + i) * F + f0;
      if (vec) {
        __stcs(reinterpret_cast<float4*>(o), make_float4(acc[0][i], acc[1][i], acc[2][i], acc[3][i]));
        __stcs(reinterpret_cast<float4*>(o) + 1, make_float4(acc[4][i], acc[5][i], acc[6][i], acc[7][i]));
      } else {
#pragma unroll
        for (int q = 0; q < kEncFB; ++q)
          if (f0 + q < F) o[q] = acc[q][i];
      }
    }
  }
  if (blockIdx.z == 0 && threadIdx.x < kEncFB && f0 + (int)threadIdx.x < F)
    db[(size_t)l * F + f0 + threadIdx.x] = bsum;
}

template <class T>
__global__ void gather_enc_cols_kernel(const T* __restrict__ W, const float* __restrict__ b_enc,
                                       const int* __restrict__ dead_list, const int* __restrict__ n_dead,
                                       T* __restrict__ Wc, float* __restrict__ bc, int D, int F, int nd_pad) {
  const int l = blockIdx.z;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= nd_pad) return;
  const int f = j < n_dead[l] ? dead_list[(size_t)l * F + j] : -1;
  if (blockIdx.y == 0) bc[(size_t)l * nd_pad + j] = f >= 0 ? __ldg(b_enc + (size_t)l * F + f) : -1.f;
  for (int d = blockIdx.y; d < D; d += gridDim.y) {
    const size_t r = (size_t)l * D + d;
    T v;
    if (f >= 0) v = W[r * F + f];
    else if constexpr (sizeof(T) == 2) v = __float2bfloat16_rn(0.f);
    else v = 0.f;
    Wc[r * nd_pad + j] = v;
  }
}

template <class T>
__global__ void gather_rows_kernel(const T* __restrict__ W, const int* __restrict__ dead_list,
                                   const int* __restrict__ n_dead, T* __restrict__ out, int F, int D, int nd_pad,
                                   int crosslayer) {
  const int j = blockIdx.x, p = blockIdx.y;
  int s = p, t = p;
  if (crosslayer) pair_split(p, t, s);
  const bool live = j < n_dead[s];
  const int f = live ? dead_list[(size_t)s * F + j] : 0;
  const uint4* src = reinterpret_cast<const uint4*>(W + ((size_t)p * F + f) * D);
  uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)p * nd_pad + j) * D);
  const int nv = D * (int)sizeof(T) / 16;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = live ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
}

// dst[p, dead_list[s(p)][j], :] += src[p, j, :]   (fp32 gradients)
__global__ void scatter_rows_kernel(const float* __restrict__ src, const int* __restrict__ dead_list,
                                    const int* __restrict__ n_dead, float* __restrict__ dst, int F, int D, int nd_pad,
                                    int crosslayer) {
  const int j = blockIdx.x, p = blockIdx.y;
  int s = p, t = p;
  if (crosslayer) pair_split(p, t, s);
  if (j >= n_dead[s]) return;
  const int f = dead_list[(size_t)s * F + j];
  const float4* a = reinterpret_cast<const float4*>(src + ((size_t)p * nd_pad + j) * D);
  float4* o = reinterpret_cast<float4*>(dst + ((size_t)p * F + f) * D);
  for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
    float4 x = o[i];
    const float4 y = a[i];
    x.x += y.x, x.y += y.y, x.z += y.z, x.w += y.w;
    o[i] = x;
  }
}

template <class T>
int launch_dec_fwd(const int* idx, const float* val, const int* row_start, const int* row_cnt, long long npl,
                   const void* W, const float* b_dec, float* recon, int B, int L, int D, int F, int k, int crosslayer,
                   int short_rows, int* status, cudaStream_t s, PushDst push = PushDst{{0ull}, 0, 0, 0}) {
  const int vpl = (D / 8 + 31) / 32;
  dim3 grid(B, L);
  const size_t smem = 4 * (size_t)D * sizeof(float);
  const unsigned wgrid = (unsigned)(((long long)B * L + 3) / 4);
#define CLT_DEC_FWD(V)                                                                                              \
  case V:                                                                                                           \
    if (short_rows) {                                                                                               \
      sparse_dec_fwd_warp_kernel<T, V><<<wgrid, 128, 0, s>>>(idx, val, row_start, row_cnt, npl, (const T*)W, b_dec, \
                                                             recon, B, L, D, F, k, crosslayer, status, push);       \
      break;                                                                                                        \
    }                                                                                                               \
    CLT_CHECK_CUDA(cudaFuncSetAttribute(sparse_dec_fwd_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                        (int)smem));                                                                \
    sparse_dec_fwd_kernel<T, V><<<grid, 128, smem, s>>>(idx, val, row_start, row_cnt, npl, (const T*)W, b_dec,      \
                                                        recon, B, L, D, F, k, crosslayer, status, push);            \
    break;
  switch (vpl) {
    CLT_DEC_FWD(1) CLT_DEC_FWD(2) CLT_DEC_FWD(3) CLT_DEC_FWD(4) CLT_DEC_FWD(6) CLT_DEC_FWD(8) CLT_DEC_FWD(9)
    CLT_DEC_FWD(12)
    default:
      set_error("sparse decoder: d_acts=%d is not supported (needs D/256 in {1,2,3,4,6,8,9,12} after rounding up)", D);
      return 1;
  }
#undef CLT_DEC_FWD
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <class T>
int launch_bwd_dec(const int* col_ptr, const int* ent, const float* val, const int* etok, long long npl, const void* W,
                   const void* drecon, float* dW, float* dval, int B, int L, int D, int F, int k, int crosslayer,
                   cudaStream_t s) {
  const int vpl = (D / 8 + 31) / 32;
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  const long long rows = (long long)P * F;
  const long long blocks = (rows + 3) / 4;
  CLT_CHECK_ARG(blocks < (1ll << 31), "sparse decoder backward: too many rows");
  const unsigned grid = (unsigned)blocks;
  const bool grouped = F % 8 == 0 && vpl <= 4;          // one warp per 8 features (see the kernel's comment)
  const long long n_groups = rows / 8;
  const unsigned ggrid = (unsigned)((n_groups + 3) / 4);
#define CLT_BWD_DEC(V)                                                                                            \
  case V:                                                                                                         \
    if (grouped && V <= 4)                                                                                        \
      sparse_bwd_dec_group_kernel<T, (V <= 4 ? V : 1)><<<ggrid, 128, 0, s>>>(                                     \
          col_ptr, ent, val, etok, npl, (const T*)W, (const T*)drecon, dW, dval, B, L, D, F, k, crosslayer,       \
          n_groups);                                                                                              \
    else                                                                                                          \
      sparse_bwd_dec_kernel<T, V><<<grid, 128, 0, s>>>(col_ptr, ent, val, etok, npl, (const T*)W,                 \
                                                       (const T*)drecon, dW, dval, B, L, D, F, k, crosslayer,     \
                                                       rows);                                                     \
    break;
  switch (vpl) {
    CLT_BWD_DEC(1) CLT_BWD_DEC(2) CLT_BWD_DEC(3) CLT_BWD_DEC(4) CLT_BWD_DEC(6) CLT_BWD_DEC(8) CLT_BWD_DEC(9)
    CLT_BWD_DEC(12)
    default:
      set_error("sparse decoder backward: d_acts=%d is not supported", D);
      return 1;
  }
#undef CLT_BWD_DEC
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_sparse_decoder_fwd(const int* idx, const float* val, const int* row_start, const int* row_cnt, int64_t npl,
                           const void* W_dec, const float* b_dec, float* recon, int B, int L, int D, int F, int k,
                           int crosslayer, int short_rows, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && F > 0 && k > 0, "sparse_decoder_fwd: bad dims B=%d L=%d D=%d F=%d k=%d", B,
                L, D, F, k);
  CLT_CHECK_ARG(D % 8 == 0, "sparse_decoder_fwd: d_acts=%d must be a multiple of 8", D);
  CLT_CHECK_ARG(idx && val && W_dec && recon, "sparse_decoder_fwd: null pointer");
  CLT_CHECK_ARG((row_start == nullptr) == (row_cnt == nullptr), "sparse_decoder_fwd: row_start and row_cnt go together");
  CLT_CHECK_ARG(row_start != nullptr || npl == (int64_t)B * k, "sparse_decoder_fwd: fixed slots need npl = B*k");
  CLT_CHECK_ARG(B <= 2147483647 && L <= 65535, "sparse_decoder_fwd: grid too large");
  if (bf16)
    return launch_dec_fwd<__nv_bfloat16>(idx, val, row_start, row_cnt, npl, W_dec, b_dec, recon, B, L, D, F, k,
                                         crosslayer, short_rows, status, (cudaStream_t)stream);
  return launch_dec_fwd<float>(idx, val, row_start, row_cnt, npl, W_dec, b_dec, recon, B, L, D, F, k, crosslayer,
                               short_rows, status, (cudaStream_t)stream);
}

int clt_sparse_decoder_fwd_push(const int* idx, const float* val, const int* row_start, const int* row_cnt, int64_t npl,
                                const void* W_dec, const float* b_dec, const uint64_t* rank_bases, int rows_per_rank,
                                int n_ranks, int my_slot, int slot_bf16, int B, int L, int D, int F, int k,
                                int crosslayer, int short_rows, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && F > 0 && k > 0, "sparse_decoder_fwd_push: bad dims B=%d L=%d D=%d F=%d k=%d",
                B, L, D, F, k);
  CLT_CHECK_ARG(D % 8 == 0, "sparse_decoder_fwd_push: d_acts=%d must be a multiple of 8", D);
  CLT_CHECK_ARG(idx && val && W_dec && rank_bases, "sparse_decoder_fwd_push: null pointer");
  CLT_CHECK_ARG((row_start == nullptr) == (row_cnt == nullptr),
                "sparse_decoder_fwd_push: row_start and row_cnt go together");
  CLT_CHECK_ARG(row_start != nullptr || npl == (int64_t)B * k, "sparse_decoder_fwd_push: fixed slots need npl = B*k");
  CLT_CHECK_ARG(B <= 2147483647 && L <= 65535, "sparse_decoder_fwd_push: grid too large");
  CLT_CHECK_ARG(n_ranks > 0 && n_ranks <= kMaxPushRanks && rows_per_rank > 0 &&
                    (long long)rows_per_rank * n_ranks >= B,
                "sparse_decoder_fwd_push: %d ranks x %d rows do not cover B=%d (at most %d ranks)", n_ranks,
                rows_per_rank, B, kMaxPushRanks);
  PushDst push;
  for (int r = 0; r < kMaxPushRanks; ++r) push.bases[r] = r < n_ranks ? (unsigned long long)rank_bases[r] : 0ull;
  CLT_CHECK_ARG(my_slot >= 0 && my_slot < n_ranks, "sparse_decoder_fwd_push: slot %d of %d", my_slot, n_ranks);
  push.rows_per_rank = rows_per_rank;
  push.slot_offset = (long long)my_slot * rows_per_rank * L * D;
  push.slot_bf16 = slot_bf16 ? 1 : 0;
  if (bf16)
    return launch_dec_fwd<__nv_bfloat16>(idx, val, row_start, row_cnt, npl, W_dec, b_dec, nullptr, B, L, D, F, k,
                                         crosslayer, short_rows, status, (cudaStream_t)stream, push);
  return launch_dec_fwd<float>(idx, val, row_start, row_cnt, npl, W_dec, b_dec, nullptr, B, L, D, F, k, crosslayer,
                               short_rows, status, (cudaStream_t)stream, push);
}

int clt_csc_build(const int* idx, const float* val, int* col_ptr, int* cursor, int* ent, int64_t npl, int L, int F,
                  int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(npl > 0 && L > 0 && F > 0, "csc_build: bad dims npl=%lld L=%d F=%d", (long long)npl, L, F);
  CLT_CHECK_ARG(idx && val && col_ptr && cursor && ent, "csc_build: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_ARG(npl < (1ll << 31), "csc_build: too many entries per layer");
  CLT_CHECK_CUDA(cudaMemsetAsync(col_ptr, 0, sizeof(int) * (size_t)L * (F + 1), s));
  const long long total = npl * L;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  csc_count_kernel<<<blocks, 256, 0, s>>>(idx, val, col_ptr, npl, F, L, status);
  csc_scan_kernel<<<L, 1024, 0, s>>>(col_ptr, cursor, F);
  csc_fill_kernel<<<blocks, 256, 0, s>>>(idx, val, cursor, ent, npl, F, L);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Host-side address of g_static_cursor per device.  In host code the array's name is only a
// stand-in for the symbol, not a device address, so it is resolved once per device, with that
// device current, and the resolved pointer is what the kernels receive.
static int* static_cursor_ptr(int* err) {
  static int* ptr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("csc_build_static: cannot identify the current device (%s)", cudaGetErrorString(e));
    *err = 2;
    return nullptr;
  }
  if (ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_cursor);
    if (e != cudaSuccess || p == nullptr) {
      set_error("csc_build_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      *err = 2;
      return nullptr;
    }
    ptr[dev] = static_cast<int*>(p);
  }
  *err = 0;
  return ptr[dev];
}

int clt_csc_build_static(const int* idx, const float* val, int* col_ptr, int* ent, int64_t npl, int L, int F,
                         int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(npl > 0 && L > 0 && F > 0, "csc_build_static: bad dims npl=%lld L=%d F=%d", (long long)npl, L, F);
  CLT_CHECK_ARG(idx && val && col_ptr && ent, "csc_build_static: null pointer");
  CLT_CHECK_ARG((long long)L * F <= kStaticCursorCap,
                "csc_build_static: L*F = %lld exceeds the built-in scratch of %lld entries; use clt_csc_build with a "
                "caller-provided cursor buffer",
                (long long)L * F, kStaticCursorCap);
  int err = 0;
  int* cursor = static_cursor_ptr(&err);
  if (cursor == nullptr) return err;
  // every cursor entry in [0, L*F) is rewritten by the scan before the fill reads it, so nothing left
  // in the array by an earlier call is ever observed
  return clt_csc_build(idx, val, col_ptr, cursor, ent, npl, L, F, status, stream);
}

int clt_sparse_bwd_dec(const int* col_ptr, const int* ent, const float* val, const int* etok, int64_t npl,
                       const void* W_dec, const void* drecon, float* dW, float* dval, int B, int L, int D, int F, int k,
                       int crosslayer, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && F > 0 && k > 0 && npl > 0, "sparse_bwd_dec: bad dims");
  CLT_CHECK_ARG(D % 8 == 0, "sparse_bwd_dec: d_acts=%d must be a multiple of 8", D);
  CLT_CHECK_ARG(col_ptr && ent && val && W_dec && drecon && dW && dval, "sparse_bwd_dec: null pointer");
  CLT_CHECK_CUDA(cudaMemsetAsync(dval, 0, sizeof(float) * (size_t)L * npl, (cudaStream_t)stream));
  if (bf16)
    return launch_bwd_dec<__nv_bfloat16>(col_ptr, ent, val, etok, npl, W_dec, drecon, dW, dval, B, L, D, F, k,
                                         crosslayer, (cudaStream_t)stream);
  return launch_bwd_dec<float>(col_ptr, ent, val, etok, npl, W_dec, drecon, dW, dval, B, L, D, F, k, crosslayer,
                               (cudaStream_t)stream);
}

int clt_sparse_bwd_enc(const int* col_ptr, const int* ent, const float* dval, const int* etok, int64_t npl,
                       const void* xn, float* dW_enc, float* db_enc, const float* dW_aux, const float* db_aux,
                       const int* dead_pos, int nd_pad, int B, int L, int D, int F, int k, int bf16,
                       clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && F > 0 && k > 0 && npl > 0, "sparse_bwd_enc: bad dims");
  CLT_CHECK_ARG(col_ptr && ent && dval && xn && dW_enc && db_enc, "sparse_bwd_enc: null pointer");
  CLT_CHECK_ARG((dW_aux == nullptr) == (db_aux == nullptr) && (dW_aux == nullptr) == (dead_pos == nullptr),
                "sparse_bwd_enc: dW_aux, db_aux and dead_pos go together");
  CLT_CHECK_ARG(dW_aux == nullptr || nd_pad > 0, "sparse_bwd_enc: nd_pad=%d", nd_pad);
  dim3 grid((F + kEncFB - 1) / kEncFB, L, (D + 767) / 768);
  CLT_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "sparse_bwd_enc: grid too large");
  static_assert(kEncFB == 8, "the vector form writes its 8 features as two float4");
  if (D % 8 == 0 && (uintptr_t)xn % 16 == 0) {   // 16-byte loads of the x rows
    dim3 vgrid(grid.x, L, (D / 8 + 127) / 128);
    if (bf16)
      sparse_bwd_enc_vec_kernel<__nv_bfloat16><<<vgrid, 128, 0, (cudaStream_t)stream>>>(
          col_ptr, ent, dval, etok, npl, (const __nv_bfloat16*)xn, dW_enc, db_enc, B, D, F, k, dW_aux, db_aux, dead_pos,
          nd_pad);
    else
      sparse_bwd_enc_vec_kernel<float><<<vgrid, 128, 0, (cudaStream_t)stream>>>(
          col_ptr, ent, dval, etok, npl, (const float*)xn, dW_enc, db_enc, B, D, F, k, dW_aux, db_aux, dead_pos, nd_pad);
    CLT_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (bf16)
    sparse_bwd_enc_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        col_ptr, ent, dval, etok, npl, (const __nv_bfloat16*)xn, dW_enc, db_enc, B, D, F, k, dW_aux, db_aux, dead_pos,
        nd_pad);
  else
    sparse_bwd_enc_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(col_ptr, ent, dval, etok, npl,
                                                                        (const float*)xn, dW_enc, db_enc, B, D, F, k,
                                                                        dW_aux, db_aux, dead_pos, nd_pad);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_gather_enc_cols(const void* W_enc, const float* b_enc, const int* dead_list, const int* n_dead, void* Wc,
                        float* bc, int L, int D, int F, int nd_pad, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(L > 0 && F > 0 && D > 0 && nd_pad > 0, "gather_enc_cols: bad dims");
  CLT_CHECK_ARG(W_enc && b_enc && dead_list && n_dead && Wc && bc, "gather_enc_cols: null pointer");
  dim3 grid((nd_pad + 255) / 256, D < 64 ? D : 64, L);
  if (bf16)
    gather_enc_cols_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)W_enc, b_enc, dead_list, n_dead, (__nv_bfloat16*)Wc, bc, D, F, nd_pad);
  else
    gather_enc_cols_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)W_enc, b_enc, dead_list,
                                                                         n_dead, (float*)Wc, bc, D, F, nd_pad);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_gather_rows(const void* W_dec, const int* dead_list, const int* n_dead, void* out, int L, int F, int D,
                    int nd_pad, int crosslayer, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(L > 0 && F > 0 && D > 0 && nd_pad > 0, "gather_rows: bad dims");
  CLT_CHECK_ARG((D * (bf16 ? 2 : 4)) % 16 == 0, "gather_rows: rows must be multiples of 16 bytes");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  dim3 grid(nd_pad, P);
  if (bf16)
    gather_rows_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)W_dec, dead_list, n_dead, (__nv_bfloat16*)out, F, D, nd_pad, crosslayer);
  else
    gather_rows_kernel<float><<<grid, 128, 0, (cudaStream_t)stream>>>((const float*)W_dec, dead_list, n_dead,
                                                                     (float*)out, F, D, nd_pad, crosslayer);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_scatter_rows(const float* src, const int* dead_list, const int* n_dead, float* dW_dec, int L, int F, int D,
                     int nd_pad, int crosslayer, clt_stream_t stream) {
  CLT_CHECK_ARG(L > 0 && F > 0 && D > 0 && nd_pad > 0 && D % 4 == 0, "scatter_rows: bad dims");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  dim3 grid(nd_pad, P);
  scatter_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(src, dead_list, n_dead, dW_dec, F, D, nd_pad, crosslayer);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
