// TopK selection kernels (HBM-bound, no tensor cores).
//
// Per (token, layer) row the reference keeps the k largest pre-activations and passes
// them through a ReLU (crosslayer_transcoder/model/topk.py:56-61).  A kept value that
// is not positive becomes 0 and receives no gradient, so the result equals "the
// min(k, #positive) largest POSITIVE values": these kernels select among positive
// values only, whose IEEE bit patterns order like unsigned integers.
//
// Selection is an exact three-level radix select on the 31 value bits (11 + 11 + 9):
// a shared-memory histogram per level narrows the bucket that holds the k-th largest
// value until the threshold key T and the number r of elements equal to T that still
// fit are known; everything above T and the first r elements equal to T are emitted.
// One CTA of 256 threads owns a row and re-reads it from L1/L2 for every level.
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {

namespace {

constexpr int kSelThreads = 256;
constexpr int kBins = 2048;

template <class T>
__device__ __forceinline__ float ld_as_float(const T* p, int i);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p, int i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int i) {
  return __bfloat162float(__ldg(p + i));
}

// digit of `key` at a radix level, and whether `key` lies in the bucket selected so far
__device__ __forceinline__ bool level_digit(unsigned key, int level, unsigned prefix, unsigned& digit) {
  if (level == 0) {
    digit = key >> 20;  // sign bit is 0 for positive values: 11 significant bits
    return true;
  }
  if (level == 1) {
    digit = (key >> 9) & 0x7ffu;
    return (key >> 20) == prefix;
  }
  digit = key & 0x1ffu;
  return (key >> 9) == prefix;
}

// Find the bucket d with  count(buckets > d) < want <= count(buckets >= d) and the count
// strictly above it.  256 threads, 8 bins each; suffix sums by warp shuffles.
__device__ void pick_bucket(const int* hist, int want, int* sh_digit, int* sh_above) {
  __shared__ int wtot[kSelThreads / 32];
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  int local[8];
  int s = 0;
#pragma unroll
  for (int i = 7; i >= 0; --i) {
    s += hist[t * 8 + i];
    local[i] = s;  // sum of bins t*8+i .. t*8+7
  }
  int x = s;  // becomes the sum over lanes >= lane of this warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_down_sync(0xffffffffu, x, o);
    if (lane + o < 32) x += y;
  }
  if (lane == 0) wtot[w] = x;
  __syncthreads();
  int above = x - s;  // threads after this one in the warp
  for (int j = w + 1; j < kSelThreads / 32; ++j) above += wtot[j];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gt = above + (i < 7 ? local[i + 1] : 0);
    const int ge = above + local[i];
    if (gt < want && want <= ge) {
      *sh_digit = t * 8 + i;
      *sh_above = gt;
    }
  }
  __syncthreads();
}

struct RowSelect {
  unsigned T;   // threshold key (0: every positive value is kept)
  int r;        // how many elements equal to T are kept
};

// Exact k-th largest positive value of one row, by all threads of the CTA.
// key_at(i) returns the key of element i (0 for elements that do not take part).
template <class KeyFn>
__device__ RowSelect radix_select(int n, int k, KeyFn key_at) {
  __shared__ int hist[kBins];
  __shared__ int sh_digit, sh_above, sh_total;
  unsigned prefix = 0;
  int want = k;
  RowSelect out{0u, 0};
  for (int level = 0; level < 3; ++level) {
    for (int i = threadIdx.x; i < kBins; i += kSelThreads) hist[i] = 0;
    if (threadIdx.x == 0) sh_total = 0;
    __syncthreads();
    int mine = 0;
    for (int i = threadIdx.x; i < n; i += kSelThreads) {
      const unsigned key = key_at(i);
      unsigned d;
      if (key != 0u && level_digit(key, level, prefix, d)) {
        atomicAdd(&hist[d], 1);
        ++mine;
      }
    }
    if (mine) atomicAdd(&sh_total, mine);
    __syncthreads();
    if (sh_total < want) {  // fewer candidates than slots: keep them all (only possible at level 0)
      __syncthreads();
      return RowSelect{0u, 0};
    }
    if (threadIdx.x == 0) sh_digit = 0, sh_above = 0;
    __syncthreads();
    pick_bucket(hist, want, &sh_digit, &sh_above);
    const unsigned d = (unsigned)sh_digit;
    want -= sh_above;
    if (level == 0)
      prefix = d;
    else if (level == 1)
      prefix = (prefix << 11) | d;
    else
      out.T = (prefix << 9) | d;
    __syncthreads();
  }
  out.r = want;  // elements equal to T still to take (>= 1)
  return out;
}

__device__ __forceinline__ unsigned positive_key(float v) { return v > 0.f ? __float_as_uint(v) : 0u; }

// ---------------------------------------------------------------------------------------
// Main selection: idx/val [L, B, k] of the k largest positive pre-activations per row,
// unused slots (fewer than k positives) hold idx 0 / val 0.  Marks fired features.
//
// Fast path (k <= 256): two sweeps over the row and no histogram.
//   sweep 1  every thread keeps the maximum of its strided share of the row; the k-th
//            largest of the 256 thread maxima is a lower bound T_lo of the row's k-th
//            largest value (the maxima are 256 distinct elements of the row)
//   sweep 2  the elements >= T_lo (k of them at least, a few more in expectation) go to
//            a shared-memory candidate list
//   finish   rank the candidates by counting; rank < k is the selection, slot = rank
// A row whose candidate list overflows (masses of equal values) falls back to the exact
// radix select above.
// ---------------------------------------------------------------------------------------
constexpr int kCandCap = 1024;

template <class T>
struct RowReader;
template <>
struct RowReader<__nv_bfloat16> {
  // 8 consecutive elements starting at a multiple of 8
  __device__ static __forceinline__ void load8(const __nv_bfloat16* z, const float* b, int i, float (&o)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4*>(z + i));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + i));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(b + i) + 1);
    o[0] = __uint_as_float(t.x << 16) + b0.x;
    o[1] = __uint_as_float(t.x & 0xffff0000u) + b0.y;
    o[2] = __uint_as_float(t.y << 16) + b0.z;
    o[3] = __uint_as_float(t.y & 0xffff0000u) + b0.w;
    o[4] = __uint_as_float(t.z << 16) + b1.x;
    o[5] = __uint_as_float(t.z & 0xffff0000u) + b1.y;
    o[6] = __uint_as_float(t.w << 16) + b1.z;
    o[7] = __uint_as_float(t.w & 0xffff0000u) + b1.w;
  }
};
template <>
struct RowReader<float> {
  __device__ static __forceinline__ void load8(const float* z, const float* b, int i, float (&o)[8]) {
    const float4 z0 = __ldg(reinterpret_cast<const float4*>(z + i));
    const float4 z1 = __ldg(reinterpret_cast<const float4*>(z + i) + 1);
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + i));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(b + i) + 1);
    o[0] = z0.x + b0.x, o[1] = z0.y + b0.y, o[2] = z0.z + b0.z, o[3] = z0.w + b0.w;
    o[4] = z1.x + b1.x, o[5] = z1.y + b1.y, o[6] = z1.z + b1.z, o[7] = z1.w + b1.w;
  }
};

template <class T>
__global__ void __launch_bounds__(kSelThreads)
select_topk_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, int* __restrict__ idx_out,
                   float* __restrict__ val_out, unsigned* __restrict__ fired_bits, int B, int F, int k) {
  const int row = blockIdx.x;  // l * B + b
  const int l = row / B;
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  int* io = idx_out + (size_t)row * k;
  float* vo = val_out + (size_t)row * k;
  const int words = (F + 31) / 32;
  const int tid = threadIdx.x;

  __shared__ float tmax[kSelThreads];
  __shared__ float cand_v[kCandCap];
  __shared__ int cand_i[kCandCap];
  __shared__ int n_cand;
  __shared__ float t_lo;

  bool fast = (k <= kSelThreads) && (F % 8 == 0) && (F >= 8 * kSelThreads);
  if (fast) {
    // ---- sweep 1: per-thread maxima
    float m = 0.f;
    for (int i = 8 * tid; i < F; i += 8 * kSelThreads) {
      float v[8];
      RowReader<T>::load8(zr, br, i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) m = fmaxf(m, v[q]);
    }
    tmax[tid] = m;  // 0 when the thread saw no positive value
    if (tid == 0) n_cand = 0, t_lo = 0.f;
    __syncthreads();
    // k-th largest of the 256 maxima by rank counting (ties ordered by thread id)
    int rank = 0;
    for (int j = 0; j < kSelThreads; ++j) {
      const float o = tmax[j];
      rank += (o > m || (o == m && j < tid)) ? 1 : 0;
    }
    if (rank == k - 1) t_lo = m;
    __syncthreads();
    const float lo = t_lo;  // 0: fewer than k threads saw a positive value -> take every positive
    // ---- sweep 2: candidates
    for (int i = 8 * tid; i < F; i += 8 * kSelThreads) {
      float v[8];
      RowReader<T>::load8(zr, br, i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (v[q] > 0.f && v[q] >= lo) {
          const int c = atomicAdd(&n_cand, 1);
          if (c < kCandCap) cand_v[c] = v[q], cand_i[c] = i + q;
        }
      }
    }
    __syncthreads();
    const int nc = n_cand;
    if (nc > kCandCap) {
      fast = false;  // uniform: n_cand is shared
    } else {
      // ---- finish: rank by counting, rank < k selected, slot = rank
      for (int c = tid; c < nc; c += kSelThreads) {
        const float v = cand_v[c];
        const int fi = cand_i[c];
        int r = 0;
        for (int j = 0; j < nc; ++j) {
          const float o = cand_v[j];
          r += (o > v || (o == v && cand_i[j] < fi)) ? 1 : 0;
        }
        if (r < k) {
          io[r] = fi;
          vo[r] = v;
          if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + fi / 32, 1u << (fi & 31));
        }
      }
      for (int s2 = nc + tid; s2 < k; s2 += kSelThreads) io[s2] = 0, vo[s2] = 0.f;
      return;
    }
  }
  __syncthreads();

  // ---- exact radix select (general k, ragged F, or heavy ties)
  auto key_at = [&](int i) { return positive_key(ld_as_float<T>(zr, i) + __ldg(br + i)); };
  const RowSelect sel = radix_select(F, k, key_at);
  __shared__ int n_out, n_tie;
  if (tid == 0) n_out = 0, n_tie = 0;
  __syncthreads();
  for (int i = tid; i < F; i += kSelThreads) {
    const float v = ld_as_float<T>(zr, i) + __ldg(br + i);
    const unsigned key = positive_key(v);
    bool take = key > sel.T;
    if (!take && key != 0u && key == sel.T) take = atomicAdd(&n_tie, 1) < sel.r;
    if (take) {
      const int slot = atomicAdd(&n_out, 1);
      if (slot < k) {
        io[slot] = i;
        vo[slot] = v;
        if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + i / 32, 1u << (i & 31));
      }
    }
  }
  __syncthreads();
  for (int s2 = n_out + tid; s2 < k; s2 += kSelThreads) io[s2] = 0, vo[s2] = 0.f;
}

// ---------------------------------------------------------------------------------------
// Main selection for short rows (a feature shard's slice): one WARP per row, 8 rows per CTA,
// so that the per-row launch and synchronisation overhead does not dominate when F is a few
// thousand.  Same scheme as above with 32 lanes instead of 256 threads (k <= 32):
//   sweep 1  the two largest values per lane; T_lo = k-th largest of those 64 (bisection on bits)
//   sweep 2  elements >= T_lo appended to the warp's shared-memory list
//   finish   exact k-th largest of the list by bisection on the key bits, then emit
// If the list overflows (masses of equal values) the exact k-th value is found by bisection on
// the key bits over the row, and the row is emitted from that threshold.
// ---------------------------------------------------------------------------------------
constexpr int kWarpCand = 256;

template <class T>
__global__ void __launch_bounds__(256)
select_topk_warp_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, int* __restrict__ idx_out,
                        float* __restrict__ val_out, unsigned* __restrict__ fired_bits, long long rows, int B, int F,
                        int k) {
  __shared__ float cand_v[8][kWarpCand];
  __shared__ int cand_i[8][kWarpCand];
  __shared__ int cand_n[8];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8ll + wib;
  if (row >= rows) return;
  const int l = (int)(row / B);
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  int* io = idx_out + (size_t)row * k;
  float* vo = val_out + (size_t)row * k;
  const int words = (F + 31) / 32;
  float* cv = cand_v[wib];
  int* ci = cand_i[wib];

  // sweep 1: the two largest values of every lane's share -> 64 distinct elements of the row
  float m1 = 0.f, m2 = 0.f;
  for (int i = 8 * lane; i < F; i += 256) {
    float v[8];
    RowReader<T>::load8(zr, br, i, v);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float x = v[q];
      m2 = fmaxf(m2, fminf(m1, x));
      m1 = fmaxf(m1, x);
    }
  }
  // T_lo = k-th largest of the 64 values (lower bound of the row's k-th largest): bisection on the bits
  const unsigned k1 = positive_key(m1), k2 = positive_key(m2);
  unsigned lo_key = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = lo_key | (1u << bit);
    const int c = __popc(__ballot_sync(0xffffffffu, k1 >= trial)) + __popc(__ballot_sync(0xffffffffu, k2 >= trial));
    if (c >= k) lo_key = trial;
  }
  if (lane == 0) cand_n[wib] = 0;
  __syncwarp();
  // sweep 2: candidates (>= T_lo; every positive value when fewer than k of the 64 are positive)
  for (int i = 8 * lane; i < F; i += 256) {
    float v[8];
    RowReader<T>::load8(zr, br, i, v);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const unsigned key = positive_key(v[q]);
      if (key != 0u && key >= lo_key) {
        const int c = atomicAdd(&cand_n[wib], 1);
        if (c < kWarpCand) cv[c] = v[q], ci[c] = i + q;
      }
    }
  }
  __syncwarp();
  const int nc = cand_n[wib];
  if (nc <= kWarpCand) {
    // exact k-th largest key among the candidates by bisection, then emit (> T, then ties in list order)
    unsigned ck[kWarpCand / 32];
#pragma unroll
    for (int q = 0; q < kWarpCand / 32; ++q) ck[q] = (lane + 32 * q) < nc ? positive_key(cv[lane + 32 * q]) : 0u;
    unsigned Tk = 0u;
    if (nc > k) {
      for (int bit = 30; bit >= 0; --bit) {
        const unsigned trial = Tk | (1u << bit);
        int c = 0;
#pragma unroll
        for (int q = 0; q < kWarpCand / 32; ++q) c += ck[q] >= trial ? 1 : 0;
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= k) Tk = trial;
      }
    }
    int n_gt = 0;
#pragma unroll
    for (int q = 0; q < kWarpCand / 32; ++q) n_gt += ck[q] > Tk ? 1 : 0;
    n_gt = __reduce_add_sync(0xffffffffu, n_gt);
    int n_out = 0, ties_left = (nc > k) ? k - n_gt : 0x7fffffff;
#pragma unroll
    for (int q = 0; q < kWarpCand / 32; ++q) {
      const unsigned key = ck[q];
      const bool gt = key > Tk;
      const bool tie = key != 0u && key == Tk;
      const unsigned tb = __ballot_sync(0xffffffffu, tie);
      const bool take = gt || (tie && __popc(tb & ((1u << lane) - 1u)) < ties_left);
      const unsigned bal = __ballot_sync(0xffffffffu, take);
      if (take) {
        const int slot = n_out + __popc(bal & ((1u << lane) - 1u));
        const int c = lane + 32 * q;
        if (slot < k) {
          const int fi = ci[c];
          io[slot] = fi;
          vo[slot] = cv[c];
          if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + fi / 32, 1u << (fi & 31));
        }
      }
      n_out += __popc(bal);
      ties_left -= min(ties_left, __popc(tb));
    }
    for (int s2 = n_out + lane; s2 < k; s2 += 32) io[s2] = 0, vo[s2] = 0.f;
    return;
  }
  // overflow: exact threshold by bisection on the key bits (largest T with count(key >= T) >= k)
  unsigned Tk = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = Tk | (1u << bit);
    int c = 0;
    for (int i = lane; i < F; i += 32) c += positive_key(ld_as_float<T>(zr, i) + __ldg(br + i)) >= trial ? 1 : 0;
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) Tk = trial;
  }
  int n_gt = 0;
  for (int i = lane; i < F; i += 32) n_gt += positive_key(ld_as_float<T>(zr, i) + __ldg(br + i)) > Tk ? 1 : 0;
  n_gt = __reduce_add_sync(0xffffffffu, n_gt);
  int n_out = 0, ties_left = k - n_gt;  // Tk == 0 only if fewer than k positives: then every positive is above it
  for (int i0 = 0; i0 < F; i0 += 32) {
    const int i = i0 + lane;
    const float v = i < F ? ld_as_float<T>(zr, i) + __ldg(br + i) : 0.f;
    const unsigned key = positive_key(v);
    const bool gt = key > Tk;
    const bool tie = key != 0u && key == Tk;
    const unsigned tb = __ballot_sync(0xffffffffu, tie);
    const bool tie_take = tie && (__popc(tb & ((1u << lane) - 1u)) < ties_left);
    const bool take = gt || tie_take;
    const unsigned bal = __ballot_sync(0xffffffffu, take);
    if (take) {
      const int slot = n_out + __popc(bal & ((1u << lane) - 1u));
      if (slot < k) {
        io[slot] = i;
        vo[slot] = v;
        if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + i / 32, 1u << (i & 31));
      }
    }
    n_out += __popc(bal);
    ties_left -= min(ties_left, __popc(tb));
  }
  for (int s2 = n_out + lane; s2 < k; s2 += 32) io[s2] = 0, vo[s2] = 0.f;
}

// ---------------------------------------------------------------------------------------
// Main selection for long rows in ONE sweep: a warp streams its row once and keeps a running
// candidate list in shared memory.
//
//   * A value joins the list when its key is at least tau (tau starts at the smallest positive key).
//   * When the list could overflow, the warp finds the k-th largest key T of the list (bisection on the
//     key bits over values held in registers), keeps the k best entries and raises tau to T + 1: from
//     then on only values that would displace one of the k held ones join (a value equal to the current
//     k-th is interchangeable with it).  After the first few hundred elements tau sits near the row's
//     final threshold and almost nothing joins any more: k (1 + ln(F / 256)) entries in expectation.
//   * At the end of the row one more such step leaves exactly min(k, #positive) entries.
//
// A CTA is 8 independent warps = 8 consecutive tokens of one layer (no CTA-wide barrier).  The row is
// read exactly once, 256 columns per step with the next step's values already requested; the fp32 bias
// comes through L1, which the warps of the CTAs resident on an SM share because they walk the same
// layer's bias at about the same pace.  The filter is one floating-point compare per element
// (pre >= tau with tau > 0 also rejects everything that is not positive).  k <= kStreamCap - 256.
// ---------------------------------------------------------------------------------------
constexpr int kStreamWarps = 8;
constexpr int kStreamMinF = 2048;   // shorter rows keep the one-warp-per-row two-sweep kernel
constexpr int kStreamCap = 512;

template <class T>
struct ChunkLoader;
template <>
struct ChunkLoader<__nv_bfloat16> {
  using Raw = uint4;  // 8 values
  __device__ static __forceinline__ Raw load(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ static __forceinline__ void unpack(const Raw& t, float (&o)[8]) {
    o[0] = __uint_as_float(t.x << 16), o[1] = __uint_as_float(t.x & 0xffff0000u);
    o[2] = __uint_as_float(t.y << 16), o[3] = __uint_as_float(t.y & 0xffff0000u);
    o[4] = __uint_as_float(t.z << 16), o[5] = __uint_as_float(t.z & 0xffff0000u);
    o[6] = __uint_as_float(t.w << 16), o[7] = __uint_as_float(t.w & 0xffff0000u);
  }
};
template <>
struct ChunkLoader<float> {
  struct Raw {
    float4 a, b;
  };
  __device__ static __forceinline__ Raw load(const float* p) {
    Raw r;
    r.a = __ldcs(reinterpret_cast<const float4*>(p));
    r.b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    return r;
  }
  __device__ static __forceinline__ void unpack(const Raw& r, float (&o)[8]) {
    o[0] = r.a.x, o[1] = r.a.y, o[2] = r.a.z, o[3] = r.a.w, o[4] = r.b.x, o[5] = r.b.y, o[6] = r.b.z, o[7] = r.b.w;
  }
};

// Keep the k best of the n entries of a warp's candidate list (n <= kStreamCap, n > k); returns the k-th
// largest key.  Entries equal to it are kept in list order until k are held.
__device__ __forceinline__ unsigned stream_keep_top(float* cv, int* ci, int n, int k) {
  const int lane = threadIdx.x & 31;
  constexpr int kPer = kStreamCap / 32;
  unsigned key[kPer];
#pragma unroll
  for (int q = 0; q < kPer; ++q) key[q] = (lane + 32 * q) < n ? __float_as_uint(cv[lane + 32 * q]) : 0u;
  unsigned Tk = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = Tk | (1u << bit);
    int c = 0;
#pragma unroll
    for (int q = 0; q < kPer; ++q) c += key[q] >= trial ? 1 : 0;
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) Tk = trial;
  }
  int n_gt = 0;
#pragma unroll
  for (int q = 0; q < kPer; ++q) n_gt += key[q] > Tk ? 1 : 0;
  n_gt = __reduce_add_sync(0xffffffffu, n_gt);
  int ties_left = k - n_gt, n_out = 0;
#pragma unroll
  for (int q = 0; q < kPer; ++q) {   // in-place: an entry never moves to a later position
    const int c = lane + 32 * q;
    const bool gt = key[q] > Tk, tie = key[q] == Tk && key[q] != 0u;
    const unsigned tb = __ballot_sync(0xffffffffu, tie);
    const bool take = gt || (tie && __popc(tb & ((1u << lane) - 1u)) < ties_left);
    const unsigned bal = __ballot_sync(0xffffffffu, take);
    const float v = c < n ? cv[c] : 0.f;
    const int f = c < n ? ci[c] : 0;
    __syncwarp();
    if (take) {
      const int slot = n_out + __popc(bal & ((1u << lane) - 1u));
      cv[slot] = v;
      ci[slot] = f;
    }
    __syncwarp();
    n_out += __popc(bal);
    ties_left -= min(ties_left, __popc(tb));
  }
  return Tk;
}

template <class T>
__global__ void __launch_bounds__(kStreamWarps * 32, 4)
select_topk_stream_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, int* __restrict__ idx_out,
                          float* __restrict__ val_out, unsigned* __restrict__ fired_bits, int B, int F, int k) {
  __shared__ float c_val[kStreamWarps][kStreamCap];
  __shared__ int c_idx[kStreamWarps][kStreamCap];
  __shared__ int c_cnt[kStreamWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int l = blockIdx.y;
  const int b = blockIdx.x * kStreamWarps + warp;
  if (b >= B) return;                       // warps are independent: no CTA-wide barrier below
  const size_t row = (size_t)l * B + b;
  const T* zr = z + row * F;
  const float* br = b_enc + (size_t)l * F;  // read through L1: the 8 warps of a CTA walk the same layer's bias
  float* cv = c_val[warp];
  int* ci = c_idx[warp];
  float tau = __uint_as_float(1u);          // smallest positive value: every positive value qualifies at first
  int* cnt = &c_cnt[warp];
  if (lane == 0) *cnt = 0;
  __syncwarp();
  using CL = ChunkLoader<T>;
  // 256 columns per step (8 per lane); the next step's row values are requested before this step's are used
  const int n_steps = F / 256;              // whole steps; the ragged end (F % 256, a multiple of 8) follows
  const int i_last = n_steps * 256 + 8 * lane;
  typename CL::Raw cur, nxt;
  float4 b0c, b1c, b0n, b1n;
  auto fetch = [&](int i, typename CL::Raw& r, float4& c0, float4& c1) {
    r = CL::load(zr + i);
    c0 = __ldg(reinterpret_cast<const float4*>(br + i));
    c1 = __ldg(reinterpret_cast<const float4*>(br + i) + 1);
  };
  auto consume = [&](int i, const typename CL::Raw& r, const float4& c0, const float4& c1) {
    float v[8];
    CL::unpack(r, v);
    v[0] += c0.x, v[1] += c0.y, v[2] += c0.z, v[3] += c0.w;
    v[4] += c1.x, v[5] += c1.y, v[6] += c1.z, v[7] += c1.w;
    bool any = false;
#pragma unroll
    for (int q = 0; q < 8; ++q) any |= v[q] >= tau;
    if (any) {
      // append (only lanes with hits run this): a shared-memory counter hands out the slots.  A step adds at
      // most 256 entries and the list is trimmed whenever it holds more than kStreamCap - 256, so it fits.
      int mine = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) mine += v[q] >= tau ? 1 : 0;
      int slot = atomicAdd(cnt, mine);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (v[q] >= tau) {
          cv[slot] = v[q];
          ci[slot] = i + q;
          ++slot;
        }
      }
    }
    __syncwarp();
    const int count = *reinterpret_cast<volatile int*>(cnt);
    if (count > kStreamCap - 256) {        // the next step could overflow the list: keep the k best, raise tau
      if (count > k) {
        tau = __uint_as_float(stream_keep_top(cv, ci, count, k) + 1u);
        if (lane == 0) *cnt = k;
      }
      __syncwarp();
    }
  };
  if (n_steps > 0) fetch(8 * lane, cur, b0c, b1c);
#pragma unroll 2
  for (int st = 0; st < n_steps; ++st) {
    const int i = st * 256 + 8 * lane;
    if (st + 1 < n_steps) fetch(i + 256, nxt, b0n, b1n);
    consume(i, cur, b0c, b1c);
    cur = nxt, b0c = b0n, b1c = b1n;
  }
  if (i_last < F) fetch(i_last, cur, b0c, b1c);
  if (__any_sync(0xffffffffu, i_last < F)) {
    // ragged end (F % 256 columns): lanes beyond F have nothing to add
    if (i_last < F) consume(i_last, cur, b0c, b1c);
    else consume(i_last, typename CL::Raw{}, make_float4(-1.f, -1.f, -1.f, -1.f), make_float4(-1.f, -1.f, -1.f, -1.f));
  }
  __syncwarp();
  int count = *reinterpret_cast<volatile int*>(cnt);
  if (count > k) {
    stream_keep_top(cv, ci, count, k);
    count = k;
  }
  __syncwarp();
  // Largest value first, as torch.topk returns them (bitonic sort of the <= 256 survivors in shared memory;
  // equal values in ascending feature order, so the output does not depend on the arrival order).  The order
  // matters to the token-major decoder gather that walks these lists (measurements at that kernel).
  {
    int n2 = 32;
    while (n2 < count) n2 <<= 1;
    for (int j = count + lane; j < n2; j += 32) ci[j] = 0x7fffffff, cv[j] = -1.f;
    __syncwarp();
    for (int size = 2; size <= n2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = lane; t < (n2 >> 1); t += 32) {
          const int i = ((t / stride) * (stride << 1)) + (t & (stride - 1)), j = i + stride;
          const bool up = (i & size) == 0;
          const float va = cv[i], vc = cv[j];
          const int a = ci[i], c = ci[j];
          const bool after = va < vc || (va == vc && a > c);     // entry i belongs after entry j
          if (after == up) ci[i] = c, ci[j] = a, cv[i] = vc, cv[j] = va;
        }
        __syncwarp();
      }
    }
  }
  int* io = idx_out + row * k;
  float* vo = val_out + row * k;
  const int words = (F + 31) / 32;
  for (int j = lane; j < k; j += 32) {
    const bool live = j < count;
    const int f = live ? ci[j] : 0;
    io[j] = f;
    vo[j] = live ? cv[j] : 0.f;
    if (live && fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + f / 32, 1u << (f & 31));
  }
}

// ---------------------------------------------------------------------------------------
// Dead-feature list per layer: dead_list[l, 0..n_dead[l]) = ascending indices with dead != 0.
// One CTA per layer.
// ---------------------------------------------------------------------------------------
__global__ void dead_compact_kernel(const unsigned char* __restrict__ dead, int* __restrict__ dead_list,
                                    int* __restrict__ n_dead, int F) {
  const int l = blockIdx.x;
  __shared__ int base;
  __shared__ int wsum[32];
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int f0 = 0; f0 < F; f0 += blockDim.x) {
    const int f = f0 + threadIdx.x;
    const int flag = (f < F && dead[(size_t)l * F + f]) ? 1 : 0;
    const unsigned bal = __ballot_sync(0xffffffffu, flag);
    const int before = __popc(bal & ((1u << lane) - 1u));
    if (lane == 0) wsum[w] = __popc(bal);
    __syncthreads();
    int woff = 0;
    for (int j = 0; j < w; ++j) woff += wsum[j];
    if (flag) dead_list[(size_t)l * F + base + woff + before] = f;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int j = 0; j < nw; ++j) tot += wsum[j];
      base += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) n_dead[l] = base;
}

// ---------------------------------------------------------------------------------------
// Auxiliary selection over the dead features of a row, written as a dense row of the
// compacted feature matrix:  a[l, b, j] = pre(dead_list[l][j]) if it is among the k_aux
// largest positive dead pre-activations of the row, else 0   (j < nd_pad; 0 beyond n_dead[l]).
// Values tied with the k_aux-th are all kept.
// ---------------------------------------------------------------------------------------
// mode 0: threshold computed here, dense row written (single GPU)
// mode 1: only the row's candidates are written: cand_out[row, 0..k_aux) = its k_aux largest positive
//         dead pre-activations (0-padded), for the exchange between feature shards
// mode 2: threshold given (thr[row], from the exchanged candidates), dense row written
template <class T>
__global__ void __launch_bounds__(kSelThreads)
select_aux_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, const int* __restrict__ dead_list,
                  const int* __restrict__ n_dead, T* __restrict__ a_out, float* __restrict__ cand_out,
                  const float* __restrict__ thr, int mode, int B, int F, int k_aux, int nd_pad,
                  const int* __restrict__ row_count, int* status) {
  extern __shared__ float cand[];  // pre-activations of the dead features of this row
  const int row = blockIdx.x;
  const int l = row / B;
  const int nd = min(n_dead[l], nd_pad);
  if (threadIdx.x == 0) {
    // the caller sized the compact operands (nd_pad) and chose the mode from counts of an earlier step:
    // more dead features than columns, or a row that needed the candidate exchange, is reported
    if (n_dead[l] > nd_pad) report_status(status, kOverflow);
    if (mode == 0 && row_count != nullptr && row_count[row] > k_aux) report_status(status, kOverflow);
  }
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  const int* dl = dead_list + (size_t)l * F;
  __shared__ int n_pos;
  if (threadIdx.x == 0) n_pos = 0;
  __syncthreads();
  int mine = 0;
  for (int j = threadIdx.x; j < nd; j += kSelThreads) {
    const int f = __ldg(dl + j);
    const float c = ld_as_float<T>(zr, f) + __ldg(br + f);
    cand[j] = c;
    mine += c > 0.f ? 1 : 0;
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  if ((threadIdx.x & 31) == 0 && mine > 0) atomicAdd(&n_pos, mine);
  __syncthreads();
  RowSelect sel{0u, 0};
  if (mode == 2) {
    sel.T = positive_key(thr[row]);
  } else if (n_pos > k_aux) {
    // (a row with at most k_aux positive values keeps all of them: threshold key 0, no select passes —
    // the usual case, dead features are rarely positive)
    auto key_at = [&](int j) { return positive_key(cand[j]); };
    sel = radix_select(nd, k_aux, key_at);
  }
  if (mode == 1) {
    __shared__ int n_out, n_tie;
    if (threadIdx.x == 0) n_out = 0, n_tie = 0;
    __syncthreads();
    float* co = cand_out + (size_t)row * k_aux;
    for (int j = threadIdx.x; j < nd; j += kSelThreads) {
      const float c = cand[j];
      const unsigned key = positive_key(c);
      bool take = key > sel.T;
      if (!take && key != 0u && key == sel.T) take = atomicAdd(&n_tie, 1) < sel.r;
      if (take) {
        const int slot = atomicAdd(&n_out, 1);
        if (slot < k_aux) co[slot] = c;
      }
    }
    __syncthreads();
    for (int s = n_out + threadIdx.x; s < k_aux; s += kSelThreads) co[s] = 0.f;
    return;
  }
  T* ao = a_out + (size_t)row * nd_pad;
  for (int j = threadIdx.x; j < nd_pad; j += kSelThreads) {
    float v = 0.f;
    if (j < nd) {
      const float c = cand[j];
      const unsigned key = positive_key(c);
      if (key != 0u && key >= sel.T) v = c;
    }
    if constexpr (sizeof(T) == 2)
      ao[j] = __float2bfloat16_rn(v);
    else
      ao[j] = v;
  }
}

// ---------------------------------------------------------------------------------------
// cnt[row] = number of positive pre-activations among the dead features of the row.  Feature
// shards sum these counts: a row whose total does not exceed k_aux keeps all of them, so no
// candidate exchange is needed for it.  One warp per row.
// ---------------------------------------------------------------------------------------
template <class T>
__global__ void aux_count_kernel(const T* __restrict__ z, const float* __restrict__ b_enc,
                                 const int* __restrict__ dead_list, const int* __restrict__ n_dead,
                                 int* __restrict__ cnt, long long rows, int B, int F) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int l = (int)(row / B);
  const int nd = n_dead[l];
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  const int* dl = dead_list + (size_t)l * F;
  int c = 0;
  for (int j = lane; j < nd; j += 32) {
    const int f = __ldg(dl + j);
    c += (ld_as_float<T>(zr, f) + __ldg(br + f) > 0.f) ? 1 : 0;
  }
  c = __reduce_add_sync(0xffffffffu, c);
  if (lane == 0) cnt[row] = c;
}

// ---------------------------------------------------------------------------------------
// Exchange between feature shards: every rank contributes its k best values of a row;
// thr[row] = the k-th largest positive value among all R * k of them (0 when there are fewer
// than k positive ones, i.e. every positive value stays).  vals [R, rows, k].
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSelThreads)
topk_threshold_kernel(const float* __restrict__ vals, float* __restrict__ thr, long long rows, int R, int k) {
  const long long row = blockIdx.x;
  auto key_at = [&](int i) { return positive_key(__ldg(vals + ((size_t)(i / k) * rows + row) * k + i % k)); };
  const RowSelect sel = radix_select(R * k, k, key_at);
  if (threadIdx.x == 0) thr[row] = __uint_as_float(sel.T);
}

// Same threshold for short candidate lists (R * k <= 256): one warp per row holds all values in
// registers and bisects on the key bits (31 steps of compare + popcount).
__global__ void topk_threshold_warp_kernel(const float* __restrict__ vals, float* __restrict__ thr, long long rows, int R,
                                           int k) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int n = R * k;
  unsigned key[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int i = lane + 32 * q;
    key[q] = i < n ? positive_key(__ldg(vals + ((size_t)(i / k) * rows + row) * k + i % k)) : 0u;
  }
  unsigned Tk = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = Tk | (1u << bit);
    int c = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) c += key[q] >= trial ? 1 : 0;
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) Tk = trial;
  }
  if (lane == 0) thr[row] = __uint_as_float(Tk);
}

// Keep the local candidates at or above the exchanged threshold (ties are all kept), move them to
// the front of the row's slots, clear the rest, mark the fired features.  One warp per row.
__global__ void topk_apply_threshold_kernel(int* __restrict__ idx, float* __restrict__ val,
                                            const float* __restrict__ thr, unsigned* __restrict__ fired_bits,
                                            long long rows, int B, int F, int k) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int words = (F + 31) / 32;
  const int l = (int)(row / B);
  const unsigned tk = positive_key(thr[row]);
  int* ir = idx + (size_t)row * k;
  float* vr = val + (size_t)row * k;
  int n_out = 0;
  for (int j0 = 0; j0 < k; j0 += 32) {
    const int j = j0 + lane;
    const float v = j < k ? vr[j] : 0.f;
    const int f = j < k ? ir[j] : 0;
    const bool keep = v > 0.f && positive_key(v) >= tk;
    const unsigned bal = __ballot_sync(0xffffffffu, keep);
    __syncwarp();
    if (keep) {
      const int slot = n_out + __popc(bal & ((1u << lane) - 1u));  // slot <= j: never overtakes the reads
      vr[slot] = v;
      ir[slot] = f;
      if (fired_bits != nullptr && f >= 0 && f < F) atomicOr(fired_bits + (size_t)l * words + f / 32, 1u << (f & 31));
    }
    n_out += __popc(bal);
    __syncwarp();
  }
  for (int j = n_out + lane; j < k; j += 32) vr[j] = 0.f, ir[j] = 0;
}

}  // namespace

}  // namespace clt

using namespace clt;

extern "C" {

int clt_select_topk(const void* z, const float* b_enc, int* idx_out, float* val_out, uint32_t* fired_bits, int B,
                    int L, int F, int k, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0, "select_topk: bad dims B=%d L=%d F=%d", B, L, F);
  CLT_CHECK_ARG(k >= 0 && k <= F, "select_topk: k=%d must be in [0, F=%d]", k, F);
  CLT_CHECK_ARG(z && b_enc && (k == 0 || (idx_out && val_out)), "select_topk: null pointer");
  if (k == 0) return 0;
  const long long rows = (long long)L * B;
  CLT_CHECK_ARG(rows < (1ll << 31), "select_topk: too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  const bool warp_rows = k <= 64 && F % 8 == 0 && F >= 512 && F <= 8192;   // short rows: one warp each
  const unsigned wblocks = (unsigned)((rows + 7) / 8);
  if (!warp_rows && F % 8 == 0 && F >= kStreamMinF && k <= kStreamCap - 256 && L <= 65535 &&
      ((uintptr_t)z | (uintptr_t)b_enc) % 16 == 0) {
    // long rows: one streaming sweep per row.  Rows of up to 8192 columns (a feature shard's slice) stay with
    // the two-sweep warp kernel, whose second sweep comes from L2 and whose per-row bookkeeping is lighter:
    // 0.22 ms against 0.42 ms at 4096 columns, 0.36 against 0.67 ms at 8192 (12 layers x 4000 rows, k = 32)
    dim3 grid((B + kStreamWarps - 1) / kStreamWarps, L);
    if (bf16)
      select_topk_stream_kernel<__nv_bfloat16><<<grid, kStreamWarps * 32, 0, s>>>(
          (const __nv_bfloat16*)z, b_enc, idx_out, val_out, fired_bits, B, F, k);
    else
      select_topk_stream_kernel<float><<<grid, kStreamWarps * 32, 0, s>>>((const float*)z, b_enc, idx_out, val_out,
                                                                          fired_bits, B, F, k);
    CLT_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (bf16) {
    if (warp_rows)
      select_topk_warp_kernel<__nv_bfloat16><<<wblocks, 256, 0, s>>>((const __nv_bfloat16*)z, b_enc, idx_out, val_out,
                                                                      fired_bits, rows, B, F, k);
    else
      select_topk_kernel<__nv_bfloat16><<<(unsigned)rows, kSelThreads, 0, s>>>((const __nv_bfloat16*)z, b_enc, idx_out,
                                                                                 val_out, fired_bits, B, F, k);
  } else {
    if (warp_rows)
      select_topk_warp_kernel<float><<<wblocks, 256, 0, s>>>((const float*)z, b_enc, idx_out, val_out, fired_bits, rows,
                                                              B, F, k);
    else
      select_topk_kernel<float><<<(unsigned)rows, kSelThreads, 0, s>>>((const float*)z, b_enc, idx_out, val_out,
                                                                        fired_bits, B, F, k);
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_dead_compact(const uint8_t* dead, int* dead_list, int* n_dead, int L, int F, clt_stream_t stream) {
  CLT_CHECK_ARG(L > 0 && F > 0 && dead && dead_list && n_dead, "dead_compact: bad arguments");
  dead_compact_kernel<<<L, 1024, 0, (cudaStream_t)stream>>>(dead, dead_list, n_dead, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_select_aux(const void* z, const float* b_enc, const int* dead_list, const int* n_dead, void* a_out,
                   float* cand_out, const float* thr, int mode, int B, int L, int F, int k_aux, int nd_pad, int bf16,
                   const int* row_count, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && nd_pad > 0, "select_aux: bad dims B=%d L=%d F=%d nd_pad=%d", B, L, F, nd_pad);
  CLT_CHECK_ARG(k_aux >= 1, "select_aux: k_aux=%d must be positive", k_aux);
  CLT_CHECK_ARG(mode >= 0 && mode <= 2, "select_aux: unknown mode %d", mode);
  CLT_CHECK_ARG(z && b_enc && dead_list && n_dead, "select_aux: null pointer");
  CLT_CHECK_ARG(mode == 1 ? cand_out != nullptr : a_out != nullptr, "select_aux: missing output for mode %d", mode);
  CLT_CHECK_ARG(mode != 2 || thr != nullptr, "select_aux: mode 2 needs the thresholds");
  const size_t smem = (size_t)nd_pad * sizeof(float);
  CLT_CHECK_ARG(smem <= 200 * 1024, "select_aux: %d dead features per layer exceed the shared-memory candidate buffer",
                nd_pad);
  const long long rows = (long long)L * B;
  cudaStream_t s = (cudaStream_t)stream;
  if (bf16) {
    auto kern = select_aux_kernel<__nv_bfloat16>;
    CLT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, kSelThreads, smem, s>>>((const __nv_bfloat16*)z, b_enc, dead_list, n_dead,
                                                   (__nv_bfloat16*)a_out, cand_out, thr, mode, B, F, k_aux, nd_pad,
                                                   row_count, status);
  } else {
    auto kern = select_aux_kernel<float>;
    CLT_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, kSelThreads, smem, s>>>((const float*)z, b_enc, dead_list, n_dead, (float*)a_out, cand_out,
                                                   thr, mode, B, F, k_aux, nd_pad, row_count, status);
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_aux_count(const void* z, const float* b_enc, const int* dead_list, const int* n_dead, int* cnt, int B, int L,
                  int F, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0, "aux_count: bad dims");
  CLT_CHECK_ARG(z && b_enc && dead_list && n_dead && cnt, "aux_count: null pointer");
  const long long rows = (long long)L * B;
  const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
  if (bf16)
    aux_count_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)z, b_enc, dead_list,
                                                                              n_dead, cnt, rows, B, F);
  else
    aux_count_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)z, b_enc, dead_list, n_dead, cnt,
                                                                     rows, B, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_topk_threshold(const float* vals, float* thr, int64_t rows, int R, int k, clt_stream_t stream) {
  CLT_CHECK_ARG(rows > 0 && R > 0 && k > 0 && rows < (1ll << 31), "topk_threshold: bad dims");
  CLT_CHECK_ARG(vals && thr, "topk_threshold: null pointer");
  if ((long long)R * k <= 256) {
    const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
    topk_threshold_warp_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(vals, thr, rows, R, k);
  } else {
    topk_threshold_kernel<<<(unsigned)rows, kSelThreads, 0, (cudaStream_t)stream>>>(vals, thr, rows, R, k);
  }
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_topk_apply_threshold(int* idx, float* val, const float* thr, uint32_t* fired_bits, int B, int L, int F, int k,
                             clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && k > 0, "topk_apply_threshold: bad dims");
  CLT_CHECK_ARG(idx && val && thr, "topk_apply_threshold: null pointer");
  const long long rows = (long long)L * B;
  const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
  topk_apply_threshold_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(idx, val, thr, fired_bits, rows, B, F, k);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
