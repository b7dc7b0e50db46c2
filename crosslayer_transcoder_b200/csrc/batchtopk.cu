// BatchTopK selection: ONE threshold for the whole batch, all layers and features together
// (reference: crosslayer_transcoder/model/topk.py:76-96 keeps the k*B*L largest of the flattened
// [B*L*F] pre-activations and passes them through a ReLU).
//
// As in the per-row selection only positive values can end up non-zero, so the threshold is the
// n-th largest POSITIVE pre-activation (n = k*B*L; if there are fewer positives, all stay).
// It is found exactly by a three-level radix select on the 31 value bits (11 + 11 + 9): every
// level is one streaming pass that histograms the digit of the elements inside the bucket chosen
// so far (per-CTA shared-memory histograms flushed to a 2048-bin global one), followed by a
// one-CTA kernel that picks the next bucket.  Between the two, feature shards sum their
// histograms (all-reduce of 2048 counters), which makes the threshold global.
// A last pass walks the rows: one CTA per (layer, token) counts the row's survivors, reserves a
// segment of the layer's entry list with one atomic and writes (feature, value, token).
//
// PerLayerBatchTopK (topk.py:99-133) is the same selection run independently per layer: the kernels
// take a number of groups (1 = whole batch, L = one per layer), with one state block and one
// histogram per group.
//
// State block (device memory, 8 x 64-bit words per group):
//   [0] prefix (bits fixed so far)   [1] want (rank of the threshold inside the current bucket)
//   [2] threshold key T (valid after level 2; 0 = keep every positive)
//   [3] ties: number of elements equal to T that are kept (all ranks together)
//   [4] ties_taken (atomic counter of the collecting pass)   [5] local count of elements equal to T
//   [6] low bits: 0 = threshold found, 1 = fewer positives than wanted (keep all), 2 = the guessed floor was
//       too high (retry); bit 4 (value 16): this step's selection runs on full sweeps of z (set by the
//       first pick), clear: it runs on the candidate list
//   [7] guessed floor for the next step: 0.9 of this step's threshold (as a key).
//
// Candidate list (steady state: ONE sweep of z per step instead of five).  The threshold moves little from
// step to step, so the first pass keeps every element at or above the floor — a few times n_keep
// elements — in a compact list (feature, value, row; one segment per row, in a fixed scrambled order), and the
// three radix levels and the final collection read that list instead of z.  Whenever the list cannot be
// trusted — no floor yet, a row or the list overflowed on any rank, fewer than n_keep elements above the
// floor — the first pick sets bit 4 of state[6] and the same step falls back to the full sweeps, which the
// host has already enqueued (kernels of the path not taken return at once).  Feature shards sum an
// "invalid" flag together with the histograms, so all ranks take the same path.
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {
namespace {

constexpr int kBins = 2048;
constexpr int kRowCand = 2048;      // candidates one row may hold (shared memory of the first pass)
typedef unsigned long long u64;

__device__ __forceinline__ unsigned st_code(const u64* st) { return (unsigned)st[6] & 15u; }
__device__ __forceinline__ bool st_full(const u64* st) { return ((unsigned)st[6] & 16u) != 0u; }

template <class T>
__device__ __forceinline__ float ld_f(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p, size_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(__ldg(p + i));
}

__device__ __forceinline__ unsigned pos_key(float v) { return v > 0.f ? __float_as_uint(v) : 0u; }

// 8 consecutive pre-activations (z + b) starting at a multiple of 8
template <class T>
__device__ __forceinline__ void pre8(const T* z, const float* b, int i, float (&o)[8]);
template <>
__device__ __forceinline__ void pre8<__nv_bfloat16>(const __nv_bfloat16* z, const float* b, int i, float (&o)[8]) {
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(z + i));
  const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + i)), b1 = __ldg(reinterpret_cast<const float4*>(b + i) + 1);
  o[0] = __uint_as_float(t.x << 16) + b0.x, o[1] = __uint_as_float(t.x & 0xffff0000u) + b0.y;
  o[2] = __uint_as_float(t.y << 16) + b0.z, o[3] = __uint_as_float(t.y & 0xffff0000u) + b0.w;
  o[4] = __uint_as_float(t.z << 16) + b1.x, o[5] = __uint_as_float(t.z & 0xffff0000u) + b1.y;
  o[6] = __uint_as_float(t.w << 16) + b1.z, o[7] = __uint_as_float(t.w & 0xffff0000u) + b1.w;
}
template <>
__device__ __forceinline__ void pre8<float>(const float* z, const float* b, int i, float (&o)[8]) {
  const float4 z0 = __ldg(reinterpret_cast<const float4*>(z + i)), z1 = __ldg(reinterpret_cast<const float4*>(z + i) + 1);
  const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + i)), b1 = __ldg(reinterpret_cast<const float4*>(b + i) + 1);
  o[0] = z0.x + b0.x, o[1] = z0.y + b0.y, o[2] = z0.z + b0.z, o[3] = z0.w + b0.w;
  o[4] = z1.x + b1.x, o[5] = z1.y + b1.y, o[6] = z1.z + b1.z, o[7] = z1.w + b1.w;
}

__device__ __forceinline__ bool digit_of(unsigned key, int level, unsigned prefix, unsigned& d) {
  if (level == 0) {
    d = key >> 20;
    return true;
  }
  if (level == 1) {
    d = (key >> 9) & 0x7ffu;
    return (key >> 20) == prefix;
  }
  d = key & 0x1ffu;
  return (key >> 9) == prefix;
}

// One streaming pass over z [L, B, F]: histogram of the level's digit.
template <class T>
__global__ void __launch_bounds__(256)
bt_hist_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, const u64* __restrict__ state_all,
               u64* __restrict__ hist_all, const u64* __restrict__ list_invalid, int level, int retry,
               long long rows_per_group, int B, int F) {
  __shared__ unsigned sh[kBins];
  const int grp = blockIdx.y;
  const u64* state = state_all + 8 * grp;
  // nothing to do: a retry that is not pending, or finer levels after "keep all"
  if (retry ? st_code(state) != 2 : (level > 0 && st_code(state) == 1)) return;
  // nothing to do either while the candidate list stands in for z
  if (list_invalid != nullptr && !retry && (level == 0 ? *list_invalid == 0 : !st_full(state))) return;
  for (int i = threadIdx.x; i < kBins; i += blockDim.x) sh[i] = 0u;
  __syncthreads();
  u64* hist = hist_all + (size_t)kBins * grp;
  const unsigned prefix = (unsigned)state[0];
  const unsigned floor_key = (level == 0 && !retry) ? (unsigned)state[7] : 0u;
  const long long row_lo = grp * rows_per_group, rows = row_lo + rows_per_group;
  const bool vec = F % 8 == 0;
  for (long long row = row_lo + blockIdx.x; row < rows; row += gridDim.x) {
    const int l = (int)(row / B);
    const T* zr = z + (size_t)row * F;
    const float* br = b_enc + (size_t)l * F;
    if (vec) {
      for (int f = 8 * threadIdx.x; f < F; f += 8 * blockDim.x) {
        float v[8];
        pre8<T>(zr, br, f, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const unsigned key = pos_key(v[q]);
          unsigned d;
          if (key != 0u && key >= floor_key && digit_of(key, level, prefix, d)) atomicAdd(&sh[d], 1u);
        }
      }
    } else {
      for (int f = threadIdx.x; f < F; f += blockDim.x) {
        const unsigned key = pos_key(ld_f<T>(zr, f) + __ldg(br + f));
        unsigned d;
        if (key != 0u && key >= floor_key && digit_of(key, level, prefix, d)) atomicAdd(&sh[d], 1u);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins; i += blockDim.x)
    if (sh[i] != 0u) atomicAdd(hist + i, (u64)sh[i]);
}

// Pick the bucket of the current level from the (summed) histogram; one CTA of 256 threads.
__global__ void bt_pick_kernel(const u64* __restrict__ hist_all, const u64* __restrict__ hist_local_all,
                               u64* __restrict__ state_all, const u64* __restrict__ list_invalid, int level, int retry,
                               u64 n_keep) {
  if (retry ? st_code(state_all + 8 * blockIdx.x) != 2 : (level > 0 && st_code(state_all + 8 * blockIdx.x) == 1))
    return;
  // bit 4 of state[6]: full sweeps for the rest of this step.  Decided by the first pick: no list (NULL), a
  // list that some rank could not complete, or a floor that proves too high below.
  const u64 full = (level == 0 && !retry) ? ((list_invalid == nullptr || *list_invalid != 0) ? 16u : 0u)
                                          : (state_all[8 * blockIdx.x + 6] & 16u);
  const u64* hist = hist_all + (size_t)kBins * blockIdx.x;
  const u64* hist_local = hist_local_all != nullptr ? hist_local_all + (size_t)kBins * blockIdx.x : nullptr;
  u64* state = state_all + 8 * blockIdx.x;
  __shared__ u64 tot[256];
  __shared__ int sh_digit;
  __shared__ u64 sh_above;
  __shared__ int sh_none;
  const int t = threadIdx.x;
  u64 want = level == 0 ? n_keep : state[1];
  u64 local[8];
  u64 s = 0;
#pragma unroll
  for (int i = 7; i >= 0; --i) {
    s += hist[t * 8 + i];
    local[i] = s;
  }
  tot[t] = s;
  if (t == 0) sh_digit = -1, sh_above = 0, sh_none = 0;
  __syncthreads();
  u64 above = 0;
  for (int j = t + 1; j < 256; ++j) above += tot[j];
  if (level == 0 && t == 0 && above + s < want) sh_none = 1;  // fewer elements than n_keep above the floor
  __syncthreads();
  if (sh_none) {
    if (t == 0) {
      const bool floored = !retry && state[7] != 0;
      state[0] = 0, state[1] = 0, state[2] = 0, state[3] = 0, state[4] = 0, state[5] = 0;
      // retry without the floor (on full sweeps), or (no floor) fewer positives than wanted: keep all
      state[6] = floored ? (2 | 16) : (1 | full);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const u64 gt = above + (i < 7 ? local[i + 1] : 0);
    const u64 ge = above + local[i];
    if (gt < want && want <= ge) {
      sh_digit = t * 8 + i;
      sh_above = gt;
    }
  }
  __syncthreads();
  if (t == 0) {
    const unsigned d = (unsigned)sh_digit;
    const unsigned prefix = (unsigned)state[0];
    const u64 left = want - sh_above;
    state[1] = left;
    if (level == 0) {
      state[0] = d;
      state[6] = full;
    } else if (level == 1) {
      state[0] = (u64)((prefix << 11) | d);
    } else {
      state[2] = (u64)((prefix << 9) | d);                // threshold key
      state[3] = left;                                     // elements equal to it that are kept, all ranks
      state[4] = 0;
      state[5] = hist_local != nullptr ? hist_local[d] : hist[d];   // this rank's elements equal to it
    }
  }
}

// Collect the survivors row by row.  One CTA per (layer, token) row:
//   sweep 1 counts the row's elements above T (plus ties while the quota lasts), one atomic on the
//   layer's fill counter reserves the row's segment, sweep 2 writes (feature, value, token).
template <class T>
__global__ void __launch_bounds__(256)
bt_collect_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, u64* __restrict__ state_all,
                  const long long* __restrict__ tie_quota_all, int* __restrict__ idx, float* __restrict__ val,
                  int* __restrict__ etok, int* __restrict__ row_start, int* __restrict__ row_cnt,
                  int* __restrict__ layer_fill, unsigned* __restrict__ fired_bits, int B, int F, long long npl,
                  int groups, int* status) {
  const long long row = blockIdx.x;
  const int l = (int)(row / B), b = (int)(row % B);
  u64* state = state_all + 8 * (groups > 1 ? l : 0);
  if (!st_full(state)) return;              // this step's survivors come from the candidate list
  const long long* tie_quota = tie_quota_all != nullptr ? tie_quota_all + (groups > 1 ? l : 0) : nullptr;
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  const unsigned Tk = (unsigned)state[2];
  const long long quota = tie_quota != nullptr ? *tie_quota : (long long)state[3];
  const int words = (F + 31) / 32;
  __shared__ int n_row, base, cursor;
  if (threadIdx.x == 0) n_row = 0, cursor = 0;
  __syncthreads();
  // sweep 1: count the row's elements above the threshold and those equal to it
  const bool vec = F % 8 == 0;
  __shared__ int n_tie;
  if (threadIdx.x == 0) n_tie = 0;
  __syncthreads();
  int mine = 0, mine_tie = 0;
  if (vec) {
    for (int f = 8 * threadIdx.x; f < F; f += 8 * blockDim.x) {
      float v[8];
      pre8<T>(zr, br, f, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const unsigned key = pos_key(v[q]);
        mine += key > Tk ? 1 : 0;
        mine_tie += (key != 0u && key == Tk) ? 1 : 0;
      }
    }
  } else {
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
      const unsigned key = pos_key(ld_f<T>(zr, f) + __ldg(br + f));
      mine += key > Tk ? 1 : 0;
      mine_tie += (key != 0u && key == Tk) ? 1 : 0;
    }
  }
  if (mine) atomicAdd(&n_row, mine);
  if (mine_tie && Tk != 0u && quota > 0) atomicAdd(&n_tie, mine_tie);
  __syncthreads();
  __shared__ int tie_take;
  if (threadIdx.x == 0) {
    int take = 0;
    if (n_tie > 0) {
      const u64 before = atomicAdd(&state[4], (u64)n_tie);
      const long long room = quota - (long long)before;
      take = room <= 0 ? 0 : (room < n_tie ? (int)room : n_tie);
    }
    tie_take = take;
    const int total = n_row + take;
    int start = 0;
    if (total > 0) {
      start = atomicAdd(layer_fill + l, total);
      if ((long long)start + total > npl) {
        report_status(status, kOverflow);
        start = -1;
      }
    }
    base = start;
    row_start[row] = start < 0 ? 0 : start;
    row_cnt[row] = start < 0 ? 0 : total;
    n_tie = 0;  // reused as the running count of ties written
  }
  __syncthreads();
  if (base < 0 || n_row + tie_take == 0) return;
  // sweep 2: write
  const size_t o = (size_t)l * npl + base;
  auto emit = [&](int f, float v) {
    const unsigned key = pos_key(v);
    bool take = key > Tk;
    if (!take && key != 0u && key == Tk && tie_take > 0) take = atomicAdd(&n_tie, 1) < tie_take;
    if (take) {
      const int c = atomicAdd(&cursor, 1);
      idx[o + c] = f;
      val[o + c] = v;
      etok[o + c] = b;
      if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + f / 32, 1u << (f & 31));
    }
  };
  if (vec) {
    for (int f = 8 * threadIdx.x; f < F; f += 8 * blockDim.x) {
      float v[8];
      pre8<T>(zr, br, f, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) emit(f + q, v[q]);
    }
  } else {
    for (int f = threadIdx.x; f < F; f += blockDim.x) emit(f, ld_f<T>(zr, f) + __ldg(br + f));
  }
}

// First pass of the candidate path.  One CTA per (layer, token) row: ONE sweep; every element at or above
// the group's floor goes to shared memory, is put in a fixed order and written as the row's segment of the
// global candidate list (segment reserved with one atomic).  No floor yet, more than kRowCand candidates in
// a row or a full list: *invalid = 1 and the step falls back to the full sweeps.
template <class T>
__global__ void __launch_bounds__(256)
bt_candidates_kernel(const T* __restrict__ z, const float* __restrict__ b_enc, const u64* __restrict__ state_all,
                     int* __restrict__ cand_feat, float* __restrict__ cand_val, int* __restrict__ cand_row,
                     int* __restrict__ cand_fill, int* __restrict__ cand_row_start, int* __restrict__ cand_row_cnt,
                     u64* __restrict__ invalid, int B, int F, int groups, long long cap) {
  __shared__ int s_feat[kRowCand];
  __shared__ float s_val[kRowCand];
  __shared__ int s_cnt, s_base;
  const long long row = blockIdx.x;
  const int l = (int)(row / B);
  const u64* state = state_all + 8 * (groups > 1 ? l : 0);
  const unsigned floor_key = (unsigned)state[7];
  if (floor_key == 0u) {                    // no guess yet (first step, or nothing was cut last step)
    if (threadIdx.x == 0) {
      *invalid = 1;
      cand_row_cnt[row] = 0;
    }
    return;
  }
  const float floor_v = __uint_as_float(floor_key);
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  const T* zr = z + (size_t)row * F;
  const float* br = b_enc + (size_t)l * F;
  auto offer = [&](int f, float v) {
    if (v >= floor_v) {
      const int c = atomicAdd(&s_cnt, 1);
      if (c < kRowCand) s_feat[c] = f, s_val[c] = v;
    }
  };
  if (F % 8 == 0) {
    for (int f = 8 * threadIdx.x; f < F; f += 8 * blockDim.x) {
      float v[8];
      pre8<T>(zr, br, f, v);
      bool any = false;
#pragma unroll
      for (int q = 0; q < 8; ++q) any |= v[q] >= floor_v;
      if (any) {
#pragma unroll
        for (int q = 0; q < 8; ++q) offer(f + q, v[q]);
      }
    }
  } else {
    for (int f = threadIdx.x; f < F; f += blockDim.x) offer(f, ld_f<T>(zr, f) + __ldg(br + f));
  }
  __syncthreads();
  const int cnt = s_cnt;
  if (cnt > kRowCand) {
    if (threadIdx.x == 0) {
      *invalid = 1;
      cand_row_cnt[row] = 0;
    }
    return;
  }
  if (cnt > 1) {
    // a fixed order unrelated to addresses and values: ascending hash of the feature (bitonic, in shared
    // memory).  Rows in feature order make the warps of the token-major decoder gather sweep the same
    // address range in step, rows in value order make them all start with the most popular features: 3.6 ms
    // either way against 3.2 ms in arrival order on the 16-layer workload.
    const unsigned salt = (unsigned)row * 0x9E3779B1u;
    auto key = [&](int f) -> unsigned long long {
      return f == 0x7fffffff ? (1ull << 32) : (unsigned long long)((unsigned)f * 2654435761u + salt);
    };
    int n2 = 2;
    while (n2 < cnt) n2 <<= 1;
    for (int j = cnt + threadIdx.x; j < n2; j += blockDim.x) s_feat[j] = 0x7fffffff, s_val[j] = 0.f;
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = threadIdx.x; t < (n2 >> 1); t += blockDim.x) {
          const int i = ((t / stride) * (stride << 1)) + (t & (stride - 1)), j = i + stride;
          const bool up = (i & size) == 0;
          const int a = s_feat[i], c = s_feat[j];
          if ((key(a) > key(c)) == up) {
            const float va = s_val[i], vc = s_val[j];
            s_feat[i] = c, s_feat[j] = a, s_val[i] = vc, s_val[j] = va;
          }
        }
        __syncthreads();
      }
    }
  }
  if (threadIdx.x == 0) {
    int base = 0;
    if (cnt > 0) {
      base = atomicAdd(cand_fill, cnt);
      if ((long long)base + cnt > cap) {
        *invalid = 1;
        base = -1;
      }
    }
    s_base = base;
    cand_row_start[row] = base < 0 ? 0 : base;
    cand_row_cnt[row] = base < 0 ? 0 : cnt;
  }
  __syncthreads();
  const int base = s_base;
  if (base < 0) return;
  for (int j = threadIdx.x; j < cnt; j += blockDim.x) {
    cand_feat[base + j] = s_feat[j];
    cand_val[base + j] = s_val[j];
    cand_row[base + j] = (int)row;
  }
}

// Histogram of one level's digit over the candidate list (the list stands in for z: every element that
// can matter at any level lies at or above the floor).  Runs only while the list is trusted: at level 0 by
// this rank's own flag (the pick then looks at the flag summed over the ranks), afterwards by bit 4 of the
// group's state.
__global__ void __launch_bounds__(256)
bt_list_hist_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_row,
                    const int* __restrict__ cand_fill, const u64* __restrict__ state_all, u64* __restrict__ hist_all,
                    const u64* __restrict__ invalid_local, int level, int groups, int B, long long cap) {
  __shared__ unsigned sh[kBins];
  if (level == 0 && *invalid_local != 0) return;
  if (groups == 1) {
    if (level > 0 && (st_full(state_all) || st_code(state_all) == 1)) return;
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) sh[i] = 0u;
    __syncthreads();
  }
  long long n = *cand_fill;
  if (n > cap) n = cap;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned key = pos_key(cand_val[i]);
    const int grp = groups > 1 ? cand_row[i] / B : 0;
    const u64* state = state_all + 8 * grp;
    if (groups > 1 && level > 0 && (st_full(state) || st_code(state) == 1)) continue;
    unsigned d;
    if (key != 0u && digit_of(key, level, (unsigned)state[0], d)) {
      if (groups == 1) atomicAdd(&sh[d], 1u);
      else atomicAdd(hist_all + (size_t)kBins * grp + d, (u64)1);
    }
  }
  if (groups == 1) {
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x)
      if (sh[i] != 0u) atomicAdd(hist_all + i, (u64)sh[i]);
  }
}

// Survivors from the candidate list.  One warp per (layer, token) row: the row's candidates (in their
// fixed order) above the threshold, plus ties while the quota lasts, are written in order as the row's segment
// of the layer's entry list.  Same outputs as bt_collect_kernel.
__global__ void __launch_bounds__(256)
bt_filter_kernel(const int* __restrict__ cand_feat, const float* __restrict__ cand_val,
                 const int* __restrict__ cand_row_start, const int* __restrict__ cand_row_cnt,
                 u64* __restrict__ state_all, const long long* __restrict__ tie_quota_all, int* __restrict__ idx,
                 float* __restrict__ val, int* __restrict__ etok, int* __restrict__ row_start,
                 int* __restrict__ row_cnt, int* __restrict__ layer_fill, unsigned* __restrict__ fired_bits,
                 long long rows, int B, int F, long long npl, int groups, int* status) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int l = (int)(row / B), b = (int)(row % B);
  u64* state = state_all + 8 * (groups > 1 ? l : 0);
  if (st_full(state)) return;               // this step's survivors come from the sweeps of z
  const long long* tie_quota = tie_quota_all != nullptr ? tie_quota_all + (groups > 1 ? l : 0) : nullptr;
  const unsigned Tk = (unsigned)state[2];
  const long long quota = tie_quota != nullptr ? *tie_quota : (long long)state[3];
  const int cs = cand_row_start[row], cc = cand_row_cnt[row];
  int n_gt = 0, n_tie = 0;
  for (int j = lane; j < cc; j += 32) {
    const unsigned key = pos_key(cand_val[cs + j]);
    n_gt += key > Tk ? 1 : 0;
    n_tie += (key == Tk && key != 0u) ? 1 : 0;
  }
  n_gt = __reduce_add_sync(0xffffffffu, n_gt);
  n_tie = __reduce_add_sync(0xffffffffu, n_tie);
  if (Tk == 0u || quota <= 0) n_tie = 0;
  int take = 0, start = 0;
  if (lane == 0) {
    if (n_tie > 0) {
      const u64 before = atomicAdd(&state[4], (u64)n_tie);
      const long long room = quota - (long long)before;
      take = room <= 0 ? 0 : (room < n_tie ? (int)room : n_tie);
    }
    const int total = n_gt + take;
    if (total > 0) {
      start = atomicAdd(layer_fill + l, total);
      if ((long long)start + total > npl) {
        report_status(status, kOverflow);
        start = -1;
      }
    }
    row_start[row] = start < 0 ? 0 : start;
    row_cnt[row] = start < 0 ? 0 : total;
  }
  take = __shfl_sync(0xffffffffu, take, 0);
  start = __shfl_sync(0xffffffffu, start, 0);
  if (start < 0 || n_gt + take == 0) return;
  const size_t o = (size_t)l * npl + start;
  const int words = (F + 31) / 32;
  int written = 0, ties_seen = 0;
  for (int j0 = 0; j0 < cc; j0 += 32) {
    const int j = j0 + lane;
    const float v = j < cc ? cand_val[cs + j] : 0.f;
    const int f = j < cc ? cand_feat[cs + j] : 0;
    const unsigned key = pos_key(v);
    const bool tie = key == Tk && key != 0u && take > 0;
    const unsigned tb = __ballot_sync(0xffffffffu, tie);
    const bool keep = key > Tk || (tie && ties_seen + __popc(tb & ((1u << lane) - 1u)) < take);
    const unsigned kb = __ballot_sync(0xffffffffu, keep);
    if (keep) {
      const size_t c = o + written + __popc(kb & ((1u << lane) - 1u));
      idx[c] = f;
      val[c] = v;
      etok[c] = b;
      if (fired_bits != nullptr) atomicOr(fired_bits + (size_t)l * words + f / 32, 1u << (f & 31));
    }
    written += __popc(kb);
    ties_seen += __popc(tb);
  }
}

// threshold <- (1 - e) threshold + e * (smallest kept value)   (topk.py:94-95)
__global__ void bt_threshold_update_kernel(u64* __restrict__ state, float* __restrict__ threshold, float e,
                                           int groups) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float tmin = __uint_as_float((unsigned)state[8 * g + 2]);  // the threshold value; 0 if nothing was cut
  threshold[g] = (1.f - e) * threshold[g] + e * tmin;
  state[8 * g + 7] = (u64)pos_key(0.9f * tmin);                   // floor of the next step's first pass
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_batchtopk_hist(const void* z, const float* b_enc, const uint64_t* state, uint64_t* hist,
                       const uint64_t* list_invalid, int level, int retry, int groups, int B, int L, int F, int bf16,
                       clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && level >= 0 && level <= 2, "batchtopk_hist: bad arguments");
  CLT_CHECK_ARG(groups == 1 || groups == L, "batchtopk_hist: groups must be 1 (whole batch) or L (per layer)");
  CLT_CHECK_ARG(z && b_enc && state && hist, "batchtopk_hist: null pointer");
  CLT_CHECK_ARG(!retry || level == 0, "batchtopk_hist: only the first level is retried");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(hist, 0, sizeof(u64) * kBins * groups, s));
  const long long rows_per_group = (long long)L * B / groups;
  const long long want = (long long)device_sm_count() * 8 / groups + 1;
  dim3 grid((unsigned)(rows_per_group < want ? rows_per_group : want), groups);
  if (bf16)
    bt_hist_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)z, b_enc, (const u64*)state, (u64*)hist,
                                                       (const u64*)list_invalid, level, retry, rows_per_group, B, F);
  else
    bt_hist_kernel<float><<<grid, 256, 0, s>>>((const float*)z, b_enc, (const u64*)state, (u64*)hist,
                                               (const u64*)list_invalid, level, retry, rows_per_group, B, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_pick(const uint64_t* hist, const uint64_t* hist_local, uint64_t* state, const uint64_t* list_invalid,
                       int level, int retry, int groups, int64_t n_keep, clt_stream_t stream) {
  CLT_CHECK_ARG(hist && state && level >= 0 && level <= 2 && n_keep > 0 && groups > 0, "batchtopk_pick: bad arguments");
  bt_pick_kernel<<<groups, 256, 0, (cudaStream_t)stream>>>((const u64*)hist, (const u64*)hist_local, (u64*)state,
                                                           (const u64*)list_invalid, level, retry, (u64)n_keep);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_collect(const void* z, const float* b_enc, uint64_t* state, const int64_t* tie_quota, int* idx,
                          float* val, int* etok, int* row_start, int* row_cnt, int* layer_fill, uint32_t* fired_bits,
                          int groups, int B, int L, int F, int64_t npl, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && npl > 0 && npl < (1ll << 31), "batchtopk_collect: bad dims");
  CLT_CHECK_ARG(groups == 1 || groups == L, "batchtopk_collect: groups must be 1 or L");
  CLT_CHECK_ARG(z && b_enc && state && idx && val && etok && row_start && row_cnt && layer_fill,
                "batchtopk_collect: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(layer_fill, 0, sizeof(int) * L, s));
  CLT_CHECK_CUDA(cudaMemsetAsync(val, 0, sizeof(float) * (size_t)L * npl, s));
  const long long rows = (long long)L * B;
  CLT_CHECK_ARG(rows < (1ll << 31), "batchtopk_collect: too many rows");
  if (bf16)
    bt_collect_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>(
        (const __nv_bfloat16*)z, b_enc, (u64*)state, (const long long*)tie_quota, idx, val, etok, row_start, row_cnt,
        layer_fill, fired_bits, B, F, npl, groups, status);
  else
    bt_collect_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)z, b_enc, (u64*)state,
                                                            (const long long*)tie_quota, idx, val, etok, row_start,
                                                            row_cnt, layer_fill, fired_bits, B, F, npl, groups, status);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_candidates(const void* z, const float* b_enc, const uint64_t* state, int* cand_feat, float* cand_val,
                             int* cand_row, int* cand_fill, int* cand_row_start, int* cand_row_cnt,
                             uint64_t* list_invalid, int groups, int B, int L, int F, int64_t cap, int bf16,
                             clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && cap > 0 && cap < (1ll << 31), "batchtopk_candidates: bad dims");
  CLT_CHECK_ARG(groups == 1 || groups == L, "batchtopk_candidates: groups must be 1 or L");
  CLT_CHECK_ARG(z && b_enc && state && cand_feat && cand_val && cand_row && cand_fill && cand_row_start &&
                    cand_row_cnt && list_invalid,
                "batchtopk_candidates: null pointer");
  const long long rows = (long long)L * B;
  CLT_CHECK_ARG(rows < (1ll << 31), "batchtopk_candidates: too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  CLT_CHECK_CUDA(cudaMemsetAsync(cand_fill, 0, sizeof(int), s));
  CLT_CHECK_CUDA(cudaMemsetAsync(list_invalid, 0, sizeof(u64), s));
  if (bf16)
    bt_candidates_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>(
        (const __nv_bfloat16*)z, b_enc, (const u64*)state, cand_feat, cand_val, cand_row, cand_fill, cand_row_start,
        cand_row_cnt, (u64*)list_invalid, B, F, groups, cap);
  else
    bt_candidates_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)z, b_enc, (const u64*)state, cand_feat,
                                                               cand_val, cand_row, cand_fill, cand_row_start,
                                                               cand_row_cnt, (u64*)list_invalid, B, F, groups, cap);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_hist_list(const float* cand_val, const int* cand_row, const int* cand_fill, const uint64_t* state,
                            uint64_t* hist, const uint64_t* list_invalid, int level, int groups, int B, int64_t cap,
                            clt_stream_t stream) {
  CLT_CHECK_ARG(cand_val && cand_row && cand_fill && state && hist && list_invalid, "batchtopk_hist_list: null pointer");
  CLT_CHECK_ARG(level >= 0 && level <= 2 && groups > 0 && B > 0 && cap > 0, "batchtopk_hist_list: bad arguments");
  bt_list_hist_kernel<<<device_sm_count() * 4, 256, 0, (cudaStream_t)stream>>>(
      cand_val, cand_row, cand_fill, (const u64*)state, (u64*)hist, (const u64*)list_invalid, level, groups, B, cap);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_filter(const int* cand_feat, const float* cand_val, const int* cand_row_start,
                         const int* cand_row_cnt, uint64_t* state, const int64_t* tie_quota, int* idx, float* val,
                         int* etok, int* row_start, int* row_cnt, int* layer_fill, uint32_t* fired_bits, int groups,
                         int B, int L, int F, int64_t npl, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(B > 0 && L > 0 && F > 0 && npl > 0 && npl < (1ll << 31), "batchtopk_filter: bad dims");
  CLT_CHECK_ARG(groups == 1 || groups == L, "batchtopk_filter: groups must be 1 or L");
  CLT_CHECK_ARG(cand_feat && cand_val && cand_row_start && cand_row_cnt && state && idx && val && etok && row_start &&
                    row_cnt && layer_fill,
                "batchtopk_filter: null pointer");
  const long long rows = (long long)L * B;
  bt_filter_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      cand_feat, cand_val, cand_row_start, cand_row_cnt, (u64*)state, (const long long*)tie_quota, idx, val, etok,
      row_start, row_cnt, layer_fill, fired_bits, rows, B, F, npl, groups, status);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_threshold_update(uint64_t* state, float* threshold, float e, int groups, clt_stream_t stream) {
  CLT_CHECK_ARG(state && threshold && groups > 0, "batchtopk_threshold_update: bad arguments");
  bt_threshold_update_kernel<<<(groups + 63) / 64, 64, 0, (cudaStream_t)stream>>>((u64*)state, threshold, e, groups);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
