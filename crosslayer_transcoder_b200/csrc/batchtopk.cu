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
//   [6] 0 = threshold found, 1 = fewer positives than wanted (keep all), 2 = the guessed floor was too high (retry)
//   [7] guessed floor for the next step's first level: half of this step's threshold (as a key).
//       The first level then histograms only the elements above the floor, which turns it into a pure
//       streaming pass (hardly any shared-memory atomics); if fewer than n_keep elements lie above it,
//       the pick kernel asks for a retry without the floor, which the host has already enqueued
//       (the retry kernels return immediately when no retry is pending).
#include "../../include/clt_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace clt {
namespace {

constexpr int kBins = 2048;
typedef unsigned long long u64;

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
               u64* __restrict__ hist_all, int level, int retry, long long rows_per_group, int B, int F) {
  __shared__ unsigned sh[kBins];
  const int grp = blockIdx.y;
  const u64* state = state_all + 8 * grp;
  // nothing to do: a retry that is not pending, or finer levels after "keep all"
  if (retry ? state[6] != 2 : (level > 0 && state[6] == 1)) return;
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
                               u64* __restrict__ state_all, int level, int retry, u64 n_keep) {
  if (retry ? state_all[8 * blockIdx.x + 6] != 2 : (level > 0 && state_all[8 * blockIdx.x + 6] == 1)) return;
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
      state[6] = floored ? 2 : 1;   // retry without the floor, or (no floor) fewer positives than wanted: keep all
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
      state[6] = 0;
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

// threshold <- (1 - e) threshold + e * (smallest kept value)   (topk.py:94-95)
__global__ void bt_threshold_update_kernel(u64* __restrict__ state, float* __restrict__ threshold, float e,
                                           int groups) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float tmin = __uint_as_float((unsigned)state[8 * g + 2]);  // the threshold value; 0 if nothing was cut
  threshold[g] = (1.f - e) * threshold[g] + e * tmin;
  state[8 * g + 7] = (u64)pos_key(0.5f * tmin);                   // floor of the next step's first pass
}

}  // namespace
}  // namespace clt

using namespace clt;

extern "C" {

int clt_batchtopk_hist(const void* z, const float* b_enc, const uint64_t* state, uint64_t* hist, int level, int retry,
                       int groups, int B, int L, int F, int bf16, clt_stream_t stream) {
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
                                                       level, retry, rows_per_group, B, F);
  else
    bt_hist_kernel<float><<<grid, 256, 0, s>>>((const float*)z, b_enc, (const u64*)state, (u64*)hist, level, retry,
                                               rows_per_group, B, F);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int clt_batchtopk_pick(const uint64_t* hist, const uint64_t* hist_local, uint64_t* state, int level, int retry,
                       int groups, int64_t n_keep, clt_stream_t stream) {
  CLT_CHECK_ARG(hist && state && level >= 0 && level <= 2 && n_keep > 0 && groups > 0, "batchtopk_pick: bad arguments");
  bt_pick_kernel<<<groups, 256, 0, (cudaStream_t)stream>>>((const u64*)hist, (const u64*)hist_local, (u64*)state, level,
                                                           retry, (u64)n_keep);
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

int clt_batchtopk_threshold_update(uint64_t* state, float* threshold, float e, int groups, clt_stream_t stream) {
  CLT_CHECK_ARG(state && threshold && groups > 0, "batchtopk_threshold_update: bad arguments");
  bt_threshold_update_kernel<<<(groups + 63) / 64, 64, 0, (cudaStream_t)stream>>>((u64*)state, threshold, e, groups);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
