// fp32 contraction on the CUDA cores, for the fp32 configuration whose parity
// bar (1e-4 relative) a single-pass tensor-core format cannot meet.
//
// One CTA of 128 threads computes a 128 x 64 output tile.  Thread t owns row t
// of the tile and all 64 columns (64 accumulators): the A value is private to
// the thread, the B values are shared-memory broadcasts.  That is the same
// accumulator shape the tcgen05 kernel reads out of tensor memory, so both
// kernels share their epilogue functors.
#pragma once

#include "epilogues.cuh"
#include "gemm.cuh"

namespace clt {

struct SimtOperands {
  const float* A;
  const float* B;
  // element strides: A(za, m, k) = A[za*sAz + m*sAm + k*sAk], B(zb, k, n) = B[zb*sBz + k*sBk + n*sBn]
  long long sAz, sAm, sAk;
  long long sBz, sBk, sBn;
};

constexpr int kSimtBM = 128, kSimtBN = 64, kSimtBK = 16;

template <class Epi>
__global__ void __launch_bounds__(128) gemm_simt_kernel(GemmGeom g, SimtOperands op, typename Epi::Params ep) {
  __shared__ float As[kSimtBK][kSimtBM + 4];
  __shared__ __align__(16) float Bs[kSimtBK][kSimtBN];

  const int tid = threadIdx.x;
  const int z = slab_of_rank(g, blockIdx.z);
  const int m0 = blockIdx.y * kSimtBM;
  const int n0 = blockIdx.x * kSimtBN;
  const int row = m0 + tid;
  const bool row_ok = row < g.M;

  float acc[kSimtBN];
#pragma unroll
  for (int i = 0; i < kSimtBN; ++i) acc[i] = 0.f;

  const int nseg = seg_count(g, z);
  for (int j = 0; j < nseg; ++j) {
    int za, zb;
    seg_index(g, z, j, za, zb);
    const float* Ap = op.A + (long long)za * op.sAz;
    const float* Bp = op.B + (long long)zb * op.sBz;
    for (int k0 = 0; k0 < g.Kseg; k0 += kSimtBK) {
      // A tile: every thread fetches the 16 k-values of its own row
#pragma unroll
      for (int kk = 0; kk < kSimtBK; ++kk) {
        const int k = k0 + kk;
        As[kk][tid] = (row_ok && k < g.Kseg) ? __ldg(Ap + (long long)row * op.sAm + (long long)k * op.sAk) : 0.f;
      }
      // B tile: 16 x 64 values, 8 per thread; consecutive threads along the contiguous axis
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + 128 * i;
        int kk, nn;
        if (op.sBn == 1) {
          nn = e % kSimtBN, kk = e / kSimtBN;
        } else {
          kk = e % kSimtBK, nn = e / kSimtBK;
        }
        const int k = k0 + kk, n = n0 + nn;
        Bs[kk][nn] = (k < g.Kseg && n < g.N) ? __ldg(Bp + (long long)k * op.sBk + (long long)n * op.sBn) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kSimtBK; ++kk) {
        const float a = As[kk][tid];
#pragma unroll
        for (int i = 0; i < kSimtBN / 4; ++i) {
          const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][4 * i]);
          acc[4 * i + 0] = fmaf(a, b.x, acc[4 * i + 0]);
          acc[4 * i + 1] = fmaf(a, b.y, acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(a, b.z, acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(a, b.w, acc[4 * i + 3]);
        }
      }
      __syncthreads();
    }
  }

  // per-column parameters of this tile, staged once and read as broadcasts
  constexpr int kCols = Epi::kColArrays > 0 ? Epi::kColArrays : 1;
  __shared__ __align__(16) float colp[kCols][kSimtBN];
  if (Epi::kColArrays > 0) {
    for (int e = tid; e < Epi::kColArrays * kSimtBN; e += 128) {
      const int arr = e / kSimtBN, j = e % kSimtBN;
      colp[arr][j] = (n0 + j < g.N) ? Epi::col_value(ep, arr, z, n0 + j, g.N) : 0.f;
    }
    __syncthreads();
  }
  __shared__ __align__(16) unsigned char stage[4][epi::kStageBytes];
  typename Epi::State st;
  Epi::init(st);
#pragma unroll
  for (int c = 0; c < kSimtBN / 32; ++c) {
    if (n0 + 32 * c < g.N) {  // uniform over the CTA
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = acc[32 * c + i];
      Epi::template apply<kSimtBN>(ep, st, z, row, row_ok, n0 + 32 * c, g.M, g.N, v, &colp[0][32 * c],
                                   stage[tid >> 5]);
    }
  }
  Epi::finish(ep, st);
}

template <class Epi>
int launch_gemm_simt(const GemmGeom& g, const SimtOperands& op, const typename Epi::Params& ep, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.nz <= 0) return 0;
  dim3 grid((g.N + kSimtBN - 1) / kSimtBN, (g.M + kSimtBM - 1) / kSimtBM, g.nz);
  CLT_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "gemm_simt: grid too large (M=%d nz=%d)", g.M, g.nz);
  gemm_simt_kernel<Epi><<<grid, 128, 0, stream>>>(g, op, ep);
  CLT_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace clt
