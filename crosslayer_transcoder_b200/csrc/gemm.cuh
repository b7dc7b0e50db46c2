// Geometry shared by the two contraction kernels (fp32 SIMT and bf16 tcgen05).
//
// Every contraction of the training step is one launch over a set of
// independent output slabs z = 0..nz-1, each of shape [M, N].  A slab's
// contraction runs over one or more K-segments; segment j of slab z reads
// A-matrix number za(z, j) and B-matrix number zb(z, j) out of stacked
// operands.  The four addressing modes are
//
//   kBatched   z = layer l            : 1 segment,  za = zb = z
//                (encoder forward, per-layer decoder, encoder weight gradient)
//   kDecFwd    z = target layer t     : t+1 segments, segment j = source layer j:
//                za = j (features of layer j), zb = pair(t, j)
//   kDecDFeat  z = source layer s     : L-s segments, segment j = target t = s+j:
//                za = t (reconstruction gradient of layer t), zb = pair(t, s)
//   kDecDW     z = pair(t, s)         : 1 segment, za = s (features), zb = t
//                (reconstruction gradient)
//
// pair(t, s) = t (t+1)/2 + s is the position of decoder block (source s ->
// target t) in the flat [P, F, D] decoder buffer.
#pragma once

#include "common.cuh"

namespace clt {

enum GemmMode : int { kBatched = 0, kDecFwd = 1, kDecDFeat = 2, kDecDW = 3 };

struct GemmGeom {
  int mode;
  int M, N, Kseg;  // slab shape and the length of one K-segment
  int L;           // number of layers (crosslayer modes)
  int nz;          // number of output slabs
};

__host__ __device__ inline int pair_index(int t, int s) { return t * (t + 1) / 2 + s; }

__host__ __device__ inline void pair_split(int p, int& t, int& s) {
  int tt = 0;
  while ((tt + 1) * (tt + 2) / 2 <= p) ++tt;
  t = tt;
  s = p - tt * (tt + 1) / 2;
}

// Slabs are visited longest-first so that a static round-robin over CTAs ends evenly.
__host__ __device__ inline int slab_of_rank(const GemmGeom& g, int rank) {
  return g.mode == kDecFwd ? g.nz - 1 - rank : rank;
}

__host__ __device__ inline int seg_count(const GemmGeom& g, int z) {
  if (g.mode == kDecFwd) return z + 1;
  if (g.mode == kDecDFeat) return g.L - z;
  return 1;
}

__host__ __device__ inline void seg_index(const GemmGeom& g, int z, int j, int& za, int& zb) {
  switch (g.mode) {
    case kDecFwd:
      za = j;
      zb = pair_index(z, j);
      break;
    case kDecDFeat:
      za = z + j;
      zb = pair_index(z + j, z);
      break;
    case kDecDW: {
      int t, s;
      pair_split(z, t, s);
      za = s;
      zb = t;
      break;
    }
    default:
      za = z;
      zb = z;
  }
}

}  // namespace clt
