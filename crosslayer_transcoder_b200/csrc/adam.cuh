// The Adam / AdamW update of torch.optim.Adam, shared by the plain optimizer kernel and by the
// decoder backward that applies the update to each row as soon as its gradient is complete.
#pragma once

#include <math.h>

#include "common.cuh"

namespace clt {

struct AdamScalars {
  float lr, beta1, beta2, eps, inv_bc1, inv_sqrt_bc2, weight_decay;
  int decoupled;
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamScalars& a) {
  if (a.weight_decay != 0.f) {
    if (a.decoupled)
      p *= 1.f - a.lr * a.weight_decay;
    else
      g = fmaf(a.weight_decay, p, g);
  }
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) * a.inv_sqrt_bc2 + a.eps;
  p -= (a.lr * a.inv_bc1) * (m / denom);
}

__device__ __forceinline__ float sqrt_approx(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// adam_one with approximate square root and division: the relative error of about 2^-22 on a step of at
// most lr is far below the rounding of the fp32 parameter itself
__device__ __forceinline__ void adam_fast(float& p, float g, float& m, float& v, const AdamScalars& a) {
  if (a.weight_decay != 0.f) {
    if (a.decoupled)
      p *= 1.f - a.lr * a.weight_decay;
    else
      g = fmaf(a.weight_decay, p, g);
  }
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = fmaf(sqrt_approx(v), a.inv_sqrt_bc2, a.eps);
  p = fmaf(-(a.lr * a.inv_bc1), __fdividef(m, denom), p);
}

inline AdamScalars make_adam_scalars(float lr, float beta1, float beta2, float eps, float weight_decay, int decoupled,
                                     long long step) {
  AdamScalars a;
  a.lr = lr, a.beta1 = beta1, a.beta2 = beta2, a.eps = eps, a.weight_decay = weight_decay, a.decoupled = decoupled;
  const double bc1 = 1.0 - pow((double)beta1, (double)step);
  const double bc2 = 1.0 - pow((double)beta2, (double)step);
  a.inv_bc1 = (float)(1.0 / bc1);
  a.inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
  return a;
}

}  // namespace clt
