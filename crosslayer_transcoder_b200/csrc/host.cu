// Host-side plumbing of the library: error string, device queries, TMA tensor-map
// encoding, and the C entry points that are thin wrappers over elementwise kernels.
#include <cuda.h>
#include <stdarg.h>
#include <string.h>

#include "../../include/clt_b200.h"
#include "common.cuh"
#include "gemm_tc.cuh"
#include "kernels.h"

namespace clt {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }

int device_sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 3-D bf16 tensor map (contiguous axis, rows, stacked matrices) with the 128-byte swizzle.
// K-major operands use one box of 64 x tile_rows; MN-major operands boxes of 64 x 64.
int encode_operand_map(CUtensorMap* map, const TcOperand& o, int tile_rows_if_k_major) {
  EncodeTiledFn fn = encode_fn();
  CLT_CHECK_ARG(fn != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  CLT_CHECK_ARG(((uintptr_t)o.ptr & 15) == 0, "tensor-core operand must be 16-byte aligned");
  CLT_CHECK_ARG(o.row_stride % 8 == 0 && o.z_stride % 8 == 0,
                "tensor-core operand strides must be multiples of 8 elements (row %lld, matrix %lld)", o.row_stride,
                o.z_stride);
  CLT_CHECK_ARG(o.inner > 0 && o.rows > 0 && o.z_count > 0, "empty tensor-core operand");
  cuuint64_t dims[3] = {(cuuint64_t)o.inner, (cuuint64_t)o.rows, (cuuint64_t)o.z_count};
  cuuint64_t strides[2] = {(cuuint64_t)o.row_stride * 2, (cuuint64_t)(o.z_count > 1 ? o.z_stride : o.row_stride * o.rows) * 2};
  if (strides[1] == 0) strides[1] = strides[0];
  cuuint32_t box[3] = {64, (cuuint32_t)(o.mn_major ? 64 : tile_rows_if_k_major), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(o.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CLT_CHECK_ARG(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (inner %lld rows %lld z %lld)", (int)r,
                o.inner, o.rows, o.z_count);
  return 0;
}

}  // namespace tc
}  // namespace clt

using namespace clt;

extern "C" {

int clt_version(void) { return 1; }
const char* clt_last_error(void) { return last_error(); }

int clt_device_check(void) {
  int dev = 0;
  CLT_CHECK_CUDA(cudaGetDevice(&dev));
  int major = 0;
  CLT_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  CLT_CHECK_ARG(major == 10, "this library is built for sm_100a only; device %d has compute capability %d.x", dev,
                major);
  return 0;
}

int clt_prep_input(const void* batch, int in_dtype, const float* mu, const float* sd, void* xn, int bf16, int B, int L,
                   int D, clt_stream_t stream) {
  return prep_input(batch, in_dtype, mu, sd, xn, bf16, B, L, D, 2, (cudaStream_t)stream);
}

int clt_loss_fwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu_out,
                 const float* sd_out, float* acc, int B, int L, int D, clt_stream_t stream) {
  return loss_fwd(recon, aux, batch, in_dtype, mu_out, sd_out, acc, B, L, D, (cudaStream_t)stream);
}

int clt_finalize_loss(const float* mse_acc, const float* enc_acc, float* loss, float* terms, float inv_bld,
                      float lam_over_b, float pal_over_bl, float aux_scale, clt_stream_t stream) {
  return finalize_loss(mse_acc, enc_acc, loss, terms, inv_bld, lam_over_b, pal_over_bl, aux_scale,
                       (cudaStream_t)stream);
}

int clt_loss_bwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu_out,
                 const float* sd_out, const float* gscale, float aux_scale, void* drecon, void* daux, int bf16,
                 float* db_dec, int B, int L, int D, clt_stream_t stream) {
  return loss_bwd(recon, aux, batch, in_dtype, mu_out, sd_out, gscale, aux_scale, drecon, daux, bf16, db_dec, B, L, D,
                  (cudaStream_t)stream);
}

int clt_sum_slots(const void* slots, float* out, int n_slots, int64_t n, int slots_bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(slots && out && n_slots > 0 && n >= 0 && n % (slots_bf16 ? 8 : 4) == 0,
                "sum_slots: bad arguments (n must be a multiple of 4, of 8 for bf16 slots)");
  return sum_slots(slots, out, n_slots, (long long)n, slots_bf16, (cudaStream_t)stream);
}

int clt_loss_bwd_push(const float* recon_own, const float* aux_own, const void* batch, int in_dtype,
                      const float* mu_out, const float* sd_out, const float* gscale, float aux_scale,
                      const uint64_t* drecon_bases, const uint64_t* daux_bases, int n_ranks, int bf16, float* db_dec,
                      int B, int b_lo, int b_cnt, int L, int D, clt_stream_t stream) {
  CLT_CHECK_ARG(recon_own && batch && mu_out && sd_out && drecon_bases && db_dec, "loss_bwd_push: null pointer");
  CLT_CHECK_ARG((aux_own == nullptr) == (daux_bases == nullptr), "loss_bwd_push: aux_own and daux_bases go together");
  CLT_CHECK_ARG(B > 0 && L > 0 && D > 0 && D % 8 == 0, "loss_bwd_push: bad dims B=%d L=%d D=%d (D %% 8 == 0)", B, L, D);
  CLT_CHECK_ARG(b_lo >= 0 && b_cnt >= 0 && b_lo + b_cnt <= B, "loss_bwd_push: rows [%d, %d) outside [0, %d)", b_lo,
                b_lo + b_cnt, B);
  CLT_CHECK_ARG(n_ranks > 0, "loss_bwd_push: n_ranks=%d", n_ranks);
  return loss_bwd_push(recon_own, aux_own, batch, in_dtype, mu_out, sd_out, gscale, aux_scale,
                       reinterpret_cast<const unsigned long long*>(drecon_bases),
                       reinterpret_cast<const unsigned long long*>(daux_bases), n_ranks, bf16, db_dec, B, b_lo, b_cnt,
                       L, D, (cudaStream_t)stream);
}

int clt_act_fwd(const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* feat_out,
                uint32_t* fired_bits, float* loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int L, int F,
                int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(z && b_enc && feat_out && loss_acc, "act_fwd: null pointer");
  return act_fwd(z, b_enc, theta, dec_norm, feat_out, fired_bits, loss_acc, c_sparsity, use_tanh, want_pre, B, L, F,
                 bf16, (cudaStream_t)stream);
}

int clt_act_bwd(const void* g, const void* z, const float* b_enc, const float* theta, const float* dec_norm,
                void* dpre_out, float* dtheta, float* dbenc, float* dnorm, float bandwidth, float lam, float c_sparsity,
                float pal, int use_tanh, const float* gscale, int B, int L, int F, int bf16, clt_stream_t stream) {
  CLT_CHECK_ARG(g && z && b_enc && dpre_out && dbenc, "act_bwd: null pointer");
  return act_bwd(g, z, b_enc, theta, dec_norm, dpre_out, dtheta, dbenc, dnorm, bandwidth, lam, c_sparsity, pal,
                 use_tanh, gscale, B, L, F, bf16, (cudaStream_t)stream);
}

int clt_dec_norms(const float* W_dec, float* out, int L, int F, int D, int crosslayer, clt_stream_t stream) {
  return dec_norms(W_dec, out, L, F, D, crosslayer, (cudaStream_t)stream);
}

int clt_norm_coef(const float* dnorm, const float* norm, float* out, int count, clt_stream_t stream) {
  return norm_coef(dnorm, norm, out, count, (cudaStream_t)stream);
}

int clt_dead_update(int64_t* last_active, uint32_t* fired_bits, uint8_t* dead, int64_t B, int64_t limit, int L, int F,
                    int* dead_count, int* soon_dead, clt_stream_t stream) {
  return dead_update((long long*)last_active, fired_bits, dead, B, limit, L, F, dead_count, soon_dead,
                     (cudaStream_t)stream);
}

int clt_adam_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, int64_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int decoupled, int64_t step, clt_stream_t stream) {
  return adam_step(p, g, m, v, shadow_bf16, n, lr, beta1, beta2, eps, weight_decay, decoupled, step,
                   device_sm_count(), (cudaStream_t)stream);
}

int clt_cast_bf16(const float* src, void* dst, int64_t n, clt_stream_t stream) {
  return cast_bf16(src, dst, n, (cudaStream_t)stream);
}

}  // extern "C"
