// C entry points of the dense contractions.  Each builds the slab geometry and the
// operand descriptions and dispatches to the fp32 CUDA-core kernel (bf16 == 0) or the
// bf16 tcgen05 kernel (bf16 == 1) with the epilogue that fuses the rest of the op.
#include "../../include/clt_b200.h"
#include "epilogues.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "kernels.h"

using namespace clt;
typedef __nv_bfloat16 bf16_t;

namespace {

// One stacked operand described once for both kernels.
//   k_contig = 1: matrix z is [rows_mn, K] with K contiguous   (K-major)
//   k_contig = 0: matrix z is [K, rows_mn] with MN contiguous  (MN-major)
struct Operand {
  const void* ptr;
  int k_contig;
  long long mn, k, z_count;
};

tc::TcOperand tc_operand(const Operand& o) {
  tc::TcOperand t;
  t.ptr = o.ptr;
  t.mn_major = o.k_contig ? 0 : 1;
  t.inner = o.k_contig ? o.k : o.mn;
  t.rows = o.k_contig ? o.mn : o.k;
  t.row_stride = t.inner;
  t.z_count = o.z_count;
  t.z_stride = o.mn * o.k;
  return t;
}

SimtOperands simt_operands(const Operand& a, const Operand& b) {
  SimtOperands s;
  s.A = (const float*)a.ptr;
  s.B = (const float*)b.ptr;
  s.sAz = a.mn * a.k;
  s.sAm = a.k_contig ? a.k : 1;
  s.sAk = a.k_contig ? 1 : a.mn;
  s.sBz = b.mn * b.k;
  s.sBn = b.k_contig ? b.k : 1;
  s.sBk = b.k_contig ? 1 : b.mn;
  return s;
}

template <class EpiF32, class EpiBf16>
int run_gemm(const GemmGeom& g, const Operand& a, const Operand& b, const typename EpiF32::Params& p32,
             const typename EpiBf16::Params& p16, int bf16, int* status, cudaStream_t stream) {
  if (bf16) {
    CLT_CHECK_ARG(status != nullptr, "the tensor-core path needs a device status word");
    return tc::launch_gemm_tc<EpiBf16>(g, tc_operand(a), tc_operand(b), p16, status, device_sm_count(), stream);
  }
  return launch_gemm_simt<EpiF32>(g, simt_operands(a, b), p32, stream);
}

bool dims_ok(int B, int L, int D, int F) { return B > 0 && L > 0 && D > 0 && F > 0; }

}  // namespace

extern "C" {

int clt_encoder_fwd_act(const void* xn, const void* W_enc, const float* b_enc, const float* theta,
                        const float* dec_norm, void* z_out, void* feat_out, uint32_t* fired_bits, float* loss_acc,
                        float c_sparsity, int use_tanh, int want_pre, int B, int L, int D, int F, int bf16,
                        int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "encoder_fwd_act: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(xn && W_enc && b_enc && z_out && feat_out && loss_acc, "encoder_fwd_act: null pointer");
  GemmGeom g{kBatched, B, F, D, L, L};
  Operand a{xn, 1, B, D, L}, b{W_enc, 0, F, D, L};
  epi::EncJumpReLU<float>::Params p32{b_enc, theta, dec_norm, (float*)z_out, (float*)feat_out, fired_bits, loss_acc,
                                      c_sparsity, use_tanh, want_pre};
  epi::EncJumpReLU<bf16_t>::Params p16{b_enc, theta, dec_norm, (bf16_t*)z_out, (bf16_t*)feat_out, fired_bits,
                                       loss_acc, c_sparsity, use_tanh, want_pre};
  return run_gemm<epi::EncJumpReLU<float>, epi::EncJumpReLU<bf16_t>>(g, a, b, p32, p16, bf16, status,
                                                                      (cudaStream_t)stream);
}

int clt_encoder_fwd_store(const void* xn, const void* W_enc, void* z_out, int B, int L, int D, int F, int bf16,
                          int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "encoder_fwd_store: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(xn && W_enc && z_out, "encoder_fwd_store: null pointer");
  GemmGeom g{kBatched, B, F, D, L, L};
  Operand a{xn, 1, B, D, L}, b{W_enc, 0, F, D, L};
  epi::StoreZ<float>::Params p32{(float*)z_out};
  epi::StoreZ<bf16_t>::Params p16{(bf16_t*)z_out};
  return run_gemm<epi::StoreZ<float>, epi::StoreZ<bf16_t>>(g, a, b, p32, p16, bf16, status, (cudaStream_t)stream);
}

int clt_decoder_dense_fwd(const void* feat, const void* W_dec, const float* b_dec, float* recon, int B, int L, int D,
                          int F, int crosslayer, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "decoder_dense_fwd: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(feat && W_dec && recon, "decoder_dense_fwd: null pointer");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  GemmGeom g{crosslayer ? kDecFwd : kBatched, B, D, F, L, L};
  Operand a{feat, 1, B, F, L}, b{W_dec, 0, D, F, P};
  epi::DecOut::Params p{recon, b_dec, (long long)L * D, (long long)D};
  return run_gemm<epi::DecOut, epi::DecOut>(g, a, b, p, p, bf16, status, (cudaStream_t)stream);
}

int clt_decoder_dense_fwd_push(const void* feat, const void* W_dec, const float* b_dec, const uint64_t* rank_bases,
                               int rows_per_rank, int n_ranks, int my_slot, int slot_bf16, int B, int L, int D, int F,
                               int crosslayer, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "decoder_dense_fwd_push: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(feat && W_dec && rank_bases, "decoder_dense_fwd_push: null pointer");
  CLT_CHECK_ARG(n_ranks > 0 && n_ranks <= epi::kMaxPushRanks && rows_per_rank > 0 &&
                    (long long)rows_per_rank * n_ranks >= B,
                "decoder_dense_fwd_push: %d ranks x %d rows do not cover B=%d (at most %d ranks)", n_ranks,
                rows_per_rank, B, epi::kMaxPushRanks);
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  GemmGeom g{crosslayer ? kDecFwd : kBatched, B, D, F, L, L};
  Operand a{feat, 1, B, F, L}, b{W_dec, 0, D, F, P};
  epi::DecOutPush::Params p;
  for (int r = 0; r < epi::kMaxPushRanks; ++r) p.bases[r] = r < n_ranks ? (unsigned long long)rank_bases[r] : 0ull;
  p.bias = b_dec;
  p.rows_per_rank = rows_per_rank;
  CLT_CHECK_ARG(my_slot >= 0 && my_slot < n_ranks, "decoder_dense_fwd_push: slot %d of %d", my_slot, n_ranks);
  p.ld = (long long)L * D;
  p.zstride = (long long)D;
  p.slot_offset = (long long)my_slot * rows_per_rank * L * D;
  p.slot_bf16 = slot_bf16 ? 1 : 0;
  return run_gemm<epi::DecOutPush, epi::DecOutPush>(g, a, b, p, p, bf16, status, (cudaStream_t)stream);
}

int clt_decoder_dense_bwd_dfeat(const void* drecon, const void* W_dec, const void* z_in, const float* b_enc,
                                const float* theta, const float* dec_norm, void* dpre_out, float* dtheta, float* dbenc,
                                float* dnorm, float bandwidth, float lam, float c_sparsity, float pal, int use_tanh,
                                const float* gscale, int B, int L, int D, int F, int crosslayer, int bf16, int* status,
                                clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "decoder_dense_bwd_dfeat: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(drecon && W_dec && z_in && b_enc && dpre_out && dbenc, "decoder_dense_bwd_dfeat: null pointer");
  CLT_CHECK_ARG(bandwidth > 0.f, "decoder_dense_bwd_dfeat: bandwidth must be positive");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  GemmGeom g{crosslayer ? kDecDFeat : kBatched, B, F, D, L, L};
  // A: drecon[t] as [B, D] (K = D contiguous); B: W_dec[p] as [F (N), D (K)], K contiguous
  Operand a{drecon, 1, B, D, L}, b{W_dec, 1, F, D, P};
  epi::DFeatJumpReLU<float>::Params p32{(const float*)z_in, b_enc, theta, dec_norm, (float*)dpre_out, dtheta, dbenc,
                                        dnorm, bandwidth, lam, c_sparsity, pal, use_tanh, gscale};
  epi::DFeatJumpReLU<bf16_t>::Params p16{(const bf16_t*)z_in, b_enc, theta, dec_norm, (bf16_t*)dpre_out, dtheta, dbenc,
                                         dnorm, bandwidth, lam, c_sparsity, pal, use_tanh, gscale};
  return run_gemm<epi::DFeatJumpReLU<float>, epi::DFeatJumpReLU<bf16_t>>(g, a, b, p32, p16, bf16, status,
                                                                          (cudaStream_t)stream);
}

int clt_decoder_dense_bwd_dfeat_raw(const void* drecon, const void* W_dec, void* g_out, int B, int L, int D, int F,
                                    int crosslayer, int bf16, int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "decoder_dense_bwd_dfeat_raw: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(drecon && W_dec && g_out, "decoder_dense_bwd_dfeat_raw: null pointer");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  GemmGeom g{crosslayer ? kDecDFeat : kBatched, B, F, D, L, L};
  Operand a{drecon, 1, B, D, L}, b{W_dec, 1, F, D, P};
  epi::StoreZ<float>::Params p32{(float*)g_out};
  epi::StoreZ<bf16_t>::Params p16{(bf16_t*)g_out};
  return run_gemm<epi::StoreZ<float>, epi::StoreZ<bf16_t>>(g, a, b, p32, p16, bf16, status, (cudaStream_t)stream);
}

int clt_decoder_dense_bwd_dw(const void* feat, const void* drecon, float* dW, const float* rowcoef,
                             const float* W_master, int B, int L, int D, int F, int crosslayer, int bf16, int* status,
                             clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "decoder_dense_bwd_dw: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(feat && drecon && dW, "decoder_dense_bwd_dw: null pointer");
  CLT_CHECK_ARG(rowcoef == nullptr || W_master != nullptr, "decoder_dense_bwd_dw: rowcoef needs the master weights");
  const int P = crosslayer ? L * (L + 1) / 2 : L;
  GemmGeom g{crosslayer ? kDecDW : kBatched, F, D, B, L, P};
  // A: feat[s]^T, stored [B (K), F (M)] with M contiguous; B: drecon[t], stored [B (K), D (N)] with N contiguous
  Operand a{feat, 0, F, B, L}, b{drecon, 0, D, B, L};
  epi::GradOut::Params p{dW, rowcoef, W_master, crosslayer ? 1 : 0};
  return run_gemm<epi::GradOut, epi::GradOut>(g, a, b, p, p, bf16, status, (cudaStream_t)stream);
}

int clt_encoder_dense_bwd_dw(const void* xn, const void* dpre, float* dW, int B, int L, int D, int F, int bf16,
                             int* status, clt_stream_t stream) {
  CLT_CHECK_ARG(dims_ok(B, L, D, F), "encoder_dense_bwd_dw: bad dims B=%d L=%d D=%d F=%d", B, L, D, F);
  CLT_CHECK_ARG(xn && dpre && dW, "encoder_dense_bwd_dw: null pointer");
  GemmGeom g{kBatched, D, F, B, L, L};
  Operand a{xn, 0, D, B, L}, b{dpre, 0, F, B, L};
  epi::GradOut::Params p{dW, nullptr, nullptr, 0};
  return run_gemm<epi::GradOut, epi::GradOut>(g, a, b, p, p, bf16, status, (cudaStream_t)stream);
}

}  // extern "C"
