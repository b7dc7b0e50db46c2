// Internal (C++) declarations of the kernel launchers; the C ABI in abi.cu wraps them.
#pragma once
#include <cuda_runtime.h>

namespace clt {

int device_sm_count();

// elementwise.cu
int prep_input(const void* batch, int in_dtype, const float* mu, const float* sd, void* xn, int out_bf16, int B, int L,
               int D, int halves, cudaStream_t s);
int loss_fwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu, const float* sd,
             float* acc, int B, int L, int D, cudaStream_t s);
int sum_slots(const void* slots, float* out, int n_slots, long long n, int slots_bf16, cudaStream_t s);
int loss_bwd_push(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu,
                  const float* sd, const float* gscale, float aux_scale, const unsigned long long* drecon_ptrs,
                  const unsigned long long* daux_ptrs, int n_ranks, int out_bf16, float* db_dec, int B, int b_lo,
                  int b_cnt, int L, int D, cudaStream_t s);
int loss_bwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu, const float* sd,
             const float* gscale, float aux_scale, void* drecon, void* daux, int out_bf16, float* db_dec, int B, int L,
             int D, cudaStream_t s);
int act_fwd(const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* feat,
            unsigned* fired_bits, float* loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int L, int F,
            int bf16, cudaStream_t s);
int act_bwd(const void* g, const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* dpre,
            float* dtheta, float* dbenc, float* dnorm, float bandwidth, float lam, float c_sparsity, float pal,
            int use_tanh, const float* gscale, int B, int L, int F, int bf16, cudaStream_t s);
int dec_norms(const float* W, float* out, int L, int F, int D, int crosslayer, cudaStream_t s);
int norm_coef(const float* dnorm, const float* n, float* out, int count, cudaStream_t s);
int dead_update(long long* last_active, unsigned* fired_bits, unsigned char* dead, long long B, long long limit, int L,
                int F, int* dead_count, int* soon_dead, cudaStream_t s);
int adam_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float beta1,
              float beta2, float eps, float weight_decay, int decoupled, long long step, int num_sms, cudaStream_t s);
int cast_bf16(const float* src, void* dst, long long n, cudaStream_t s);
int finalize_loss(const float* mse_acc, const float* enc_acc, float* loss, float* terms, float inv_bld, float lam_over_b,
                  float pal_over_bl, float aux_scale, cudaStream_t s);

}  // namespace clt
