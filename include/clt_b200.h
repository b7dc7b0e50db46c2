/* C ABI of the B200 crosslayer-transcoder training-step library (libclt_b200.so).
 *
 * The reference project is pure Python and has no native interface; each entry
 * point below names the reference code it replaces (file:line, paths relative to
 * the reference project root).  All pointers are device pointers unless stated
 * otherwise; the library allocates and frees nothing, keeps no state between
 * calls except per-function launch attributes (and the built-in scratch array of
 * clt_csc_build_static), and launches on the stream it is given.  Every function returns 0 when its kernels were launched, non-zero when
 * an argument was rejected or a launch failed (then clt_last_error() holds the
 * reason).  Kernels never trap: a kernel that gives up on a bounded wait or meets
 * an out-of-range index writes a code to the `status` word passed by the caller
 * (one int in device memory, zero before the call) and returns.
 *
 * Shapes:  B tokens, L layers, D = d_acts, F = d_features held by this rank,
 *          P = number of decoder blocks (L (L+1)/2 crosslayer, L per-layer).
 * `bf16`:  0 = fp32 operands, CUDA-core contraction; 1 = bf16 operands, tcgen05
 *          tensor-core contraction with fp32 accumulation.  T below is float or
 *          __nv_bfloat16 accordingly.
 * Layouts: xn, drecon [L, B, D];  z, feat, dpre [L, B, F];  recon [B, L, D] fp32;
 *          W_enc [L, D, F];  W_dec flat [P, F, D], block (source s -> target t) at
 *          p = t (t+1)/2 + s (crosslayer) or p = layer (per-layer).
 * in_dtype of the raw batch [B, 2, L, D]: 0 = fp32, 1 = fp16, 2 = bf16.
 */
#ifndef CLT_B200_H
#define CLT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* clt_stream_t; /* a cudaStream_t */

int clt_version(void);
const char* clt_last_error(void);
/* 0 when the current device is compute capability 10.x; non-zero (with an error string) otherwise. */
int clt_device_check(void);

/* DimensionwiseInputStandardizer.forward (crosslayer_transcoder/model/standardize.py:49-59):
 * xn[l,b,d] = (batch[b,0,l,d] - mu[l,d]) / sd[l,d], cast to T, layer-major. */
int clt_prep_input(const void* batch, int in_dtype, const float* mu, const float* sd, void* xn, int bf16,
                   int B, int L, int D, clt_stream_t stream);

/* Encoder.forward + JumpReLU / ReLU forward (crosslayer_transcoder/model/clt.py:157-165,
 * crosslayer_transcoder/model/jumprelu.py:21-22, 33-38), plus the sums of the pre-activation
 * loss and sparsity penalty (crosslayer_transcoder/model/clt_lightning.py:450-465) and the
 * per-feature "fired" flags of update_dead_features (clt_lightning.py:284).
 * z = round_T(xn W_enc), pre = z + b_enc, feat = pre [pre > theta and pre > 0].
 * theta == NULL selects ReLU; dec_norm == NULL skips the sparsity sum; fired_bits
 * ([L, ceil(F/32)] words, one bit per feature, OR-ed into) may be NULL.
 * loss_acc[0] += sum relu(-pre) (when want_pre != 0); loss_acc[1] += sum tanh(feat dec_norm c)
 * (or the product). */
int clt_encoder_fwd_act(const void* xn, const void* W_enc, const float* b_enc, const float* theta,
                        const float* dec_norm, void* z_out, void* feat_out, uint32_t* fired_bits,
                        float* loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int L, int D,
                        int F, int bf16, int* status, clt_stream_t stream);

/* Encoder.forward alone (clt.py:157-162), for the TopK / BatchTopK selections that follow:
 * z = round_T(xn W_enc), no bias. */
int clt_encoder_fwd_store(const void* xn, const void* W_enc, void* z_out, int B, int L, int D, int F, int bf16,
                          int* status, clt_stream_t stream);

/* CrosslayerDecoder.forward (clt.py:334-343) / Decoder.forward (clt.py:241-248):
 * recon[b,t,:] = sum_{s<=t} feat[s,b,:] W_dec[pair(t,s)] (+ b_dec[t]); b_dec may be NULL. */
int clt_decoder_dense_fwd(const void* feat, const void* W_dec, const float* b_dec, float* recon, int B, int L,
                          int D, int F, int crosslayer, int bf16, int* status, clt_stream_t stream);

/* clt_decoder_dense_fwd fused with the exchange of the partial reconstructions over the feature-shard
 * ranks of one node (same buffer convention as clt_sparse_decoder_fwd_push: per-source slots
 * [n_ranks, rows_per_rank, L, D] fp32 on the owner; rank_bases is a host array of n_ranks device
 * addresses).  The contraction's epilogue stores each finished tile into slot my_slot of the owners'
 * buffers (16-byte stores, over NVLink for the peers) while the tensor cores work on the next tile.
 * Replaces the DTensor all-reduce after the decoder (crosslayer_transcoder/model/parallel.py:157-339). */
int clt_decoder_dense_fwd_push(const void* feat, const void* W_dec, const float* b_dec, const uint64_t* rank_bases,
                               int rows_per_rank, int n_ranks, int my_slot, int slot_bf16, int B, int L, int D, int F,
                               int crosslayer, int bf16, int* status, clt_stream_t stream);

/* Reconstruction MSE (clt_lightning.py:303-304) and, with aux != NULL, the TopK auxiliary
 * loss (clt_lightning.py:548-551).  acc[0] += sum diff^2, acc[1] += sum (aux + diff)^2. */
int clt_loss_fwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu_out,
                 const float* sd_out, float* acc, int B, int L, int D, clt_stream_t stream);

/* loss = acc terms scaled as the reference's means (clt_lightning.py:304, 459-468, 553);
 * terms[0..3] = mse, sparsity, pre-activation, auxiliary summands. enc_acc may be NULL. */
int clt_finalize_loss(const float* mse_acc, const float* enc_acc, float* loss, float* terms, float inv_bld,
                      float lam_over_b, float pal_over_bl, float aux_scale, clt_stream_t stream);

/* Backward of the losses w.r.t. the reconstruction(s) (what autograd derives from
 * clt_lightning.py:303-304, 548-553): drecon (and daux) [L,B,D] in T, db_dec[l,d] += column sums.
 * gscale: device scalar dLoss (NULL = 1). */
int clt_loss_bwd(const float* recon, const float* aux, const void* batch, int in_dtype, const float* mu_out,
                 const float* sd_out, const float* gscale, float aux_scale, void* drecon, void* daux, int bf16,
                 float* db_dec, int B, int L, int D, clt_stream_t stream);

/* clt_loss_bwd for the token rows [b_lo, b_lo + b_cnt) that this rank owns, fused with the all-gather of
 * the result over the feature-shard ranks of one node.  recon_own / aux_own hold the owned rows'
 * summed reconstructions as [b_cnt, L, D]; batch is the whole [B, 2, L, D] batch; the gradient rows are
 * written to row b of EVERY rank's [L, B, D] buffer (drecon_bases / daux_bases: host arrays of n_ranks
 * device addresses, this rank's own buffer included; the peers' buffers must be mapped into this
 * process, e.g. CUDA IPC or symmetric memory).  db_dec receives this rank's partial column sums.  The
 * caller orders the ranks (any stream-ordered collective after this call) before the buffers are read.
 * The reference has no counterpart: its tensor-parallel plan replicates the loss on every rank
 * (crosslayer_transcoder/model/clt_lightning.py:100-119). */
int clt_loss_bwd_push(const float* recon_own, const float* aux_own, const void* batch, int in_dtype,
                      const float* mu_out, const float* sd_out, const float* gscale, float aux_scale,
                      const uint64_t* drecon_bases, const uint64_t* daux_bases, int n_ranks, int bf16, float* db_dec,
                      int B, int b_lo, int b_cnt, int L, int D, clt_stream_t stream);

/* Backward of the decoder w.r.t. the features fused with the JumpReLU / ReLU backward
 * (jumprelu.py:41-48), the sparsity-penalty and pre-activation-loss gradients
 * (clt_lightning.py:450-465):  dfeat[s] = sum_{t>=s} drecon[t] W_dec[pair(t,s)]^T, then
 * dpre, dtheta, db_enc, d dec_norm as documented in csrc/epilogues.cuh.
 * lam = lambda / B, pal = pre_actv_loss / (B L). */
int clt_decoder_dense_bwd_dfeat(const void* drecon, const void* W_dec, const void* z_in, const float* b_enc,
                                const float* theta, const float* dec_norm, void* dpre_out, float* dtheta,
                                float* dbenc, float* dnorm, float bandwidth, float lam, float c_sparsity,
                                float pal, int use_tanh, const float* gscale, int B, int L, int D, int F,
                                int crosslayer, int bf16, int* status, clt_stream_t stream);

/* The same two fused operations split in two, for short contractions (small d_acts) where a fused
 * activation epilogue would outlast the tensor-core main loop of a tile:
 * clt_encoder_fwd_store + clt_act_fwd  ==  clt_encoder_fwd_act,
 * clt_decoder_dense_bwd_dfeat_raw (g = dfeat rounded to T) + clt_act_bwd  ==  clt_decoder_dense_bwd_dfeat.
 * dpre_out may alias g. */
int clt_act_fwd(const void* z, const float* b_enc, const float* theta, const float* dec_norm, void* feat_out,
                uint32_t* fired_bits, float* loss_acc, float c_sparsity, int use_tanh, int want_pre, int B, int L,
                int F, int bf16, clt_stream_t stream);
int clt_decoder_dense_bwd_dfeat_raw(const void* drecon, const void* W_dec, void* g_out, int B, int L, int D, int F,
                                    int crosslayer, int bf16, int* status, clt_stream_t stream);
int clt_act_bwd(const void* g, const void* z, const float* b_enc, const float* theta, const float* dec_norm,
                void* dpre_out, float* dtheta, float* dbenc, float* dnorm, float bandwidth, float lam,
                float c_sparsity, float pal, int use_tanh, const float* gscale, int B, int L, int F, int bf16,
                clt_stream_t stream);

/* Decoder weight gradient: dW_dec[pair(t,s)] = feat[s]^T drecon[t] (+ rowcoef[s,f] W_dec[p,f,:],
 * the gradient through the decoder norms of clt_lightning.py:438-448); fp32 output [P,F,D]. */
int clt_decoder_dense_bwd_dw(const void* feat, const void* drecon, float* dW, const float* rowcoef,
                             const float* W_master, int B, int L, int D, int F, int crosslayer, int bf16,
                             int* status, clt_stream_t stream);

/* Encoder weight gradient: dW_enc[l] = xn[l]^T dpre[l]; fp32 output [L,D,F]. */
int clt_encoder_dense_bwd_dw(const void* xn, const void* dpre, float* dW, int B, int L, int D, int F, int bf16,
                             int* status, clt_stream_t stream);

/* Decoder norms of the sparsity penalty (clt_lightning.py:438-448): out[s,f]. */
int clt_dec_norms(const float* W_dec, float* out, int L, int F, int D, int crosslayer, clt_stream_t stream);
/* out = dnorm / norm (0 where norm == 0) */
int clt_norm_coef(const float* dnorm, const float* norm, float* out, int count, clt_stream_t stream);

/* update_dead_features (clt_lightning.py:282-288): last_active[fired]=0; last_active+=B;
 * dead = last_active > limit (dead may be NULL).  fired_bits is [L, ceil(F/32)] words, one bit
 * per feature, and is cleared for the next step.  dead_count (one int, may be NULL) receives the
 * number of dead features, the numerator of the logged metrics/dead_features (clt_lightning.py:287).
 * soon_dead ([L] ints, may be NULL) receives per layer the number of features with last_active + 2 B > limit:
 * an upper bound of that layer's dead count in this and the next two steps (a feature only leaves the set
 * by firing), from which a caller can size the auxiliary path's operands ahead of time. */
int clt_dead_update(int64_t* last_active, uint32_t* fired_bits, uint8_t* dead, int64_t B, int64_t limit, int L,
                    int F, int* dead_count, int* soon_dead, clt_stream_t stream);

/* ---- TopK path --------------------------------------------------------------------------- */

/* PerLayerTopK._training_forward (crosslayer_transcoder/model/topk.py:53-63) on pre = z + b_enc:
 * idx / val [L, B, k] hold the (at most k) largest positive pre-activations of every row, valid
 * slots first, unused slots idx 0 / val 0 (a kept value that is not positive is zero after the ReLU and gets no
 * gradient, so it is not stored).  fired_bits as in clt_encoder_fwd_act; may be NULL. */
int clt_select_topk(const void* z, const float* b_enc, int* idx_out, float* val_out, uint32_t* fired_bits,
                    int B, int L, int F, int k, int bf16, clt_stream_t stream);

/* Ascending list of the dead features of every layer: dead_list [L, F], n_dead [L]
 * (idxs_dead of clt_lightning.py:286, compacted). */
int clt_dead_compact(const uint8_t* dead, int* dead_list, int* n_dead, int L, int F, clt_stream_t stream);

/* topk_aux(where(dead, pre, -inf)) (clt_lightning.py:544-546) written as the dense matrix of the
 * compacted dead features: a_out[l, b, j] = pre[l, b, dead_list[l][j]] if it is among the k_aux
 * largest positive dead pre-activations of the row (ties with the k_aux-th are all kept), else 0;
 * [L, B, nd_pad] in T, columns j >= n_dead[l] are 0.
 * mode 0: as above.  mode 1 (feature shards): write only cand_out [L, B, k_aux], this shard's k_aux
 * best values per row (0-padded).  mode 2: a_out from the exchanged per-row threshold thr [L, B].
 * The caller may size nd_pad and pick the mode from the counts of an earlier step: a layer with more dead
 * features than nd_pad, or (mode 0, row_count [L, B] = positive dead values per row summed over the
 * shards, may be NULL) a row with more than k_aux of them, writes the overflow code to `status`. */
int clt_select_aux(const void* z, const float* b_enc, const int* dead_list, const int* n_dead, void* a_out,
                   float* cand_out, const float* thr, int mode, int B, int L, int F, int k_aux, int nd_pad,
                   int bf16, const int* row_count, int* status, clt_stream_t stream);

/* cnt[l, b] = number of positive pre-activations among the dead features of the row (feature shards
 * sum these to see whether any row needs the candidate exchange of the auxiliary selection). */
int clt_aux_count(const void* z, const float* b_enc, const int* dead_list, const int* n_dead, int* cnt, int B,
                  int L, int F, int bf16, clt_stream_t stream);

/* Selection across feature shards (the reference has no counterpart: its tensor-parallel plan
 * rejects TopK, crosslayer_transcoder/model/parallel.py:269-274).  vals [R, rows, k] holds every
 * shard's k best values per row; thr[row] = the k-th largest positive one (0: keep all). */
int clt_topk_threshold(const float* vals, float* thr, int64_t rows, int R, int k, clt_stream_t stream);
/* Keep the local candidates at or above thr (ties stay), moved to the front of the row's slots;
 * clear the rest; mark the fired features. */
int clt_topk_apply_threshold(int* idx, float* val, const float* thr, uint32_t* fired_bits, int B, int L, int F,
                             int k, clt_stream_t stream);

/* Sparse feature lists.  Every layer owns `npl` entry slots: idx / val [L, npl] (val 0 = unused).
 * PerLayerTopK uses npl = B k with the k slots of token b at b k .. b k + k - 1 (valid ones first);
 * BatchTopK uses one list per layer in which the entries of token b occupy the segment
 * row_start[l, b] .. + row_cnt[l, b], with etok [L, npl] naming the token of every entry.
 *
 * CrosslayerDecoder.forward / Decoder.forward (clt.py:334-343, 241-248) on the selected features:
 * recon[b,t,:] = b_dec[t] + sum_{s<=t} sum_{entries e of (s,b)} val[e] W_dec[pair(t,s), idx[e], :].
 * row_start / row_cnt NULL = fixed k slots per token.  short_rows != 0 selects the variant with one
 * warp per (token, target) for lists of a few entries per row (feature shards); same result. */
int clt_sparse_decoder_fwd(const int* idx, const float* val, const int* row_start, const int* row_cnt,
                           int64_t npl, const void* W_dec, const float* b_dec, float* recon, int B, int L, int D,
                           int F, int k, int crosslayer, int short_rows, int bf16, int* status,
                           clt_stream_t stream);

/* clt_sparse_decoder_fwd fused with the exchange of the partial reconstructions over the feature-shard
 * ranks of one node: rank o owns tokens [o rows_per_rank, (o+1) rows_per_rank) and holds, in a buffer
 * mapped into every rank's process, one slot per source rank: [n_ranks, rows_per_rank, L, D] fp32
 * (rank_bases: host array of n_ranks device addresses, this rank's own included).  This rank STORES its
 * partial rows into slot my_slot of the owners' buffers (16-byte stores, over NVLink for the peers); once
 * every rank's call has finished (the caller orders the ranks with any stream-ordered collective) the
 * owner adds its slots with clt_sum_slots.  The reference sums the partial decoder outputs with a
 * DTensor all-reduce after the decoder (crosslayer_transcoder/model/parallel.py:157-339). */
int clt_sparse_decoder_fwd_push(const int* idx, const float* val, const int* row_start, const int* row_cnt,
                                int64_t npl, const void* W_dec, const float* b_dec, const uint64_t* rank_bases,
                                int rows_per_rank, int n_ranks, int my_slot, int slot_bf16, int B, int L, int D,
                                int F, int k, int crosslayer, int short_rows, int bf16, int* status,
                                clt_stream_t stream);

/* out[i] = sum_s slots[s n + i], i < n (n % 4 == 0; n % 8 == 0 for bf16 slots): the owner's local reduction
 * of the slots the ranks filled with the *_push entry points.  No reference counterpart (part of the fused
 * exchange).  slot_bf16 / slots_bf16 != 0 (both *_push entry points and this one): the slots hold the partial
 * rows rounded to bf16, which halves the bytes every rank sends over NVLink; the sum is taken in fp32.  (Under
 * bf16 autocast the reference's decoder product is itself rounded to bf16 before it is summed over the ranks.) */
int clt_sum_slots(const void* slots, float* out, int n_slots, int64_t n, int slots_bf16, clt_stream_t stream);

/* Feature-major copy of the selection: col_ptr [L, F+1], ent [L, npl] (entry slots grouped by
 * feature).  cursor [L, F] is scratch. */
int clt_csc_build(const int* idx, const float* val, int* col_ptr, int* cursor, int* ent, int64_t npl, int L,
                  int F, int* status, clt_stream_t stream);

/* Same result as clt_csc_build, for hosts that must not allocate device memory on behalf of this
 * library.  (No counterpart in the reference: it exists only for this library's callers.)
 * Some embedders hand the step a fixed set of buffers at start-up and cannot grow it afterwards:
 * a process whose device memory is wholly pre-reserved by its own pool allocator, so that a
 * cudaMalloc for scratch would fail or fragment the pool, or a latency-bound loop in which
 * cudaMalloc / cudaFree would stall the device.  For them the write cursors live in a 4 MiB
 * array inside the library image (1,048,576 ints; every GPU that loads the library carries it
 * until the process exits), so the caller passes inputs and outputs only and neither this call
 * nor anything under it calls cudaMalloc, cudaFree or an allocating library routine.
 * - L * F above 1,048,576 is rejected with an error; use clt_csc_build with your own cursor buffer.
 * - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
 *   that device current); make that first call before any stream capture begins.
 * - All calls on a device share the one array, which keeps whatever the previous call left in
 *   it.  Every entry the call reads is rewritten by the call first, so no clearing is needed,
 *   but two calls that overlap on the GPU (different streams, no ordering) race on it. */
int clt_csc_build_static(const int* idx, const float* val, int* col_ptr, int* ent, int64_t npl, int L, int F,
                         int* status, clt_stream_t stream);

/* Backward of the decoder on the selected features (autograd of clt.py:334-343 restricted to the
 * non-zero features): dval[e] = sum_{t>=s} drecon[t,b(e),:] . W_dec[pair(t,s), idx[e], :] and
 * dW_dec[pair(t,s), f, :] = sum_{e: idx[e] = f} val[e] drecon[t,b(e),:]; every row of dW is written.
 * etok NULL: token of slot e is e / k. */
int clt_sparse_bwd_dec(const int* col_ptr, const int* ent, const float* val, const int* etok, int64_t npl,
                       const void* W_dec, const void* drecon, float* dW, float* dval, int B, int L, int D, int F,
                       int k, int crosslayer, int bf16, clt_stream_t stream);

/* clt_sparse_bwd_dec with the optimizer applied in the same pass (opt-in, module.fuse_optimizer): every
 * decoder row's gradient is formed in registers (plus, for dead features, row dead_pos[s, f] of the
 * auxiliary loss's compact gradient dW_aux [P, nd_pad, D]; both may be NULL) and the torch.optim.Adam /
 * AdamW update (clt_lightning.py:339-352) is applied to the row at once: W_master, exp_avg, exp_avg_sq
 * [P, F, D] fp32 are updated in place and shadow_bf16 (the operand copy; NULL with bf16 = 0) is
 * refreshed.  The gradient is never stored and the operand copy never read (the dot products use the
 * rounded master weights, which equal it): 26 bytes per parameter instead of 6 + 30.  Rows of features
 * nobody selected get the zero-gradient update, so the result equals the separate kernels'.  Needs
 * F % 8 == 0.  dval as in clt_sparse_bwd_dec.  `step` counts from 1.  The update uses approximate square
 * root and division (relative error about 2^-22 on a step of at most lr). */
int clt_sparse_bwd_dec_adam(const int* col_ptr, const int* ent, const float* val, const int* etok, int64_t npl,
                            float* W_master, float* exp_avg, float* exp_avg_sq, void* shadow_bf16,
                            const void* drecon, float* dval, const float* dW_aux, const int* dead_pos, int nd_pad,
                            int B, int L, int D, int F, int k, int crosslayer, int bf16, float lr, float beta1,
                            float beta2, float eps, float weight_decay, int decoupled, int64_t step,
                            clt_stream_t stream);

/* dead_pos[l, f] = j where dead_list[l][j] == f (j < min(n_dead[l], nd_pad)), -1 for every other feature:
 * the inverse of clt_dead_compact's lists, [L, F], restricted to the columns the compact operands hold. */
int clt_dead_positions(const int* dead_list, const int* n_dead, int* dead_pos, int L, int F, int nd_pad,
                       clt_stream_t stream);

/* Backward of the encoder on the selected features (autograd of clt.py:157-165 through the TopK
 * scatter): dW_enc[l,:,f] = sum_{e: idx[e] = f} dval[e] xn[l,b(e),:], db_enc[l,f] = sum dval[e]; every
 * element of both is written.  With dW_aux [L, D, nd_pad], db_aux [L, nd_pad] and dead_pos [L, F] (all three or
 * none) the auxiliary loss's compact encoder gradients are added for the dead features in the same pass:
 * dW_enc[l,:,f] += dW_aux[l,:,dead_pos[l,f]], db_enc likewise (no separate scatter pass over the columns). */
int clt_sparse_bwd_enc(const int* col_ptr, const int* ent, const float* dval, const int* etok, int64_t npl,
                       const void* xn, float* dW_enc, float* db_enc, const float* dW_aux, const float* db_aux,
                       const int* dead_pos, int nd_pad, int B, int L, int D, int F, int k, int bf16,
                       clt_stream_t stream);

/* Compaction helpers of the auxiliary dead-feature path (clt_lightning.py:544-549 run as dense
 * contractions over the dead features only):
 * gather_rows : out[p, j, :] = W_dec[p, dead_list[s(p)][j], :]              (T, [P, nd_pad, D])
 * scatter_rows: dW_dec[p, dead_list[s(p)][j], :] += src[p, j, :]            (fp32)
 * (the compact encoder gradients are added inside clt_sparse_bwd_enc) */
int clt_gather_rows(const void* W_dec, const int* dead_list, const int* n_dead, void* out, int L, int F, int D,
                    int nd_pad, int crosslayer, int bf16, clt_stream_t stream);
/* Compact ENCODER operands of the dead features: Wc[l, d, j] = W_enc[l, d, dead_list[l][j]] (T, [L, D, nd_pad]),
 * bc[l, j] = b_enc[l, dead_list[l][j]] (fp32, [L, nd_pad]); padding columns get weight 0 and bias -1.  With
 * them the auxiliary path takes the dead features' pre-activations from a small contraction of its own
 * (clt_encoder_fwd_store with F = nd_pad) instead of sweeping the full pre-activations a second time:
 * clt_aux_count / clt_select_aux are then called on that compact output with dead_list = 0, 1, 2, ... */
int clt_gather_enc_cols(const void* W_enc, const float* b_enc, const int* dead_list, const int* n_dead, void* Wc,
                        float* bc, int L, int D, int F, int nd_pad, int bf16, clt_stream_t stream);
int clt_scatter_rows(const float* src, const int* dead_list, const int* n_dead, float* dW_dec, int L, int F,
                     int D, int nd_pad, int crosslayer, clt_stream_t stream);

/* ---- BatchTopK path ---------------------------------------------------------------------- */

/* BatchTopK._training_forward (crosslayer_transcoder/model/topk.py:76-96): the k B L largest of all
 * pre-activations of the batch; with groups = L, PerLayerBatchTopK._training_forward (topk.py:109-133):
 * the k B largest of every layer.  The threshold of a group is found by a three-level radix
 * select; per level: clt_batchtopk_hist fills hist [groups, 2048] (64-bit counters) with the digit
 * histogram of the elements inside the bucket chosen so far, feature shards sum their histograms,
 * clt_batchtopk_pick chooses the next bucket (n_keep = elements kept per group).
 * state: [groups, 8] 64-bit words of device memory, zero before the first step ([2] threshold key
 * after level 2, [3] kept elements equal to it, [5] this rank's count of them, [6] result code in the
 * low bits and 16 = "this step runs on full sweeps of z", [7] 0.9 of the last threshold: the first level
 * only looks at elements at or above it).  If that floor turns out too high the pick kernel requests a
 * retry: always enqueue the level-0 pair a second time with retry = 1 before levels 1 and 2; it returns
 * at once when no retry is pending.  hist_local (may be NULL) is this rank's own histogram when hist
 * holds the sum over shards.
 *
 * Candidate list (one sweep of z per step in steady state).  clt_batchtopk_candidates sweeps z once and
 * writes every element at or above the floor to cand_feat / cand_val / cand_row [cap] (one segment per
 * (layer, token) row, in a fixed scrambled order: cand_row_start / cand_row_cnt [L, B]; cand_fill: one int).  It
 * sets *list_invalid (one 64-bit word, zeroed by the call) when there is no floor yet, a row holds more
 * than 2048 candidates or the list is full.  Then, per level, BOTH clt_batchtopk_hist (given
 * list_invalid) and clt_batchtopk_hist_list are enqueued: at level 0 the former runs only if this rank's
 * list is invalid, the latter only if it is valid; clt_batchtopk_pick at level 0 looks at list_invalid
 * SUMMED OVER THE SHARDS (sum it together with the histogram) and, if it is non-zero or the floor proves
 * too high, marks the step for full sweeps; at levels 1 and 2 each kernel runs on the path chosen.
 * Likewise clt_batchtopk_collect (full sweeps) and clt_batchtopk_filter (candidate list; same outputs)
 * are both enqueued, in this order (collect's call zeroes layer_fill and val).  list_invalid = NULL in
 * clt_batchtopk_hist / _pick: no candidate list, always full sweeps. */
int clt_batchtopk_hist(const void* z, const float* b_enc, const uint64_t* state, uint64_t* hist,
                       const uint64_t* list_invalid, int level, int retry, int groups, int B, int L, int F,
                       int bf16, clt_stream_t stream);
int clt_batchtopk_pick(const uint64_t* hist, const uint64_t* hist_local, uint64_t* state,
                       const uint64_t* list_invalid, int level, int retry, int groups, int64_t n_keep,
                       clt_stream_t stream);
int clt_batchtopk_candidates(const void* z, const float* b_enc, const uint64_t* state, int* cand_feat,
                             float* cand_val, int* cand_row, int* cand_fill, int* cand_row_start,
                             int* cand_row_cnt, uint64_t* list_invalid, int groups, int B, int L, int F,
                             int64_t cap, int bf16, clt_stream_t stream);
int clt_batchtopk_hist_list(const float* cand_val, const int* cand_row, const int* cand_fill,
                            const uint64_t* state, uint64_t* hist, const uint64_t* list_invalid, int level,
                            int groups, int B, int64_t cap, clt_stream_t stream);
int clt_batchtopk_filter(const int* cand_feat, const float* cand_val, const int* cand_row_start,
                         const int* cand_row_cnt, uint64_t* state, const int64_t* tie_quota, int* idx,
                         float* val, int* etok, int* row_start, int* row_cnt, int* layer_fill,
                         uint32_t* fired_bits, int groups, int B, int L, int F, int64_t npl, int* status,
                         clt_stream_t stream);
/* Collect the survivors into per-layer entry lists idx / val / etok [L, npl] with the segment of
 * token b at row_start[l,b] .. + row_cnt[l,b]; layer_fill [L] receives the list lengths.  tie_quota
 * (device int64 per group, may be NULL = all kept ties are this rank's) bounds the elements equal to
 * the threshold this rank keeps.  Sets fired_bits (may be NULL); reports list overflow in status. */
int clt_batchtopk_collect(const void* z, const float* b_enc, uint64_t* state, const int64_t* tie_quota, int* idx,
                          float* val, int* etok, int* row_start, int* row_cnt, int* layer_fill,
                          uint32_t* fired_bits, int groups, int B, int L, int F, int64_t npl, int bf16,
                          int* status, clt_stream_t stream);
/* threshold[g] <- (1 - e) threshold[g] + e * smallest kept value of group g (topk.py:94-95, 131-132). */
int clt_batchtopk_threshold_update(uint64_t* state, float* threshold, float e, int groups, clt_stream_t stream);

/* ---- inference forward --------------------------------------------------------------------- */

/* CrossLayerTranscoder.forward without gradients (clt.py:403-425) and the per-layer forward_layer calls
 * (clt.py:134-145, 216-231, 304-317) run on the contraction / selection / decoder entry points above; the
 * entry points below move between the module surface's token-major fp32 tensors and the kernels'
 * layer-major operands.
 * clt_prep_acts: xn[l,b,:] = T((acts[b,l,:] - mu[l]) / sd[l]) for acts [B, L, D] (mu = sd = NULL: cast only).
 * clt_export_blf: out[b,l,:] = src[l,b,:] (+ bias[l,:]), src [L, B, F] in T, out [B, L, F] fp32.
 * clt_import_blf: dst[l,b,:] = T(src[b,l,:]).
 * clt_destandardize: out = recon * sd + mu (DimensionwiseOutputStandardizer.forward, standardize.py:88-98).
 * clt_scatter_features: dense [B, L, F] fp32 zeroed, then dense[token(e), l, idx[e]] = val[e] for the valid
 * entries of the lists idx / val [L, npl] (etok NULL: token = slot / k, npl = B k). */
int clt_prep_acts(const void* acts, int in_dtype, const float* mu, const float* sd, void* xn, int bf16, int B,
                  int L, int D, clt_stream_t stream);
int clt_export_blf(const void* src, const float* bias, float* out, int B, int L, int64_t F, int bf16,
                   clt_stream_t stream);
int clt_import_blf(const float* src, void* dst, int B, int L, int64_t F, int bf16, clt_stream_t stream);
int clt_destandardize(const float* recon, const float* mu, const float* sd, float* out, int B, int L, int D,
                      clt_stream_t stream);
int clt_scatter_features(const int* idx, const float* val, const int* etok, float* dense, int B, int L, int F,
                         int k, int64_t npl, int* status, clt_stream_t stream);

/* ---- batch ingestion ----------------------------------------------------------------------- */

/* The reference's activation store keeps `[buffer_size, 2, L, D]` rows in host shared memory and its
 * get_activations (crosslayer_transcoder/data/shared_memory.py:168-214) gathers a random batch of valid
 * rows into a new pageable tensor on one CPU thread.  Replacement: map the store into the device's
 * address space once (clt_host_register: cudaHostRegister, mapped + portable; *device_ptr is the address
 * the kernels use; clt_host_unregister before the mapping goes away), then per batch
 *   dst[i, :] = src[rows[i], :]     (clt_gather_batch_rows; rows: n_rows 64-bit indices in device memory)
 * read by the GPU over PCIe with 16-byte loads.  src may equally be device memory.  row_bytes must be a
 * multiple of 16 and both buffers 16-byte aligned; a row index outside [0, n_src_rows) is skipped and
 * status (may be NULL) set to 0x20. */
int clt_host_register(void* host_ptr, int64_t bytes, void** device_ptr);
int clt_host_unregister(void* host_ptr);
int clt_gather_batch_rows(const void* src, const int64_t* rows, void* dst, int64_t row_bytes, int n_rows,
                          int64_t n_src_rows, int* status, clt_stream_t stream);

/* ---- training metrics ---------------------------------------------------------------------- */

/* The sums behind the reconstruction metrics of log_training_metrics (clt_lightning.py:131-199),
 * taken on the device instead of after a copy of the features to the host.  For the n_rows tokens
 * b_lo .. b_lo + n_rows - 1 (recon_rows [n_rows, L, D] fp32 holds their normalised reconstructions;
 * batch is the whole [B, 2, L, D] batch) and every (layer, dim) c:
 *   out[c, 0..5] += sum yn, sum yn^2, sum (yn - r)^2, sum (y - (r sd + mu))^2, sum r, sum r^2
 * with yn = (y - mu) / sd the standardised target.  out [L, D, 6] fp32 is accumulated into (zero it
 * first; feature-shard ranks that each hold some of the rows add theirs and sum over the ranks). */
int clt_recon_stats(const float* recon_rows, const void* batch, int in_dtype, const float* mu_out,
                    const float* sd_out, float* out, int b_lo, int n_rows, int L, int D, clt_stream_t stream);

/* out[l] += number of positive elements of x[l, 0 .. n_per_layer) (x: dtype 0 fp32 / 1 fp16 / 2 bf16): the
 * L0 counts of clt_lightning.py:187-199 from the dense features [L, B, F] or from a sparse value list
 * [L, npl].  out: L 64-bit counters, accumulated into. */
int clt_count_active(const void* x, int dtype, int64_t n_per_layer, int L, uint64_t* out, clt_stream_t stream);

/* torch.optim.Adam / AdamW step (clt_lightning.py:339-352) over one flat fp32 buffer; `step`
 * counts from 1.  shadow_bf16 (may be NULL) receives the bf16 copy of the new parameters. */
int clt_adam_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, int64_t n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int decoupled, int64_t step,
                  clt_stream_t stream);

/* fp32 -> bf16 copy of a parameter buffer (the tensor-core operands). */
int clt_cast_bf16(const float* src, void* dst, int64_t n, clt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CLT_B200_H */
