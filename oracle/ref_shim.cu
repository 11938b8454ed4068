// C-ABI wrappers around the REFERENCE's own CUDA launchers, so the tests and the benchmark can run
// the reference's kernels (its sm_86-era sources recompiled for sm_100a) beside the new library on
// identical device buffers.  TEST INFRASTRUCTURE ONLY: this file contains no kernel code; it
// includes the reference's headers from the reference tree at build time (see oracle/Makefile) and
// is linked with objects compiled from the reference's attn.cu, gdn.cu, dsa_topk.cu, norm.cu and
// glue2.cu where they lie.  Nothing from the reference is copied into this repository.
#include "cuda/attn/attn.cuh"
#include "cuda/aux/gdn.cuh"
#include "cuda/aux/dsa_topk.cuh"
#include "cuda/aux/norm.cuh"
#include "engine/glue2.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))
using bf16 = __nv_bfloat16;
using helios::Stream;

REF_API int ref_abi_version() { return 1; }

REF_API void ref_conv1d_update(const void* x, void* state, const int* slots, const void* w,
                               const void* bias, void* out, int bsz, int dim, int seqlen,
                               int state_size, int K, int act, int history, void* stream) {
  helios::aux::cuda_causal_conv1d_update((const bf16*)x, (bf16*)state, slots, (const bf16*)w,
                                         (const bf16*)bias, (bf16*)out, bsz, dim, seqlen, state_size,
                                         K, act != 0, history != 0, (Stream)stream);
}

REF_API void ref_kda_recurrent(const void* qkv, const float* g, const void* beta, float* state,
                               void* out, int bsz, int seqlen, int Hk, int Hv, int dk, int dv,
                               int history_stride, const int* slots, int channelwise, int history,
                               void* stream) {
  helios::aux::cuda_recurrent_gated_delta_rule((const bf16*)qkv, g, (const bf16*)beta, state,
                                               (bf16*)out, bsz, seqlen, Hk, Hv, dk, dv,
                                               history_stride, slots, channelwise != 0, history != 0,
                                               (Stream)stream);
}

REF_API void ref_kpool_write(const void* idx_k, const void* idx_g, void* ring, int raw_rows,
                             void* pool_k_nt, const float* ape, int pos_start, int n_new,
                             void* stream) {
  helios::attn::kpool_write((const half*)idx_k, (const half*)idx_g, (half*)ring, raw_rows,
                            (half*)pool_k_nt, ape, pos_start, n_new, (Stream)stream);
}

REF_API void ref_indexer_score(const void* q, const void* pk, const void* w, const int* q_pos,
                               void* scores, int m, int npools, void* stream) {
  helios::attn::indexer_score((const half*)q, (const half*)pk, (const half*)w, q_pos, (half*)scores,
                              m, npools, (Stream)stream);
}

REF_API void ref_indexer_score_legacy(const void* q, const void* pk, const void* w,
                                      const int* q_pos, void* scores, int m, int npools,
                                      int pk_stride, void* stream) {
  helios::attn::indexer_score_legacy((const half*)q, (const half*)pk, (const half*)w, q_pos,
                                     (half*)scores, m, npools, pk_stride, (Stream)stream);
}

REF_API void ref_dsa_topk(const void* scores, int s_stride, int* indices, int R, int T, int k,
                          int k_pad, int t_seq, void* stream) {
  helios::aux::dsa_topk((const half*)scores, s_stride, indices, R, T, k, k_pad, nullptr, t_seq,
                        (Stream)stream);
}

REF_API void ref_dsa_topk_free_workspace() { helios::aux::dsa_topk_free_workspace(); }

REF_API void ref_pool_expand(const int* pool_idx, const int* q_pos, int* raw, int m, int cur_pos,
                             void* stream) {
  helios::attn::pool_expand(pool_idx, q_pos, raw, m, cur_pos, (Stream)stream);
}

REF_API void ref_pool_expand_row(const int* pool_idx, const int* q_pos, int* raw, int m,
                                 void* stream) {
  helios::attn::pool_expand_row(pool_idx, q_pos, raw, m, (Stream)stream);
}

REF_API void ref_mla_sparse_decode(const void* q_lat, const void* ckv, const int* raw_idx, int kidx,
                                   void* lat_out, int m, void* stream) {
  helios::attn::mla_sparse_decode((const half*)q_lat, (const half*)ckv, raw_idx, kidx,
                                  (half*)lat_out, m, (Stream)stream);
}

REF_API void ref_mla_dense_prefill(const void* q_lat, const void* ckv, void* lat_out, int qlen,
                                   int pos_start, void* stream) {
  helios::attn::mla_dense_prefill((const half*)q_lat, (const half*)ckv, (half*)lat_out, qlen,
                                  pos_start, (Stream)stream);
}

REF_API void ref_q_latent(const void* q_nope, const void* kv_b, void* q_lat, int m, void* stream) {
  helios::attn::q_latent((const half*)q_nope, (const half*)kv_b, (half*)q_lat, m, (Stream)stream);
}

REF_API void ref_o_absorb(const void* lat_out, const void* kv_b, void* o, int m, void* stream) {
  helios::attn::o_absorb((const half*)lat_out, (const half*)kv_b, (half*)o, m, (Stream)stream);
}

REF_API void ref_q_latent_t(const void* q_nope, const void* kv_b, void* q_lat, int n, void* stream) {
  helios::attn::q_latent_t((const half*)q_nope, (const half*)kv_b, (half*)q_lat, n, (Stream)stream);
}

REF_API void ref_wuv_transpose(const void* kv_b, void* wuv_t, void* stream) {
  helios::attn::wuv_transpose((const half*)kv_b, (half*)wuv_t, (Stream)stream);
}

REF_API void ref_o_absorb_t(const void* lat_out, const void* wuv_t, void* o, int n, void* stream) {
  helios::attn::o_absorb_t((const half*)lat_out, (const half*)wuv_t, (half*)o, n, (Stream)stream);
}

REF_API void ref_kda_transpose_cast(void* dst_bf16, const float* src, int S, int F, void* stream) {
  helios::glue::kda_transpose_cast(dst_bf16, src, S, F, (Stream)stream);
}

REF_API void ref_kda_gate(const float* b, const float* f, const float* dt_bias, const float* a_log,
                          float lower_bound, void* beta_bf16, float* g, int S, int H, int Dk,
                          void* stream) {
  helios::glue::kda_gate(b, f, dt_bias, a_log, lower_bound, beta_bf16, g, S, H, Dk, (Stream)stream);
}

REF_API void ref_kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                             const float* a_log, float lower_bound, void* mixed_qkv_bf16,
                             void* beta_bf16, float* g, int S, int F, int H, int Dk, void* stream) {
  helios::glue::kda_prepare(qkv, b, f, dt_bias, a_log, lower_bound, mixed_qkv_bf16, beta_bf16, g, S, F,
                            H, Dk, (Stream)stream);
}

// dtype codes of this wrapper: 0 = half, 1 = bfloat16, 2 = float
static helios::aux::DType ref_dtype(int code) {
  return code == 0 ? helios::aux::kHalf : (code == 1 ? helios::aux::kBFloat16 : helios::aux::kFloat);
}

REF_API void ref_gated_rms_norm(const void* x, const void* w, int tw, void* y, int ty, const void* g,
                                int tg, int rows, int dim, float epsilon, float constant_bias,
                                int w_groups, int gate_first, int gate_act, void* stream) {
  helios::aux::gated_rms_norm(x, w, ref_dtype(tw), y, ref_dtype(ty), g, ref_dtype(tg), rows, dim, epsilon,
                              constant_bias, w_groups, gate_first != 0, gate_act, (Stream)stream);
}

REF_API void ref_rms_norm(const void* x, int tx, const void* w, int tw, void* y, int ty, int rows, int dim,
                          float epsilon, void* stream) {
  helios::aux::rms_norm(x, ref_dtype(tx), w, ref_dtype(tw), y, ref_dtype(ty), rows, dim, epsilon, 0.0f, 1.0f,
                        false, 1, (Stream)stream);
}

REF_API void ref_layernorm_f16(const void* x, const void* w, const void* b, void* y, int rows, int dim,
                               float eps, void* stream) {
  helios::glue::layernorm_f16((const half*)x, (const half*)w, (const half*)b, (half*)y, rows, dim, eps,
                              (Stream)stream);
}
