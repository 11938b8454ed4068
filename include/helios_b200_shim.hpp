// helios_b200_shim.hpp — the reference engine's launcher entry points, served by libhelios_b200.
//
// These are the C++-linkage free functions that Helios's layer loop calls
// (src/engine/runner.cpp:443, :468, :584, :608, :620-625, :630, :658-662, :215) and that its own
// kernel tests link against (src/cuda/attn/test/test_attn_parity.cpp, test/
// test_deterministic_reductions.cu).  Names, namespaces, argument order, argument meaning and the
// error behaviour (precondition failure -> message on stderr + abort()) are the reference's
// (declared there in src/cuda/attn/attn.cuh:24-108, src/cuda/aux/gdn.cuh:47-83,
// src/cuda/aux/dsa_topk.cuh:15-43, src/cuda/aux/norm.cuh:71-87, src/engine/glue2.cuh:57-67); the bodies forward to the hk_* C ABI (helios_b200.h).
//
// Differences a maintainer should know:
//   * the reference signatures carry no scratch pointers, so this layer keeps one device scratch buffer
//     per GPU, shared by all launchers of that GPU: call them from ONE stream, as the engine's layer
//     loop does.  By default it is grow-only (cudaMalloc on first use / growth after a device
//     synchronisation, like the reference's own dsa_topk workspace, src/cuda/aux/dsa_topk.cu:299-306)
//     and helios::b200::release_scratch() frees it.  An engine that owns all device memory hands over
//     its own block once with helios::b200::set_scratch(ptr, bytes) (size it with
//     scratch_bytes_needed): the launchers then never allocate or synchronise, also under stream
//     capture, and abort with a message if a call needs more.  The hk_* ABI underneath never allocates.
//   * cuda_recurrent_gated_delta_rule runs the chunked tensor-core kernel when
//     channelwise && !history && seqlen >= 64 && head dims are 128, and the per-token kernel
//     otherwise; results agree within the tolerances stated in the test-suite.
//   * HELIOS_SPARSE_K is not read: there is one sparse kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>

namespace helios {

using Stream = cudaStream_t;

namespace attn {
constexpr int N_HEADS = 64, QK_NOPE = 256, KV_LORA = 512, V_DIM = 256;
constexpr int IDX_HEADS = 32, IDX_DIM = 128, POOL = 4;
constexpr float SCALE = 0.0625f;
constexpr float IDX_SCALE = 0.08838834764f * 0.17677669530f;

void q_latent(const half* q_nope, const half* kv_b, half* q_lat, int m, Stream s = 0);
void wuv_transpose(const half* kv_b, half* wuv_t, Stream s = 0);
void o_absorb_t(const half* lat_out, const half* wuv_t, half* o, int nrows, Stream s = 0);
void q_latent_t(const half* q_nope, const half* kv_b, half* q_lat, int nrows, Stream s = 0);
void o_absorb(const half* lat_out, const half* kv_b, half* o, int m, Stream s = 0);
void indexer_score_mma(const half* q_idx, const half* pool_k_nt, const half* w, const int* q_pos,
                       half* scores, int m, int npools, Stream s = 0);
void indexer_score_legacy(const half* q_idx, const half* pool_k, const half* w, const int* q_pos,
                          half* scores, int m, int npools, int pk_stride, Stream s = 0);
void indexer_score(const half* q_idx, const half* pool_k_nt, const half* w, const int* q_pos,
                   half* scores, int m, int npools, Stream s = 0);
void pool_expand(const int* pool_idx, const int* q_pos, int* raw_idx, int m, int cur_pos,
                 Stream s = 0);
void pool_expand_row(const int* pool_idx, const int* q_pos, int* raw_idx, int m, Stream s = 0);
void kpool_write(const half* idx_k, const half* idx_g, half* raw_ring, int raw_rows,
                 half* pool_k_nt, const float* ape, int pos_start, int n_new, Stream s = 0);
void mla_sparse_decode(const half* q_lat, const half* ckv, const int* raw_idx, int kidx,
                       half* lat_out, int m, Stream s = 0);
void mla_dense_prefill(const half* q_lat, const half* ckv, half* lat_out, int qlen, int pos_start,
                       Stream s = 0);
}  // namespace attn

namespace aux {
using bfloat16 = __nv_bfloat16;

void cuda_recurrent_gated_delta_rule(const bfloat16* mixed_qkv, const float* g,
                                     const bfloat16* beta, float* recurrent_state,
                                     bfloat16* core_attn_out, int bsz, int seqlen, int num_k_heads,
                                     int num_v_heads, int k_head_dim, int v_head_dim,
                                     int history_stride, const int* slots, bool channelwise,
                                     bool history, Stream stream);
void cuda_causal_conv1d_update(const bfloat16* x, bfloat16* conv_state, const int* slots,
                               const bfloat16* weight, const bfloat16* bias, bfloat16* out, int bsz,
                               int dim, int seqlen, int state_size, int K, bool activation,
                               bool history, Stream stream);
void dsa_topk(const half* scores, int s_stride, int* indices, int R, int T, int k, int k_pad,
              const int* t_ptr = nullptr, int t_seq = 0, Stream stream = 0);
void dsa_topk_free_workspace(void);

// dtype tags of the raw-pointer launchers (src/cuda/aux/dtypes.hpp:10-15; same values)
enum DType : int { kFloat = 0, kHalf = 1, kBFloat16 = 2 };
// y = norm(x) * w * act(g) (src/cuda/aux/norm.cuh:71-87): x bf16; w float/bf16; y half/float; g bf16/float
void gated_rms_norm(const void* x, const void* w, DType tw, void* y, DType ty, const void* g, DType tg,
                    int rows, int dim, float epsilon, float constant_bias = 0.0f, int w_groups = 1,
                    bool gate_first = false, int gate_act = 0, Stream s = 0);
}  // namespace aux

namespace glue {
// KDA producers (src/engine/glue2.cuh:57-67)
void kda_transpose_cast(void* dst_bf16, const float* src, int S, int F, Stream s = 0);
void kda_gate(const float* b, const float* f, const float* dt_bias, const float* a_log,
              float lower_bound, void* beta_bf16, float* g, int S, int H, int Dk, Stream s = 0);
void kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                 const float* a_log, float lower_bound, void* mixed_qkv_bf16, void* beta_bf16, float* g,
                 int S, int F, int H, int Dk, Stream s = 0);
// layer norm with weight + bias over fp16 rows (src/engine/glue2.cuh:73-75)
void layernorm_f16(const half* x, const half* w, const half* b, half* y, int rows, int dim, float eps,
                   Stream s = 0);
}  // namespace glue

namespace b200 {
// frees this layer's per-GPU scratch buffer on the current device (it regrows on demand); forgets a host-provided one
void release_scratch();
// makes the launchers of the current device use `bytes` bytes at `ptr` (256-byte aligned device memory owned by the
// host) as their scratch instead of allocating; (nullptr, 0) returns to the grow-only buffer
void set_scratch(void* ptr, size_t bytes);
// upper bound of what the launchers ask for when no call has more than max_rows rows (chunk length of the prefill;
// decode calls are covered), for a KDA side of kda_batch sequences x kda_heads heads
size_t scratch_bytes_needed(int max_rows, int kda_heads, int kda_batch = 1);
}  // namespace b200

}  // namespace helios
