// Reference-named C++ launchers (helios::attn::*, helios::aux::*) on top of the hk_* C ABI.
// See include/helios_b200_shim.hpp for the contract.
#pragma GCC visibility push(default)
#include "../../include/helios_b200_shim.hpp"
#pragma GCC visibility pop

#include <cstdio>
#include <cstdlib>

#include "hk_common.cuh"

namespace {

// precondition / launch failure: message + abort(), as HELIOS_ASSERT / HELIOS_CUDA_CHECK do in the
// reference (src/cuda/attn/helios_shim.cuh:29-30, src/cuda/cuda_shim.hpp:13-14)
void check(int status, const char* what) {
  if (status != HK_OK) {
    std::fprintf(stderr, "helios_b200: %s failed: %s\n", what, hk_status_string(status));
    std::abort();
  }
}

struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool injected = false;   // memory handed over by the host with set_scratch: never freed or replaced here
};
Scratch g_scratch[64];

// Scratch of the current device.  Host-provided memory (helios::b200::set_scratch) is used as it is and a request
// beyond its size aborts with a message.  Otherwise the buffer is grow-only: growth synchronises the device before
// freeing the old buffer, so kernels still using it are finished.  All launchers of a device share the buffer: they
// are meant to run on ONE stream (as the engine's layer loop does).
void* scratch(size_t bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  Scratch& s = g_scratch[dev];
  if (s.injected) {
    if (s.bytes < bytes) {
      std::fprintf(stderr, "helios_b200: the scratch given to set_scratch holds %zu bytes, a launcher needs %zu\n", s.bytes, bytes);
      std::abort();
    }
    return s.ptr;
  }
  if (s.bytes < bytes) {
    if (s.ptr) {
      cudaDeviceSynchronize();
      cudaFree(s.ptr);
      s.ptr = nullptr;
      s.bytes = 0;
    }
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (cudaMalloc(&s.ptr, want) != cudaSuccess) {
      std::fprintf(stderr, "helios_b200: cannot allocate %zu bytes of scratch\n", want);
      std::abort();
    }
    s.bytes = want;
  }
  return s.ptr;
}

}  // namespace

namespace helios {

namespace b200 {
void set_scratch(void* ptr, size_t bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return;
  release_scratch();
  if (ptr && bytes) {
    g_scratch[dev].ptr = ptr;
    g_scratch[dev].bytes = bytes;
    g_scratch[dev].injected = true;
  }
}
size_t scratch_bytes_needed(int max_rows, int kda_heads, int kda_batch) {
  // the largest request any launcher makes for calls of at most max_rows rows
  size_t need = hk_kda_chunked_workspace_bytes(kda_batch, max_rows, kda_heads);
  for (int m : {1, 2, 4, 8, max_rows}) {
    if (m > max_rows) continue;
    const int ns_sparse = hk_mla_auto_splits(m, 2052), ns_dense = hk_mla_auto_splits(m, 1 << 20);
    const size_t a = ns_sparse > 1 ? hk_mla_partial_bytes(ns_sparse, (int64_t)m * attn::N_HEADS) : 0;
    const size_t b = ns_dense > 1 ? hk_mla_partial_bytes(ns_dense, (int64_t)m * attn::N_HEADS) : 0;
    need = need > a ? need : a;
    need = need > b ? need : b;
  }
  return (need + 255) / 256 * 256;
}
void release_scratch() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return;
  if (g_scratch[dev].injected) {
    g_scratch[dev] = Scratch{};
    return;
  }
  if (g_scratch[dev].ptr) {
    cudaDeviceSynchronize();
    cudaFree(g_scratch[dev].ptr);
    g_scratch[dev] = Scratch{};
  }
}
}  // namespace b200

namespace attn {

void q_latent(const half* q_nope, const half* kv_b, half* q_lat, int m, Stream s) {
  check(hk_q_latent(q_nope, kv_b, q_lat, m, s), "q_latent");
}
void q_latent_t(const half* q_nope, const half* kv_b, half* q_lat, int nrows, Stream s) {
  check(hk_q_latent(q_nope, kv_b, q_lat, nrows, s), "q_latent_t");
}
void wuv_transpose(const half* kv_b, half* wuv_t, Stream s) {
  check(hk_wuv_transpose(kv_b, wuv_t, s), "wuv_transpose");
}
void o_absorb_t(const half* lat_out, const half* wuv_t, half* o, int nrows, Stream s) {
  check(hk_o_absorb_t(lat_out, wuv_t, o, nrows, s), "o_absorb_t");
}
void o_absorb(const half* lat_out, const half* kv_b, half* o, int m, Stream s) {
  check(hk_o_absorb(lat_out, kv_b, o, m, s), "o_absorb");
}
void indexer_score_mma(const half* q_idx, const half* pool_k_nt, const half* w, const int* q_pos,
                       half* scores, int m, int npools, Stream s) {
  check(hk_indexer_score(q_idx, pool_k_nt, w, q_pos, scores, m, npools, npools, IDX_HEADS, HK_F16, s),
        "indexer_score_mma");
}
void indexer_score(const half* q_idx, const half* pool_k_nt, const half* w, const int* q_pos,
                   half* scores, int m, int npools, Stream s) {
  check(hk_indexer_score(q_idx, pool_k_nt, w, q_pos, scores, m, npools, npools, IDX_HEADS, HK_F16, s),
        "indexer_score");
}
void indexer_score_legacy(const half* q_idx, const half* pool_k, const half* w, const int* q_pos,
                          half* scores, int m, int npools, int pk_stride, Stream s) {
  check(hk_indexer_score_legacy(q_idx, pool_k, w, q_pos, scores, m, npools, pk_stride, s),
        "indexer_score_legacy");
}
void pool_expand(const int* pool_idx, const int* q_pos, int* raw_idx, int m, int cur_pos, Stream s) {
  (void)q_pos;  // the reference ignores it here too (attn.cu:300-304)
  check(hk_pool_expand(pool_idx, nullptr, raw_idx, m, cur_pos, 512, s), "pool_expand");
}
void pool_expand_row(const int* pool_idx, const int* q_pos, int* raw_idx, int m, Stream s) {
  if (!q_pos) check(HK_ERR_INVALID, "pool_expand_row");
  check(hk_pool_expand(pool_idx, q_pos, raw_idx, m, 0, 512, s), "pool_expand_row");
}
void kpool_write(const half* idx_k, const half* idx_g, half* raw_ring, int raw_rows,
                 half* pool_k_nt, const float* ape, int pos_start, int n_new, Stream s) {
  check(hk_kpool_write(idx_k, idx_g, raw_ring, raw_rows, pool_k_nt, ape, pos_start, n_new, s),
        "kpool_write");
}
void mla_sparse_decode(const half* q_lat, const half* ckv, const int* raw_idx, int kidx,
                       half* lat_out, int m, Stream s) {
  if (m <= 0) return;
  const int n_split = hk_mla_auto_splits(m, kidx);
  size_t bytes = n_split > 1 ? hk_mla_partial_bytes(n_split, (int64_t)m * N_HEADS) : 0;
  void* ws = bytes ? scratch(bytes) : nullptr;
  check(hk_mla_sparse(q_lat, ckv, 0, raw_idx, kidx, lat_out, m, N_HEADS, SCALE, n_split, ws, bytes, s),
        "mla_sparse_decode");
}
void mla_dense_prefill(const half* q_lat, const half* ckv, half* lat_out, int qlen, int pos_start,
                       Stream s) {
  if (qlen <= 0) return;
  const int n_split = hk_mla_auto_splits(qlen, pos_start + qlen);
  size_t bytes = n_split > 1 ? hk_mla_partial_bytes(n_split, (int64_t)qlen * N_HEADS) : 0;
  void* ws = bytes ? scratch(bytes) : nullptr;
  check(hk_mla_dense(q_lat, ckv, 0, nullptr, nullptr, pos_start, lat_out, qlen, N_HEADS, SCALE, n_split,
                     ws, bytes, s),
        "mla_dense_prefill");
}

}  // namespace attn

namespace aux {

void cuda_recurrent_gated_delta_rule(const bfloat16* mixed_qkv, const float* g,
                                     const bfloat16* beta, float* recurrent_state,
                                     bfloat16* core_attn_out, int bsz, int seqlen, int num_k_heads,
                                     int num_v_heads, int k_head_dim, int v_head_dim,
                                     int history_stride, const int* slots, bool channelwise,
                                     bool history, Stream stream) {
  const bool chunked = hk_kda_dispatch_is_chunked(seqlen, num_k_heads, num_v_heads, k_head_dim, v_head_dim, history_stride,
                                                  channelwise, history) != 0;
  if (chunked) {
    size_t bytes = hk_kda_chunked_workspace_bytes(bsz, seqlen, num_v_heads);
    int st = hk_kda_chunked_prefill(mixed_qkv, g, beta, recurrent_state, core_attn_out, nullptr, bsz,
                                    seqlen, num_v_heads, slots, scratch(bytes), bytes, stream);
    if (st != HK_ERR_UNSUPPORTED) {
      check(st, "cuda_recurrent_gated_delta_rule (chunked)");
      return;
    }
  }
  check(hk_kda_recurrent(mixed_qkv, g, beta, recurrent_state, core_attn_out, nullptr, bsz, seqlen,
                         num_k_heads, num_v_heads, k_head_dim, v_head_dim, history_stride, slots,
                         channelwise, history, stream),
        "cuda_recurrent_gated_delta_rule");
}

void cuda_causal_conv1d_update(const bfloat16* x, bfloat16* conv_state, const int* slots,
                               const bfloat16* weight, const bfloat16* bias, bfloat16* out, int bsz,
                               int dim, int seqlen, int state_size, int K, bool activation,
                               bool history, Stream stream) {
  check(hk_conv1d_update(x, conv_state, slots, weight, bias, out, bsz, dim, seqlen, state_size, K,
                         activation, history, stream),
        "cuda_causal_conv1d_update");
}

void dsa_topk(const half* scores, int s_stride, int* indices, int R, int T, int k, int k_pad,
              const int* t_ptr, int t_seq, Stream stream) {
  check(hk_dsa_topk(scores, s_stride, indices, R, T, k, k_pad, t_ptr, t_seq, stream), "dsa_topk");
}

void dsa_topk_free_workspace(void) {}  // this implementation keeps no top-k workspace

void gated_rms_norm(const void* x, const void* w, DType tw, void* y, DType ty, const void* g, DType tg,
                    int rows, int dim, float epsilon, float constant_bias, int w_groups, bool gate_first,
                    int gate_act, Stream s) {
  auto code = [](DType t) { return t == kFloat ? HK_F32 : (t == kHalf ? HK_F16 : HK_BF16); };
  check(hk_gated_rms_norm(x, w, code(tw), y, code(ty), g, code(tg), rows, dim, epsilon, constant_bias,
                          w_groups, gate_first, gate_act, s),
        "gated_rms_norm");
}

}  // namespace aux

namespace glue {

void kda_transpose_cast(void* dst_bf16, const float* src, int S, int F, Stream s) {
  check(hk_kda_transpose_cast(dst_bf16, src, S, F, s), "kda_transpose_cast");
}
void kda_gate(const float* b, const float* f, const float* dt_bias, const float* a_log,
              float lower_bound, void* beta_bf16, float* g, int S, int H, int Dk, Stream s) {
  check(hk_kda_gate(b, f, dt_bias, a_log, lower_bound, beta_bf16, g, S, H, Dk, s), "kda_gate");
}
void kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                 const float* a_log, float lower_bound, void* mixed_qkv_bf16, void* beta_bf16, float* g,
                 int S, int F, int H, int Dk, Stream s) {
  check(hk_kda_prepare(qkv, b, f, dt_bias, a_log, lower_bound, mixed_qkv_bf16, beta_bf16, g, S, F, H, Dk, s),
        "kda_prepare");
}

void layernorm_f16(const half* x, const half* w, const half* b, half* y, int rows, int dim, float eps,
                   Stream s) {
  check(hk_layernorm_f16(x, w, b, y, rows, dim, eps, s), "layernorm_f16");
}

}  // namespace glue
}  // namespace helios
