"""ctypes front end of oracle/_ref/libhelios_ref.so: the reference's own CUDA kernels, built from
the reference tree by `make -C oracle ref` (prebuilt before the tests travel to a GPU machine).
Checker only.  available() is False when the library was not built."""
import ctypes
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "oracle", "_ref", "libhelios_ref.so")
_lib = None


def available():
    return os.path.exists(SO)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(SO)
    return _lib


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _s():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def conv1d_update(x, state, slots, w, bias, out, bsz, dim, seqlen, state_size, K, act, history):
    lib().ref_conv1d_update(_p(x), _p(state), _p(slots), _p(w), _p(bias), _p(out), bsz, dim, seqlen,
                            state_size, K, int(act), int(history), _s())


def kda_recurrent(qkv, g, beta, state, out, bsz, seqlen, Hk, Hv, dk, dv, history_stride, slots,
                  channelwise, history):
    lib().ref_kda_recurrent(_p(qkv), _p(g), _p(beta), _p(state), _p(out), bsz, seqlen, Hk, Hv, dk, dv,
                            history_stride, _p(slots), int(channelwise), int(history), _s())


def kpool_write(idx_k, idx_g, ring, raw_rows, pool_k_nt, ape, pos_start, n_new):
    lib().ref_kpool_write(_p(idx_k), _p(idx_g), _p(ring), raw_rows, _p(pool_k_nt), _p(ape), pos_start,
                          n_new, _s())


def indexer_score(q, pk, w, q_pos, scores, m, npools):
    lib().ref_indexer_score(_p(q), _p(pk), _p(w), _p(q_pos), _p(scores), m, npools, _s())


def indexer_score_legacy(q, pk, w, q_pos, scores, m, npools, pk_stride):
    lib().ref_indexer_score_legacy(_p(q), _p(pk), _p(w), _p(q_pos), _p(scores), m, npools, pk_stride, _s())


def dsa_topk(scores, s_stride, indices, R, T, k, k_pad, t_seq=0):
    lib().ref_dsa_topk(_p(scores), s_stride, _p(indices), R, T, k, k_pad, t_seq, _s())


def pool_expand(pool_idx, q_pos, raw, m, cur_pos):
    lib().ref_pool_expand(_p(pool_idx), _p(q_pos), _p(raw), m, cur_pos, _s())


def pool_expand_row(pool_idx, q_pos, raw, m):
    lib().ref_pool_expand_row(_p(pool_idx), _p(q_pos), _p(raw), m, _s())


def mla_sparse_decode(q_lat, ckv, raw_idx, kidx, lat_out, m):
    lib().ref_mla_sparse_decode(_p(q_lat), _p(ckv), _p(raw_idx), kidx, _p(lat_out), m, _s())


def mla_dense_prefill(q_lat, ckv, lat_out, qlen, pos_start):
    lib().ref_mla_dense_prefill(_p(q_lat), _p(ckv), _p(lat_out), qlen, pos_start, _s())


def q_latent(q_nope, kv_b, q_lat, m):
    lib().ref_q_latent(_p(q_nope), _p(kv_b), _p(q_lat), m, _s())


def o_absorb(lat_out, kv_b, o, m):
    lib().ref_o_absorb(_p(lat_out), _p(kv_b), _p(o), m, _s())


def q_latent_t(q_nope, kv_b, q_lat, n):
    lib().ref_q_latent_t(_p(q_nope), _p(kv_b), _p(q_lat), n, _s())


def wuv_transpose(kv_b, wuv_t):
    lib().ref_wuv_transpose(_p(kv_b), _p(wuv_t), _s())


def o_absorb_t(lat_out, wuv_t, o, n):
    lib().ref_o_absorb_t(_p(lat_out), _p(wuv_t), _p(o), n, _s())


def kda_transpose_cast(dst_bf16, src, S, F):
    lib().ref_kda_transpose_cast(_p(dst_bf16), _p(src), S, F, _s())


def kda_gate(b, f, dt_bias, a_log, lower_bound, beta_bf16, g, S, H, Dk):
    lib().ref_kda_gate(_p(b), _p(f), _p(dt_bias), _p(a_log), ctypes.c_float(lower_bound), _p(beta_bf16), _p(g),
                       S, H, Dk, _s())


def kda_prepare(qkv, b, f, dt_bias, a_log, lower_bound, mixed_qkv_bf16, beta_bf16, g, S, F, H, Dk):
    lib().ref_kda_prepare(_p(qkv), _p(b), _p(f), _p(dt_bias), _p(a_log), ctypes.c_float(lower_bound),
                          _p(mixed_qkv_bf16), _p(beta_bf16), _p(g), S, F, H, Dk, _s())


def gated_rms_norm(x, w, y, g, rows, dim, epsilon, constant_bias=0.0, w_groups=1, gate_first=False, gate_act=0):
    import torch
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
    lib().ref_gated_rms_norm(_p(x), _p(w), code[w.dtype], _p(y), code[y.dtype], _p(g), code[g.dtype], rows, dim,
                             ctypes.c_float(epsilon), ctypes.c_float(constant_bias), w_groups, int(gate_first),
                             int(gate_act), _s())


def rms_norm(x, w, y, rows, dim, epsilon):
    import torch
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
    lib().ref_rms_norm(_p(x), code[x.dtype], _p(w), code[w.dtype], _p(y), code[y.dtype], rows, dim,
                       ctypes.c_float(epsilon), _s())


def layernorm_f16(x, w, b, y, rows, dim, eps):
    lib().ref_layernorm_f16(_p(x), _p(w), _p(b), _p(y), rows, dim, ctypes.c_float(eps), _s())
