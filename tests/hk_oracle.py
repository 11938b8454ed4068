"""ctypes front end of oracle/liboracle.so (the CPU restatement; checker only)."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_lib = None
_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def lib():
    global _lib
    if _lib is None:
        so = os.path.join(ORACLE_DIR, "liboracle.so")
        src = os.path.join(ORACLE_DIR, "oracle.cpp")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", ORACLE_DIR, "liboracle.so"], stdout=subprocess.DEVNULL)
        _lib = ctypes.CDLL(so)
        _lib.orc_get_threads.restype = _i
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return ctypes.c_void_p(a.ctypes.data)


def threads():
    return lib().orc_get_threads()


def set_threads(n):
    lib().orc_set_threads(int(n))


def conv1d_update(x, state, w, bias, bsz, dim, seqlen, state_size, K, activation=True, history=False,
                  slots=None):
    """returns (out bf16 bits [bsz][T][dim], new state)"""
    out = np.empty((bsz, seqlen, dim), dtype=np.uint16)
    st = state.copy()
    rc = lib().orc_conv1d_update(_p(x), _p(st), _p(slots), _p(w), _p(bias), _p(out), bsz, dim, seqlen,
                                 state_size, K, int(activation), int(history))
    assert rc == 0
    return out, st


def kda_recurrent(mixed_qkv, g, beta, state, bsz, seqlen, Hk, Hv, dk, dv, history_stride=1, slots=None,
                  channelwise=True, history=False, acc64=False):
    """returns (out bf16 bits, out f32, new state)"""
    out = np.empty((bsz, seqlen, Hv, dv), dtype=np.uint16)
    out32 = np.empty((bsz, seqlen, Hv, dv), dtype=np.float32)
    st = state.copy()
    rc = lib().orc_kda_recurrent(_p(mixed_qkv), _p(g), _p(beta), _p(st), _p(out), _p(out32), bsz, seqlen,
                                 Hk, Hv, dk, dv, history_stride, _p(slots), int(channelwise),
                                 int(history), int(acc64))
    assert rc == 0
    return out, out32, st


def kpool_write(idx_k, idx_g, ring, raw_rows, pool_k_nt, ape, pos_start, n_new):
    rc = lib().orc_kpool_write(_p(idx_k), _p(idx_g), _p(ring), raw_rows, _p(pool_k_nt), _p(ape),
                               pos_start, n_new)
    assert rc == 0


def indexer_score(q_idx, pool_k_nt, w, q_pos, m, npools, n_heads=32, bf16=False, acc64=False):
    sc = np.empty((m, npools), dtype=np.uint16)
    sc32 = np.empty((m, npools), dtype=np.float32)
    rc = lib().orc_indexer_score(_p(q_idx), _p(pool_k_nt), _p(w), _p(q_pos), _p(sc), _p(sc32), m, npools,
                                 n_heads, int(bf16), int(acc64))
    assert rc == 0
    return sc, sc32


def dsa_topk(scores, s_stride, R, T, k, k_pad):
    idx = np.empty((R, k_pad), dtype=np.int32)
    rc = lib().orc_dsa_topk(_p(scores), s_stride, _p(idx), R, T, k, k_pad)
    assert rc == 0
    return idx


def pool_expand(pool_idx, q_pos, m, cur_pos=0, n_sel=512):
    raw = np.empty((m, n_sel * 4 + 4), dtype=np.int32)
    rc = lib().orc_pool_expand(_p(pool_idx), _p(q_pos), _p(raw), m, cur_pos, n_sel)
    assert rc == 0
    return raw


def mla_attend(q_lat, ckv, m, n_heads, scale, raw_idx=None, kidx=0, kv_base=None, kv_len=None,
               pos_start=0, partial=False):
    """returns (out f16 bits, out f32[, (m, l, acc)])"""
    out = np.empty((m, n_heads, 512), dtype=np.uint16)
    out32 = np.empty((m, n_heads, 512), dtype=np.float32)
    pm = pl = pa = None
    if partial:
        pm = np.empty((m * n_heads,), dtype=np.float32)
        pl = np.empty((m * n_heads,), dtype=np.float32)
        pa = np.empty((m * n_heads, 512), dtype=np.float32)
    lib().orc_mla_attend.argtypes = [_vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _f]
    rc = lib().orc_mla_attend(_p(q_lat), _p(ckv), _p(raw_idx), kidx, _p(kv_base), _p(kv_len), pos_start,
                              _p(out), _p(out32), _p(pm), _p(pl), _p(pa), m, n_heads, float(scale))
    assert rc == 0
    return (out, out32, (pm, pl, pa)) if partial else (out, out32)


def lse_combine(part_m, part_l, part_acc, n_split, rows):
    out = np.empty((rows, 512), dtype=np.uint16)
    out32 = np.empty((rows, 512), dtype=np.float32)
    lib().orc_lse_combine.argtypes = [_vp, _vp, _vp, _i, ctypes.c_int64, _vp, _vp]
    rc = lib().orc_lse_combine(_p(part_m), _p(part_l), _p(part_acc), n_split, rows, _p(out), _p(out32))
    assert rc == 0
    return out, out32


def q_latent(q_nope, kv_b, m, n_heads=64):
    out = np.empty((m, n_heads, 512), dtype=np.uint16)
    assert lib().orc_q_latent(_p(q_nope), _p(kv_b), _p(out), m, n_heads) == 0
    return out


def o_absorb(lat_out, kv_b, m, n_heads=64):
    out = np.empty((m, n_heads, 256), dtype=np.uint16)
    assert lib().orc_o_absorb(_p(lat_out), _p(kv_b), _p(out), m, n_heads) == 0
    return out


def kda_prepare(qkv, b, f, dt_bias, a_log, lower_bound, S, F, H, Dk):
    """returns (mixed bf16 bits [F][S], beta bf16 bits [S][H], g f32 [S][H][Dk]); any of qkv / b / f may be None"""
    mixed = np.empty((F, S), dtype=np.uint16) if qkv is not None else None
    beta = np.empty((S, H), dtype=np.uint16) if b is not None else None
    g = np.empty((S, H, Dk), dtype=np.float32) if f is not None else None
    rc = lib().orc_kda_prepare(_p(qkv), _p(b), _p(f), _p(dt_bias), _p(a_log), _f(lower_bound), _p(mixed), _p(beta),
                               _p(g), S, F, H, Dk)
    assert rc == 0
    return mixed, beta, g


def gated_rms_norm(x, w, g, rows, dim, eps, y_f32=False, constant_bias=0.0, w_groups=1, gate_first=False,
                   gate_act=0):
    """x bf16 bits; w / g float32 arrays or uint16 (bf16 bits); returns y as f16 bits or float32"""
    y = np.empty((rows, dim), dtype=np.float32 if y_f32 else np.uint16)
    rc = lib().orc_gated_rms_norm(_p(x), _p(w), int(w.dtype == np.uint16), _p(y), int(y_f32), _p(g),
                                  int(g.dtype == np.uint16), ctypes.c_int64(rows), dim, _f(eps), _f(constant_bias),
                                  w_groups, int(gate_first), int(gate_act))
    assert rc == 0
    return y


def mla_cache_append(kv_pre, ln_w, ckv, pos, n, eps):
    """normalises the n rows of kv_pre into ckv (f16 bits, modified in place) at rows pos.."""
    rc = lib().orc_mla_cache_append(_p(kv_pre), _p(ln_w), _p(ckv), ctypes.c_int64(pos), n, _f(eps))
    assert rc == 0
    return ckv


def layernorm_f16(x, w, b, rows, dim, eps):
    y = np.empty((rows, dim), dtype=np.uint16)
    rc = lib().orc_layernorm_f16(_p(x), _p(w), _p(b), _p(y), rows, dim, _f(eps))
    assert rc == 0
    return y
