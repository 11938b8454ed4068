"""helios_glm53flash_b200 - B200 (sm_100a) kernels for the GLM-5.3-Flash trunk-attention hot path.

The product is ``libhelios_b200.so`` (hand-written CUDA behind a C ABI, see ``include/helios_b200.h``)
plus the reference-named C++ launchers (``include/helios_b200_shim.hpp``).  This module is the
Python host side used by the tests and the benchmark: it loads the library with ctypes and exposes
one function per reference launcher, under the reference's names and argument order
(``helios::attn::*`` in src/cuda/attn/attn.cuh, ``helios::aux::*`` in src/cuda/aux/gdn.cuh and
dsa_topk.cuh of the reference tree), taking torch CUDA tensors as device buffers.

There is no CPU path: calling a compute entry point without the library or without a CUDA device
raises.  PyTorch is used for device memory and streams only.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# HELIOS_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("HELIOS_B200_LIB") or os.path.join(_HERE, "libhelios_b200.so")

HK_OK, HK_ERR_INVALID, HK_ERR_UNSUPPORTED, HK_ERR_CUDA, HK_ERR_WORKSPACE, HK_ERR_TIMEOUT = range(6)
HK_F16, HK_BF16, HK_F32 = 0, 1, 2

_c = ctypes
_vp, _i, _f, _sz, _i64 = _c.c_void_p, _c.c_int, _c.c_float, _c.c_size_t, _c.c_int64

# name -> (restype, argtypes): every symbol declared in include/helios_b200.h
SIGNATURES = {
    "hk_status_string": (_c.c_char_p, [_i]),
    "hk_abi_version": (_i, []),
    "hk_conv1d_update": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "hk_kda_recurrent": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "hk_kda_decode_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp]),
    "hk_kda_decode_layer": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _f, _f, _i, _i, _i,
                                 _vp, _vp, _vp]),
    "hk_kda_chunked_set_form": (_i, [_i]),
    "hk_kda_dispatch_is_chunked": (_i, [_i, _i, _i, _i, _i, _i, _i, _i]),
    "hk_kda_chunked_workspace_bytes": (_sz, [_i, _i, _i]),
    "hk_kda_chunked_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "hk_kda_chunked_prefill_gated": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "hk_kda_transpose_cast": (_i, [_vp, _vp, _i, _i, _vp]),
    "hk_kda_gate": (_i, [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp]),
    "hk_kda_prepare": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "hk_kda_cast_conv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "hk_gated_rms_norm": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _c.c_longlong, _i, _f, _f, _i, _i, _i, _vp]),
    "hk_kpool_write": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _vp]),
    "hk_indexer_score": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hk_indexer_score_legacy": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "hk_dsa_topk": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "hk_dsa_topk_expand": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "hk_indexer_select": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "hk_pool_expand": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "hk_mla_partial_bytes": (_sz, [_i, _i64]),
    "hk_mla_auto_splits": (_i, [_i, _i]),
    "hk_mla_sparse": (_i, [_vp, _vp, _i64, _vp, _i, _vp, _i, _i, _f, _i, _vp, _sz, _vp]),
    "hk_mla_sparse_static_max_slots": (_sz, []),
    "hk_mla_sparse_static": (_i, [_vp, _vp, _vp, _i, _vp, _i, _f, _i, _vp]),
    "hk_mla_dense": (_i, [_vp, _vp, _i64, _vp, _vp, _i, _vp, _i, _i, _f, _i, _vp, _sz, _vp]),
    "hk_mla_dense_partial": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "hk_mla_dense_partial_ws": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp, _sz, _vp]),
    "hk_lse_combine": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _vp]),
    "hk_lse_combine_ptrs": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _vp]),
    "hk_peer_signal": (_i, [_vp, _i, _i, _i, _vp]),
    "hk_mla_splitkv_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp, _sz, _vp, _vp, _vp,
                                 _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "hk_mla_splitkv_sparse_step": (_i, [_vp, _vp, _i64, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _sz, _vp,
                                        _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "hk_dsa_select_region_bytes": (_sz, [_i, _i]),
    "hk_dsa_select_splitkv": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "hk_splitkv_region_bytes": (_sz, [_i, _i]),
    "hk_splitkv_region_reset": (_i, [_vp, _i, _i, _vp]),
    "hk_mla_splitkv_heads_step": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _vp, _sz, _vp, _i, _i, _vp, _vp, _i, _i, _vp]),
    "hk_enable_peer_access": (_i, [_i]),
    "hk_peer_region_alloc": (_i, [_sz, _vp, _vp]),
    "hk_peer_region_open": (_i, [_vp, _vp]),
    "hk_peer_region_close": (_i, [_vp]),
    "hk_peer_region_free": (_i, [_vp]),
    "hk_lse_combine_peers": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _vp, _i, _i, _vp]),
    "hk_q_latent": (_i, [_vp, _vp, _vp, _i, _vp]),
    "hk_o_absorb": (_i, [_vp, _vp, _vp, _i, _vp]),
    "hk_wuv_transpose": (_i, [_vp, _vp, _vp]),
    "hk_o_absorb_t": (_i, [_vp, _vp, _vp, _i, _vp]),
    "hk_mla_cache_append": (_i, [_vp, _vp, _vp, _vp, _c.c_longlong, _i, _f, _vp]),
    "hk_layernorm_f16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "hk_mla_decode_prologue": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp]),
    "hk_read_device_status": (_i, [_vp, _i]),
    "hk_tc05_selftest": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
}

_lib = None


class HeliosB200Error(RuntimeError):
    """Raised when an hk_* entry point returns a non-zero status."""

    def __init__(self, name, status):
        self.status = status
        super().__init__("%s failed with status %d (%s)" % (name, status, status_string(status)))


def load_library():
    """Load libhelios_b200.so (built in-tree by ``build.py``); raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libhelios_b200.so is not built (run `python -m helios_glm53flash_b200.build` or "
                "__graft_entry__.build()); this package has no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def status_string(status):
    return load_library().hk_status_string(int(status)).decode()


def _require_cuda():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("helios_glm53flash_b200 needs a CUDA device (sm_100a); there is no CPU path")
    return torch


def _ptr(t):
    return None if t is None else _c.c_void_p(t.data_ptr())


def _stream(stream=None):
    torch = _require_cuda()
    s = torch.cuda.current_stream() if stream is None else stream
    return _c.c_void_p(s.cuda_stream)


def _call(name, *args):
    st = getattr(load_library(), name)(*args)
    if st != HK_OK:
        raise HeliosB200Error(name, st)


def _scratch(nbytes, device, stream=None):
    """A torch-owned scratch buffer (256-byte aligned by the caching allocator).  The kernels that use it run on
    `stream`; when that is not torch's current stream the block is recorded on it, so that the caching allocator
    does not hand it out again while they still run."""
    torch = _require_cuda()
    ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
    if stream is not None and stream != torch.cuda.current_stream():
        ws.record_stream(stream)
    return ws


# ---------------------------------------------------------------------------------------------
# helios::aux
# ---------------------------------------------------------------------------------------------
def cuda_causal_conv1d_update(x, conv_state, slots, weight, bias, out, bsz, dim, seqlen, state_size,
                              K, activation, history, stream=None):
    """helios::aux::cuda_causal_conv1d_update (src/cuda/aux/gdn.cuh:67-83)."""
    _call("hk_conv1d_update", _ptr(x), _ptr(conv_state), _ptr(slots), _ptr(weight), _ptr(bias),
          _ptr(out), bsz, dim, seqlen, state_size, K, int(bool(activation)), int(bool(history)),
          _stream(stream))


def cuda_recurrent_gated_delta_rule(mixed_qkv, g, beta, recurrent_state, core_attn_out, bsz, seqlen,
                                    num_k_heads, num_v_heads, k_head_dim, v_head_dim,
                                    history_stride, slots, channelwise, history, stream=None,
                                    out_f32=None, force_recurrent=False, workspace=None):
    """helios::aux::cuda_recurrent_gated_delta_rule (src/cuda/aux/gdn.cuh:47-65).

    As the C++ launcher of this library does, long channelwise calls go to the chunked tensor-core
    kernel; ``force_recurrent`` keeps the per-token kernel.  ``out_f32`` optionally receives the
    output before bf16 rounding."""
    chunked = not force_recurrent and load_library().hk_kda_dispatch_is_chunked(
        seqlen, num_k_heads, num_v_heads, k_head_dim, v_head_dim, history_stride, int(bool(channelwise)),
        int(bool(history))) != 0
    if chunked:
        nbytes = load_library().hk_kda_chunked_workspace_bytes(bsz, seqlen, num_v_heads)
        ws = workspace if workspace is not None else _scratch(nbytes, mixed_qkv.device, stream)
        st = load_library().hk_kda_chunked_prefill(
            _ptr(mixed_qkv), _ptr(g), _ptr(beta), _ptr(recurrent_state), _ptr(core_attn_out),
            _ptr(out_f32), bsz, seqlen, num_v_heads, _ptr(slots), _ptr(ws), ws.numel(),
            _stream(stream))
        if st == HK_OK:
            return "chunked"
        if st != HK_ERR_UNSUPPORTED:
            raise HeliosB200Error("hk_kda_chunked_prefill", st)
    _call("hk_kda_recurrent", _ptr(mixed_qkv), _ptr(g), _ptr(beta), _ptr(recurrent_state),
          _ptr(core_attn_out), _ptr(out_f32), bsz, seqlen, num_k_heads, num_v_heads, k_head_dim,
          v_head_dim, history_stride, _ptr(slots), int(bool(channelwise)), int(bool(history)),
          _stream(stream))
    return "recurrent"


_decode_tickets = {}


def kda_decode_step(x, conv_state, conv_weight, conv_bias, g, beta, rec_state, out, bsz, num_heads, slots=None,
                    out_f32=None, conv_out=None, stream=None, tickets=None):
    """cuda_causal_conv1d_update(seqlen 1, K = 4, SiLU) + cuda_recurrent_gated_delta_rule(seqlen 1, channelwise) of one
    decoded token (src/engine/runner.cpp:443-471) in one launch; head dim 128.  `tickets`: bsz * num_heads zeroed
    int32 on the device (one buffer per device is kept here when none is given: single-stream use)."""
    if tickets is None:
        torch = _require_cuda()
        key = (x.device.index, bsz * num_heads)
        tickets = _decode_tickets.get(key)
        if tickets is None:
            tickets = _decode_tickets[key] = torch.zeros(bsz * num_heads, dtype=torch.int32, device=x.device)
    _call("hk_kda_decode_step", _ptr(x), _ptr(conv_state), _ptr(conv_weight), _ptr(conv_bias), _ptr(g), _ptr(beta),
          _ptr(rec_state), _ptr(out), _ptr(out_f32), _ptr(conv_out), bsz, num_heads, _ptr(slots), _ptr(tickets),
          _stream(stream))


def kda_decode_layer(x32, conv_state, conv_weight, conv_bias, f, b, dt_bias, a_log, lower_bound, rec_state, out, norm_w,
                     gate_out, y, bsz, num_heads, epsilon=1e-6, gate_act=1, constant_bias=0.0, slots=None, out_f32=None,
                     stream=None, tickets=None):
    """The KDA layer of one decoded token in ONE launch (src/engine/runner.cpp:433-489 runs five): x = bf16(x32)
    (glue::kda_transpose_cast of one row), g / beta from f / b (glue::kda_gate), short conv + SiLU, recurrence, gated RMS
    norm of the output (aux::gated_rms_norm with gate `gate_out`, weight `norm_w`) -> y.  `out` receives the recurrence
    output as the separate calls would leave it.  `tickets`: 2 * bsz * num_heads zeroed int32."""
    if tickets is None:
        torch = _require_cuda()
        key = (x32.device.index, -2 * bsz * num_heads)
        tickets = _decode_tickets.get(key)
        if tickets is None:
            tickets = _decode_tickets[key] = torch.zeros(2 * bsz * num_heads, dtype=torch.int32, device=x32.device)
    _call("hk_kda_decode_layer", _ptr(x32), _ptr(conv_state), _ptr(conv_weight), _ptr(conv_bias), _ptr(f), _ptr(b), _ptr(dt_bias),
          _ptr(a_log), float(lower_bound), _ptr(rec_state), _ptr(out), _ptr(out_f32), _ptr(norm_w), _dtype_code(norm_w),
          _ptr(gate_out), _dtype_code(gate_out), _ptr(y), _dtype_code(y), float(epsilon), float(constant_bias), int(gate_act),
          bsz, num_heads, _ptr(slots), _ptr(tickets), _stream(stream))


def kda_chunked_set_form(form):
    """0: automatic choice between the fused persistent launch and the two-kernel form; 1: always two kernels"""
    _call("hk_kda_chunked_set_form", int(form))


def kda_chunked_workspace_bytes(bsz, seqlen, num_heads):
    return load_library().hk_kda_chunked_workspace_bytes(bsz, seqlen, num_heads)


def kda_chunked_prefill_gated(mixed_qkv, f, b, dt_bias, a_log, lower_bound, recurrent_state, core_attn_out,
                              bsz, seqlen, num_heads, slots=None, stream=None, out_f32=None, workspace=None):
    """Chunked KDA prefill that forms g and beta itself from the raw gate projection ``f``, the raw beta
    logit ``b`` and the layer's ``dt_bias`` / ``a_log`` (the arithmetic of helios::glue::kda_gate,
    src/engine/glue2.cu:347-360), head dim 128."""
    nbytes = load_library().hk_kda_chunked_workspace_bytes(bsz, seqlen, num_heads)
    ws = workspace if workspace is not None else _scratch(nbytes, mixed_qkv.device, stream)
    _call("hk_kda_chunked_prefill_gated", _ptr(mixed_qkv), _ptr(f), _ptr(b), _ptr(dt_bias), _ptr(a_log),
          float(lower_bound), _ptr(recurrent_state), _ptr(core_attn_out), _ptr(out_f32), bsz, seqlen,
          num_heads, _ptr(slots), _ptr(ws), ws.numel(), _stream(stream))


# ---------------------------------------------------------------------------------------------
# helios::glue (KDA producers) and helios::aux::gated_rms_norm (KDA consumer)
# ---------------------------------------------------------------------------------------------
def kda_transpose_cast(dst_bf16, src, S, F, stream=None):
    """helios::glue::kda_transpose_cast (src/engine/glue2.cuh:61): [S][F] f32 -> [F][S] bf16."""
    _call("hk_kda_transpose_cast", _ptr(dst_bf16), _ptr(src), S, F, _stream(stream))


def kda_gate(b, f, dt_bias, a_log, lower_bound, beta_bf16, g, S, H, Dk, stream=None):
    """helios::glue::kda_gate (src/engine/glue2.cuh:62-63)."""
    _call("hk_kda_gate", _ptr(b), _ptr(f), _ptr(dt_bias), _ptr(a_log), float(lower_bound), _ptr(beta_bf16),
          _ptr(g), S, H, Dk, _stream(stream))


def kda_prepare(qkv, b, f, dt_bias, a_log, lower_bound, mixed_qkv_bf16, beta_bf16, g, S, F, H, Dk,
                stream=None):
    """helios::glue::kda_prepare (src/engine/glue2.cuh:64-67)."""
    _call("hk_kda_prepare", _ptr(qkv), _ptr(b), _ptr(f), _ptr(dt_bias), _ptr(a_log), float(lower_bound),
          _ptr(mixed_qkv_bf16), _ptr(beta_bf16), _ptr(g), S, F, H, Dk, _stream(stream))


def kda_cast_conv(x_f32, conv_state, slots, weight, bias, out, bsz, dim, seqlen, activation, stream=None):
    """kda_transpose_cast + cuda_causal_conv1d_update(K = 4) in one pass over token-major fp32 input."""
    _call("hk_kda_cast_conv", _ptr(x_f32), _ptr(conv_state), _ptr(slots), _ptr(weight), _ptr(bias), _ptr(out),
          bsz, dim, seqlen, int(bool(activation)), _stream(stream))


def _dtype_code(t):
    torch = _require_cuda()
    return {torch.float16: HK_F16, torch.bfloat16: HK_BF16, torch.float32: HK_F32}[t.dtype]


def gated_rms_norm(x, w, y, g, rows, dim, epsilon, constant_bias=0.0, w_groups=1, gate_first=False,
                   gate_act=0, stream=None):
    """helios::aux::gated_rms_norm (src/cuda/aux/norm.cuh:71-87); dtypes taken from the tensors."""
    _call("hk_gated_rms_norm", _ptr(x), _ptr(w), _dtype_code(w), _ptr(y), _dtype_code(y), _ptr(g),
          _dtype_code(g), rows, dim, float(epsilon), float(constant_bias), w_groups, int(bool(gate_first)),
          int(gate_act), _stream(stream))


def layernorm_f16(x, w, b, y, rows, dim, eps, stream=None):
    """helios::glue::layernorm_f16 (src/engine/glue2.cuh:73-75)."""
    _call("hk_layernorm_f16", _ptr(x), _ptr(w), _ptr(b), _ptr(y), rows, dim, float(eps), _stream(stream))


def mla_decode_prologue(kv_pre, ln_w, ckv, eps_rms, idx_k, knorm_w, knorm_b, idx_kn, eps_ln, idx_g, raw_ring, raw_rows,
                        pool_k_nt, ape, pos, q_pos_out=None, stream=None):
    """cache append + indexer key layer norm + pooled-key write of ONE new token (src/engine/runner.cpp:569-584) in one
    launch; q_pos_out (device int32[1], optional) receives pos"""
    _call("hk_mla_decode_prologue", _ptr(kv_pre), _ptr(ln_w), _ptr(ckv), float(eps_rms), _ptr(idx_k), _ptr(knorm_w),
          _ptr(knorm_b), _ptr(idx_kn), float(eps_ln), _ptr(idx_g), _ptr(raw_ring), raw_rows, _ptr(pool_k_nt), _ptr(ape),
          int(pos), _ptr(q_pos_out), _stream(stream))


def mla_cache_append(kv_pre, ln_w, ckv, pos, n, eps, ckv_new=None, stream=None):
    """aux::rms_norm (fp32 in, fp16 weight, fp16 out, dim 512) + the copy into the latent cache
    (src/engine/runner.cpp:569-572) as one kernel."""
    _call("hk_mla_cache_append", _ptr(kv_pre), _ptr(ln_w), _ptr(ckv), _ptr(ckv_new), pos, n, float(eps),
          _stream(stream))


def dsa_topk(scores, s_stride, indices, R, T, k, k_pad, t_ptr=None, t_seq=0, stream=None):
    """helios::aux::dsa_topk (src/cuda/aux/dsa_topk.cuh:15-27)."""
    _call("hk_dsa_topk", _ptr(scores), s_stride, _ptr(indices), R, T, k, k_pad, _ptr(t_ptr), t_seq,
          _stream(stream))


def dsa_topk_expand(scores, s_stride, indices, raw_idx, q_pos, R, T, k, after_scorer=False, stream=None):
    """dsa_topk (k_pad = 512) with pool_expand_row folded in: indices [R, 512] and raw_idx [R, 2052] in one kernel"""
    _call("hk_dsa_topk_expand", _ptr(scores), s_stride, _ptr(indices), _ptr(raw_idx), _ptr(q_pos), R, T, k,
          int(bool(after_scorer)), _stream(stream))


def indexer_select(q_idx, pool_k_nt, w, q_pos, scores, indices, raw_idx, m, npools, k=512, stream=None, score_stride=None,
                   n_heads=32):
    """decode-step selection: indexer_score -> top-k with the expansion folded in, two launches (the second a
    programmatic dependent of the first); scores = fp16 workspace [m, score_stride]"""
    torch = _require_cuda()
    dtype = HK_BF16 if q_idx.dtype == torch.bfloat16 else HK_F16
    _call("hk_indexer_select", _ptr(q_idx), _ptr(pool_k_nt), _ptr(w), _ptr(q_pos), _ptr(scores), _ptr(indices),
          _ptr(raw_idx), m, npools, npools if score_stride is None else score_stride, n_heads, dtype, k, _stream(stream))


# ---------------------------------------------------------------------------------------------
# helios::attn
# ---------------------------------------------------------------------------------------------
def kpool_write(idx_k, idx_g, raw_ring, raw_rows, pool_k_nt, ape, pos_start, n_new, stream=None):
    """helios::attn::kpool_write (src/cuda/attn/attn.cuh:80-87)."""
    _call("hk_kpool_write", _ptr(idx_k), _ptr(idx_g), _ptr(raw_ring), raw_rows, _ptr(pool_k_nt),
          _ptr(ape), pos_start, n_new, _stream(stream))


def indexer_score(q_idx, pool_k_nt, w, q_pos, scores, m, npools, stream=None, score_stride=None,
                  n_heads=32):
    """helios::attn::indexer_score (src/cuda/attn/attn.cuh:49-55); fp16 or bf16 keys by tensor dtype."""
    torch = _require_cuda()
    dtype = HK_BF16 if q_idx.dtype == torch.bfloat16 else HK_F16
    _call("hk_indexer_score", _ptr(q_idx), _ptr(pool_k_nt), _ptr(w), _ptr(q_pos), _ptr(scores), m,
          npools, npools if score_stride is None else score_stride, n_heads, dtype, _stream(stream))


indexer_score_mma = indexer_score


def indexer_score_legacy(q_idx, pool_k, w, q_pos, scores, m, npools, pk_stride, stream=None):
    """helios::attn::indexer_score_legacy (src/cuda/attn/attn.cuh:46-48)."""
    _call("hk_indexer_score_legacy", _ptr(q_idx), _ptr(pool_k), _ptr(w), _ptr(q_pos), _ptr(scores),
          m, npools, pk_stride, _stream(stream))


def pool_expand(pool_idx, q_pos, raw_idx, m, cur_pos, stream=None, n_sel=512):
    """helios::attn::pool_expand (src/cuda/attn/attn.cuh:60-65): one cur_pos for every row."""
    _call("hk_pool_expand", _ptr(pool_idx), None, _ptr(raw_idx), m, cur_pos, n_sel, _stream(stream))


def pool_expand_row(pool_idx, q_pos, raw_idx, m, stream=None, n_sel=512):
    """helios::attn::pool_expand_row (src/cuda/attn/attn.cuh:67-72)."""
    _call("hk_pool_expand", _ptr(pool_idx), _ptr(q_pos), _ptr(raw_idx), m, 0, n_sel, _stream(stream))


def mla_auto_splits(m, n_keys):
    return load_library().hk_mla_auto_splits(m, n_keys)


def mla_partial_bytes(n_split, rows):
    return load_library().hk_mla_partial_bytes(n_split, rows)


def _cache_rows(ckv, ckv_rows):
    """rows of a [rows][512] cache tensor (0 = unknown, for buffers that are not laid out that way)"""
    if ckv_rows is not None:
        return int(ckv_rows)
    return int(ckv.numel() // 512) if ckv.dim() >= 1 and ckv.numel() % 512 == 0 else 0


def mla_sparse_decode(q_lat, ckv, raw_idx, kidx, lat_out, m, stream=None, scale=0.0625, n_heads=64,
                      n_split=0, workspace=None, ckv_rows=None):
    """helios::attn::mla_sparse_decode (src/cuda/attn/attn.cuh:93-99) with explicit scale / heads; the cache's row
    count is taken from the tensor, so row numbers beyond it are skipped instead of read."""
    if n_split <= 0:
        n_split = mla_auto_splits(m, kidx)
    ws = workspace
    if n_split > 1 and ws is None:
        ws = _scratch(mla_partial_bytes(n_split, m * n_heads), q_lat.device, stream)
    _call("hk_mla_sparse", _ptr(q_lat), _ptr(ckv), _cache_rows(ckv, ckv_rows), _ptr(raw_idx), kidx, _ptr(lat_out), m, n_heads,
          float(scale), n_split, _ptr(ws), 0 if ws is None else ws.numel(), _stream(stream))


def mla_sparse_decode_static(q_lat, ckv, raw_idx, kidx, lat_out, m, stream=None, scale=0.0625, n_split=0):
    """Sparse MLA decode for callers that cannot allocate: same result as mla_sparse_decode, but the
    split partials use the library's built-in ~8 MiB device array (n_split * m <= 64), so neither
    this wrapper nor the library allocates anything.  Calls on one device share that array: do not
    let two of them overlap on the GPU."""
    _call("hk_mla_sparse_static", _ptr(q_lat), _ptr(ckv), _ptr(raw_idx), kidx, _ptr(lat_out), m, float(scale),
          n_split, _stream(stream))


def mla_dense_prefill(q_lat, ckv, lat_out, qlen, pos_start, stream=None, scale=0.0625, n_heads=64,
                      kv_base=None, kv_len=None, n_split=0, workspace=None, n_keys_hint=None, ckv_rows=None):
    """helios::attn::mla_dense_prefill (src/cuda/attn/attn.cuh:104-108); qlen = 1 is dense decode.
    kv_base / kv_len (device int64 / int32 per row) select per-row cache ranges (batched decode)."""
    if n_split <= 0:
        n_split = mla_auto_splits(qlen, n_keys_hint if n_keys_hint else pos_start + qlen)
    ws = workspace
    if n_split > 1 and ws is None:
        ws = _scratch(mla_partial_bytes(n_split, qlen * n_heads), q_lat.device, stream)
    _call("hk_mla_dense", _ptr(q_lat), _ptr(ckv), _cache_rows(ckv, ckv_rows), _ptr(kv_base), _ptr(kv_len), pos_start,
          _ptr(lat_out), qlen, n_heads, float(scale), n_split, _ptr(ws),
          0 if ws is None else ws.numel(), _stream(stream))


def mla_dense_partial(q_lat, ckv, kv_base, kv_len, pos_start, part_m, part_l, part_acc, m,
                      n_heads=64, scale=0.0625, stream=None):
    """One split's un-normalised (m, l, acc) partial - the unit of split-KV across GPUs."""
    _call("hk_mla_dense_partial", _ptr(q_lat), _ptr(ckv), _ptr(kv_base), _ptr(kv_len), pos_start,
          _ptr(part_m), _ptr(part_l), _ptr(part_acc), m, n_heads, float(scale), _stream(stream))


def mla_dense_partial_ws(q_lat, ckv, kv_base, kv_len, pos_start, part_m, part_l, part_acc, m, n_keys_hint,
                         n_heads=64, scale=0.0625, n_split=0, workspace=None, stream=None):
    """One partial set computed with every SM of this GPU (local splits merged on the GPU)."""
    if n_split <= 0:
        n_split = mla_auto_splits(m, n_keys_hint)
    ws = workspace
    if n_split > 1 and ws is None:
        ws = _scratch(mla_partial_bytes(n_split, m * n_heads), q_lat.device, stream)
    _call("hk_mla_dense_partial_ws", _ptr(q_lat), _ptr(ckv), _ptr(kv_base), _ptr(kv_len), pos_start, _ptr(part_m),
          _ptr(part_l), _ptr(part_acc), m, n_heads, float(scale), n_split, n_keys_hint, _ptr(ws),
          0 if ws is None else ws.numel(), _stream(stream))


def lse_combine(part_m, part_l, part_acc, n_split, rows, out, stream=None):
    """Standalone split-KV log-sum-exp combine (the reference merges in-kernel, attn.cu:462-481)."""
    _call("hk_lse_combine", _ptr(part_m), _ptr(part_l), _ptr(part_acc), n_split, rows, _ptr(out),
          _stream(stream))


def lse_combine_ptrs(ptrs_m, ptrs_l, ptrs_acc, n_split, rows, out, stream=None):
    """Combine over per-split pointers (device int64 tensors of addresses, e.g. peer buffers)."""
    _call("hk_lse_combine_ptrs", _ptr(ptrs_m), _ptr(ptrs_l), _ptr(ptrs_acc), n_split, rows,
          _ptr(out), _stream(stream))


def peer_signal(flag_ptrs, n_ranks, my_rank, epoch, stream=None):
    """Publish `epoch` into slot my_rank of every rank's flag array (flag_ptrs: device int64 tensor)."""
    _call("hk_peer_signal", _ptr(flag_ptrs), n_ranks, my_rank, epoch, _stream(stream))


def mla_splitkv_step(q_lat, ckv_shard, kv_base, kv_len, parts0, parts1, m, n_heads, scale, n_split, n_keys_hint,
                     workspace, flag_ptrs, ptrs_m, ptrs_l, ptrs_acc, n_ranks, my_rank, step_ctr, local_flags, out,
                     max_wait_ms=1000, signal=True, stream=None):
    """partial over the local shard + signal + bounded-wait combine over all ranks, one host call;
    parts0 / parts1 = (m, l, acc) tensors of this rank's two exchange sets, step_ctr = device int32[1]"""
    _call("hk_mla_splitkv_step", _ptr(q_lat), _ptr(ckv_shard), _ptr(kv_base), _ptr(kv_len), _ptr(parts0[0]),
          _ptr(parts0[1]), _ptr(parts0[2]), _ptr(parts1[0]), _ptr(parts1[1]), _ptr(parts1[2]), m, n_heads, float(scale),
          n_split, n_keys_hint, _ptr(workspace), workspace.numel(), _ptr(flag_ptrs), _ptr(ptrs_m), _ptr(ptrs_l),
          _ptr(ptrs_acc), n_ranks, my_rank, _ptr(step_ctr), _ptr(local_flags), _ptr(out), max_wait_ms,
          int(bool(signal)), _stream(stream))


def mla_splitkv_sparse_step(q_lat, ckv_shard, ckv_rows, raw_local, kidx, parts0, parts1, m, n_heads, scale, n_split,
                            workspace, flag_ptrs, ptrs_m, ptrs_l, ptrs_acc, n_ranks, my_rank, step_ctr, local_flags, out,
                            max_wait_ms=1000, signal=True, stream=None):
    """mla_splitkv_step over gathered rows of the local slice (raw_local: rows relative to the slice, negative = skipped)"""
    _call("hk_mla_splitkv_sparse_step", _ptr(q_lat), _ptr(ckv_shard), int(ckv_rows), _ptr(raw_local), kidx, _ptr(parts0[0]),
          _ptr(parts0[1]), _ptr(parts0[2]), _ptr(parts1[0]), _ptr(parts1[1]), _ptr(parts1[2]), m, n_heads, float(scale),
          n_split, _ptr(workspace), workspace.numel(), _ptr(flag_ptrs), _ptr(ptrs_m), _ptr(ptrs_l), _ptr(ptrs_acc),
          n_ranks, my_rank, _ptr(step_ctr), _ptr(local_flags), _ptr(out), max_wait_ms, int(bool(signal)), _stream(stream))


def dsa_select_region_bytes(m, n_ranks):
    return load_library().hk_dsa_select_region_bytes(m, n_ranks)


def dsa_select_splitkv(scores, s_stride, n_local_pools, pool_base, local_idx, cand_bases, local_cand_base, n_ranks,
                       my_rank, m, k, q_pos, row_base, n_local_rows, sel_pools, raw_local, step_ctr, max_wait_ms=1000,
                       signal=True, phases=3, stream=None):
    """local top-k -> candidate exchange -> selection over all ranks' candidates -> rows of the local slice;
    cand_bases = device int64 [n_ranks] (candidate areas as mapped here), local_cand_base = address of the own one"""
    _call("hk_dsa_select_splitkv", _ptr(scores), s_stride, n_local_pools, pool_base, _ptr(local_idx), _ptr(cand_bases),
          _c.c_void_p(int(local_cand_base)), n_ranks, my_rank, m, k, _ptr(q_pos), row_base, n_local_rows,
          _ptr(sel_pools), _ptr(raw_local), _ptr(step_ctr), max_wait_ms, int(bool(signal)), int(phases), _stream(stream))


def enable_peer_access(peer_device):
    """kernels of the current device may then dereference memory of `peer_device`"""
    _call("hk_enable_peer_access", int(peer_device))


class DeviceRegion:
    """Raw device memory that is not owned by torch (an exchange region or a peer's mapping of one).
    as_tensor(offset, nbytes, dtype) gives a torch view of a slice (through __cuda_array_interface__)."""

    def __init__(self, ptr, nbytes):
        self.ptr, self.nbytes = int(ptr), int(nbytes)

    def data_ptr(self):
        return self.ptr

    def as_tensor(self, offset, nbytes, dtype):
        torch = _require_cuda()

        class _View:
            pass
        v = _View()
        v.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (self.ptr + int(offset), False),
                                      "version": 2, "strides": None}
        return torch.as_tensor(v, device="cuda").view(dtype)


def peer_region_alloc(nbytes):
    """(DeviceRegion, 64-byte handle) of zeroed device memory that other processes can map"""
    p, h = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    _call("hk_peer_region_alloc", int(nbytes), ctypes.byref(p), h)
    return DeviceRegion(p.value, nbytes), h.raw


def peer_region_open(handle, nbytes):
    """map another process's region for kernels of the CURRENT device"""
    p = ctypes.c_void_p()
    _call("hk_peer_region_open", ctypes.create_string_buffer(handle, 64), ctypes.byref(p))
    return DeviceRegion(p.value, nbytes)


def peer_region_close(region):
    _call("hk_peer_region_close", ctypes.c_void_p(region.ptr))


def peer_region_free(region):
    _call("hk_peer_region_free", ctypes.c_void_p(region.ptr))


def lse_combine_peers(ptrs_m, ptrs_l, ptrs_acc, n_split, rows, out, local_flags, epoch, max_wait_ms=1000,
                      stream=None):
    """Bounded wait on this GPU's flag array, then combine over peer-mapped partial buffers."""
    _call("hk_lse_combine_peers", _ptr(ptrs_m), _ptr(ptrs_l), _ptr(ptrs_acc), n_split, rows, _ptr(out),
          _ptr(local_flags), epoch, max_wait_ms, _stream(stream))


def q_latent(q_nope, kv_b, q_lat, m, stream=None):
    _call("hk_q_latent", _ptr(q_nope), _ptr(kv_b), _ptr(q_lat), m, _stream(stream))


q_latent_t = q_latent


def o_absorb(lat_out, kv_b, o, m, stream=None):
    _call("hk_o_absorb", _ptr(lat_out), _ptr(kv_b), _ptr(o), m, _stream(stream))


def wuv_transpose(kv_b, wuv_t, stream=None):
    _call("hk_wuv_transpose", _ptr(kv_b), _ptr(wuv_t), _stream(stream))


def o_absorb_t(lat_out, wuv_t, o, nrows, stream=None):
    _call("hk_o_absorb_t", _ptr(lat_out), _ptr(wuv_t), _ptr(o), nrows, _stream(stream))


def read_device_status(reset=True):
    """0 unless a bounded device-side wait expired since the last reset (synchronises)."""
    _require_cuda()
    v = _c.c_int(0)
    _call("hk_read_device_status", _c.byref(v), int(reset))
    return v.value


def tc05_selftest(a, b, M, N, K, b_layout, stream=None):
    """Raw TMEM accumulator [128][N] of D = A * B through the tcgen05 helper layer."""
    torch = _require_cuda()
    d = torch.zeros(128, N, dtype=torch.float32, device=a.device)
    status = torch.zeros(4, dtype=torch.int32, device=a.device)
    _call("hk_tc05_selftest", _ptr(a), _ptr(b), _ptr(d), M, N, K, b_layout, _ptr(status),
          _stream(stream))
    return d, status
