"""The benchmark configurations at their FULL sizes, through the C ABI, on seeded synthetic inputs with the
configurations' shapes and distributions.

Where the CPU oracle finishes in seconds it is the checker (KDA prefill at 32,768 tokens x 32 heads: the
oracle is linear in tokens; single-row decode at 262,144 tokens of context).  Where it does not (the
4,096-row prefill chunks: teraflops of work), a sample of rows is checked against the oracle, every row
against size-independent properties (a chunk processed in pieces equals the chunk processed at once; the
split count does not change the result)."""
import numpy as np
import pytest
import torch

import hk_oracle as orc
from gpu_util import bits, dev, dev_bf16, dev_f16, frob_rel, max_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 2e-3   # max |a-b| / max |b|: the tolerance the benchmark definition states for this path


def test_config1_kda_prefill_32k_then_1024_decode_steps_vs_oracle():
    T, H, D, extra = 32768, 32, 128, 1024
    inp = synth.kda_inputs(T + extra, H, D, seed=0)
    s0 = np.zeros((1, 1, H, D, D), dtype=np.float32)
    _, o32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, 1, T + extra, H, H, D, D)
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    out = torch.empty(1, T + extra, H, D, dtype=torch.bfloat16, device="cuda")
    g32 = torch.empty(1, T + extra, H, D, dtype=torch.float32, device="cuda")
    path = hk.cuda_recurrent_gated_delta_rule(q[:, :T], g[:, :T], b[:, :T], st, out[:, :T], 1, T, H, H, D, D, 1, None,
                                              True, False, out_f32=g32[:, :T])
    assert path == "chunked"
    torch.cuda.synchronize()
    st_after_prefill = st.clone()
    for s in range(T, T + extra):
        hk.cuda_recurrent_gated_delta_rule(q[:, s:s + 1], g[:, s:s + 1], b[:, s:s + 1], st, out[:, s:s + 1], 1, 1, H, H,
                                           D, D, 1, None, True, False, out_f32=g32[:, s:s + 1])
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    got = g32.cpu().numpy()
    e_pre, e_dec = max_rel(got[:, :T], o32[:, :T]), max_rel(got[:, T:], o32[:, T:])
    e_st = frob_rel(st.cpu().numpy(), o_st)
    print("config 1: prefill out %.2e, decode out %.2e, final state %.2e" % (e_pre, e_dec, e_st))
    assert e_pre < TOL and e_dec < TOL
    assert e_st < 1e-2, "state within 1e-2 relative Frobenius after 33,792 tokens"
    # the bf16 output is the round-toward-zero of the fp32 output, everywhere
    assert np.array_equal(bits(out), (got.view(np.uint32) >> 16).astype(np.uint16))
    # property: the same prefill cut into 8 segments that carry the state gives the same bits
    st2 = dev(s0)
    out2 = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    for s in range(0, T, 4096):
        hk.cuda_recurrent_gated_delta_rule(q[:, s:s + 4096], g[:, s:s + 4096], b[:, s:s + 4096], st2, out2[:, s:s + 4096], 1,
                                           4096, H, H, D, D, 1, None, True, False)
    torch.cuda.synchronize()
    assert torch.equal(out2, out[:, :T]) and torch.equal(st2, st_after_prefill)


def test_config1_conv_32k_windows_vs_oracle():
    """12,288 channels x 32,768 tokens: every output depends on 4 inputs only, so windows of the full-size
    result are checked against the oracle run on the window (its state = the 4 inputs before it)"""
    dim, T = 3 * 32 * 128, 32768
    inp = synth.conv_inputs(T, dim, seed=1)
    x, st, w = dev_bf16(inp["x"]), dev_bf16(inp["state"]), dev_bf16(inp["weight"])
    out = torch.empty(1, T, dim, dtype=torch.bfloat16, device="cuda")
    hk.cuda_causal_conv1d_update(x, st, None, w, None, out, 1, dim, T, 4, 4, True, False)
    torch.cuda.synchronize()
    got = bits(out)
    assert np.array_equal(bits(st)[0], inp["x"][0, :, T - 4:]), "window state = the last 4 inputs"
    for t0, n in [(0, 64), (4093, 40), (16384 - 8, 16), (T - 32, 32)]:
        xs = np.ascontiguousarray(inp["x"][:, :, t0:t0 + n])
        s_in = inp["state"] if t0 == 0 else np.ascontiguousarray(inp["x"][:, :, t0 - 4:t0])
        want, _ = orc.conv1d_update(xs, s_in, inp["weight"], None, 1, dim, n, 4, 4)
        diff = np.abs(got[:, t0:t0 + n].astype(np.int32) - want.astype(np.int32))
        assert diff.max() <= 1 and (diff > 0).mean() < 2e-3   # the device's fast exponential may flip a rounding


@pytest.mark.parametrize("B", [1, 8])
def test_config2_dense_mla_decode_32k_vs_oracle(B):
    L = 32768
    inp = synth.mla_inputs(B * L, B, seed=2)
    base = (np.arange(B) * L).astype(np.int64)
    lens = np.full(B, L, dtype=np.int32)
    scale = 512 ** -0.5
    _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], B, 64, scale, kv_base=base, kv_len=lens)
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    out = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(q, c, out, B, 0, scale=scale, kv_base=dev(base), kv_len=dev(lens), n_keys_hint=L)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    got = synth.f16_bits_to_f32(bits(out))
    assert max_rel(got, o32) < TOL
    # property: the result does not depend on how the keys are split over the SMs
    out1 = torch.empty_like(out)
    hk.mla_dense_prefill(q, c, out1, B, 0, scale=scale, kv_base=dev(base), kv_len=dev(lens), n_split=3, n_keys_hint=L)
    torch.cuda.synchronize()
    assert max_rel(synth.f16_bits_to_f32(bits(out1)), got) < 1e-3


def test_config2_prefill_chunk_4096_rows_after_32k():
    """4,096 causal rows appended to a 32,768-row cache (9.4 TFLOP): sampled rows vs the oracle, all rows vs
    the same chunk processed as 16 pieces of 256 rows"""
    pos, qlen, scale = 32768, 4096, 512 ** -0.5
    inp = synth.mla_inputs(pos + qlen, qlen, seed=3)
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    out = torch.empty(qlen, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(q, c, out, qlen, pos, scale=scale)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    got = synth.f16_bits_to_f32(bits(out))
    for r in (0, 1, 127, 128, 2049, 4095):
        _, o32 = orc.mla_attend(np.ascontiguousarray(inp["q_lat"][r:r + 1]), inp["ckv"], 1, 64, scale, pos_start=pos + r)
        assert max_rel(got[r:r + 1], o32) < TOL, r
    out2 = torch.empty_like(out)
    for r0 in range(0, qlen, 256):
        hk.mla_dense_prefill(q[r0:r0 + 256], c, out2[r0:r0 + 256], 256, pos + r0, scale=scale)
    torch.cuda.synchronize()
    assert max_rel(synth.f16_bits_to_f32(bits(out2)), got) < 1e-3


def _dsa_chain(qi, pk, w, q_pos, ql, ck, m, npools):
    sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")
    idx = torch.empty(m, 512, dtype=torch.int32, device="cuda")
    raw = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
    lo = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    hk.indexer_score(qi, pk, w, q_pos, sc, m, npools)
    hk.dsa_topk(sc, npools, idx, m, npools, 512, 512)
    hk.pool_expand_row(idx, q_pos, raw, m)
    hk.mla_sparse_decode(ql, ck, raw, 2052, lo, m, scale=512 ** -0.5)
    torch.cuda.synchronize()
    return sc, idx, raw, lo


def test_config3_dsa_decode_at_262k_vs_oracle():
    """one decode row at 262,144 tokens of context: 65,536 bf16 pooled keys -> scores -> top-512 pools ->
    2,052 gathered latents -> 64-head MLA; every stage against the oracle"""
    L, npools = 262144, 65536
    ix = synth.indexer_inputs(npools, 1, seed=4, bf16=True)
    ml = synth.mla_inputs(L, 1, seed=5)
    q_pos = np.array([L - 1], dtype=np.int32)
    qi, pk, w = dev_bf16(ix["q_idx"]), dev_bf16(ix["pool_k"]), dev_bf16(ix["w"])
    sc, idx, raw, lo = _dsa_chain(qi, pk, w, dev(q_pos), dev_f16(ml["q_lat"]), dev_f16(ml["ckv"]), 1, npools)
    assert hk.read_device_status() == 0
    o_sc, o_sc32 = orc.indexer_score(ix["q_idx"], ix["pool_k"], ix["w"], q_pos, 1, npools, bf16=True)
    g_sc = synth.f16_bits_to_f32(bits(sc))
    assert np.max(np.abs(g_sc - o_sc32)) <= 4e-3 * max(1.0, np.max(np.abs(o_sc32)))
    # selection and expansion are integer work: bit-exact given the same (device) scores
    assert np.array_equal(idx.cpu().numpy(), orc.dsa_topk(bits(sc), npools, 1, npools, 512, 512))
    assert np.array_equal(raw.cpu().numpy(), orc.pool_expand(idx.cpu().numpy(), q_pos, 1))
    _, o32 = orc.mla_attend(ml["q_lat"], ml["ckv"], 1, 64, 512 ** -0.5, raw_idx=raw.cpu().numpy(), kidx=2052)
    assert max_rel(synth.f16_bits_to_f32(bits(lo)), o32) < TOL


def test_config3_dsa_prefill_chunk_4096_rows_sampled():
    """the same chain as a 4,096-row prefill chunk ending at 262,144: sampled rows against the oracle, all rows
    against the chunk processed in pieces of 512 rows (integer stages bit-exact, attention within tolerance)"""
    L, npools, m = 262144, 65536, 4096
    ix = synth.indexer_inputs(npools, m, seed=6, bf16=True)
    ml = synth.mla_inputs(L, m, seed=7)
    q_pos = (L - m + np.arange(m)).astype(np.int32)
    qi, pk, w = dev_bf16(ix["q_idx"]), dev_bf16(ix["pool_k"]), dev_bf16(ix["w"])
    ql, ck, dq = dev_f16(ml["q_lat"]), dev_f16(ml["ckv"]), dev(q_pos)
    sc, idx, raw, lo = _dsa_chain(qi, pk, w, dq, ql, ck, m, npools)
    assert hk.read_device_status() == 0
    sc_np, idx_np, raw_np, lo_np = bits(sc), idx.cpu().numpy(), raw.cpu().numpy(), synth.f16_bits_to_f32(bits(lo))
    for r in (0, 777, 4095):
        _, o_sc32 = orc.indexer_score(np.ascontiguousarray(ix["q_idx"][r:r + 1]), ix["pool_k"], np.ascontiguousarray(ix["w"][r:r + 1]),
                                      q_pos[r:r + 1], 1, npools, bf16=True)
        g = synth.f16_bits_to_f32(sc_np[r:r + 1])
        vis = np.isfinite(o_sc32)
        assert np.array_equal(np.isfinite(g), vis), "same visibility mask"
        assert np.max(np.abs(g[vis] - o_sc32[vis])) <= 4e-3 * max(1.0, np.max(np.abs(o_sc32[vis])))
        assert np.array_equal(idx_np[r:r + 1], orc.dsa_topk(np.ascontiguousarray(sc_np[r:r + 1]), npools, 1, npools, 512, 512))
        assert np.array_equal(raw_np[r:r + 1], orc.pool_expand(np.ascontiguousarray(idx_np[r:r + 1]), q_pos[r:r + 1], 1))
        _, o32 = orc.mla_attend(np.ascontiguousarray(ml["q_lat"][r:r + 1]), ml["ckv"], 1, 64, 512 ** -0.5,
                                raw_idx=np.ascontiguousarray(raw_np[r:r + 1]), kidx=2052)
        assert max_rel(lo_np[r:r + 1], o32) < TOL
    for r0 in range(0, m, 512):
        s2, i2, w2, l2 = _dsa_chain(qi[r0:r0 + 512], pk, w[r0:r0 + 512], dq[r0:r0 + 512], ql[r0:r0 + 512], ck, 512, npools)
        assert torch.equal(s2, sc[r0:r0 + 512]) and torch.equal(i2, idx[r0:r0 + 512]) and torch.equal(w2, raw[r0:r0 + 512])
        assert max_rel(synth.f16_bits_to_f32(bits(l2)), lo_np[r0:r0 + 512]) < 1e-3
