"""End-to-end compositions of the hot path through the C ABI, against the CPU oracle (and the reference's own
kernels where they apply):

* benchmark configuration 0 as one test: a single KDA layer, batch 1, 32 heads x 128, a 512-token prefill and
  16 decode steps from zero state, the short conv FEEDING the recurrence;
* a cut-down hybrid stack (2 KDA layers + 1 MLA layer) in the engine's call order: 8,192 tokens in two chunks of
  4,096 and 16 decode steps, with the KDA state, the latent cache, the ring and the pooled keys carried across
  chunks, in both forms of the KDA layer (fused entry points, and the reference's call sequence).
"""
import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bf16_ulp_diff, bits, dev, dev_bf16, frob_rel, max_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth
from helios_glm53flash_b200.trunk import KIDX, TrunkAttention

pytestmark = pytest.mark.gpu


def test_config0_kda_layer_prefill_512_then_16_decode_steps_conv_feeding_recurrence():
    T, steps, H, D = 512, 16, 32, 128
    dim, N = 3 * H * D, 512 + 16
    r = synth.rng(0)
    # pre-conv q|k|v ~ N(0,1) channel-major, conv weights N(0, 0.1), beta = sigmoid(N(0,1)), g = -softplus(N(0,1))
    x = synth.f32_to_bf16_bits(r.standard_normal((dim, N), dtype=np.float32))
    w = synth.f32_to_bf16_bits((0.1 * r.standard_normal((dim, 4), dtype=np.float32)).astype(np.float32))
    gates = synth.kda_gates(N, H, D, seed=0)
    g_np, beta_np = gates["g"], gates["beta"]
    cst0 = np.zeros((1, dim, 4), dtype=np.uint16)
    s0 = np.zeros((1, 1, H, D, D), dtype=np.float32)
    # ---- oracle: conv over all 528 tokens, then the recurrence ----
    o_qkv, o_cst = orc.conv1d_update(x.reshape(1, dim, N), cst0, w, None, 1, dim, N, 4, 4)
    _, o_32, o_st = orc.kda_recurrent(o_qkv, g_np, beta_np, s0, 1, N, H, H, D, D)
    # ---- this library: prefill call pair, then 16 single-token steps (one launch each) ----
    xd, wd, gd, bd = dev_bf16(x), dev_bf16(w), dev(g_np), dev_bf16(beta_np)
    cs, st = dev_bf16(cst0), dev(s0)
    qkv = torch.empty(1, N, dim, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, N, H, D, dtype=torch.bfloat16, device="cuda")
    o32 = torch.empty(1, N, H, D, dtype=torch.float32, device="cuda")
    x_pre = xd[:, :T].contiguous()
    hk.cuda_causal_conv1d_update(x_pre.view(1, dim, T), cs, None, wd, None, qkv[:, :T], 1, dim, T, 4, 4, True, False)
    assert hk.cuda_recurrent_gated_delta_rule(qkv[:, :T], gd[:, :T], bd[:, :T], st, out[:, :T], 1, T, H, H, D, D, 1, None,
                                              True, False, out_f32=o32[:, :T]) == "chunked"
    for s in range(T, N):
        hk.kda_decode_step(xd[:, s].contiguous().view(1, dim), cs, wd, None, gd[:, s], bd[:, s], st, out[:, s], 1, H,
                           out_f32=o32[:, s], conv_out=qkv[:, s])
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    assert bf16_ulp_diff(o_qkv, bits(qkv)).max() <= 1, "conv + SiLU output"
    assert np.array_equal(o_cst, bits(cs)), "conv window after 528 tokens"
    # the recurrence is compared on what the GPU conv produced (the oracle's conv may differ in the last bf16 bit)
    _, o_32g, o_stg = orc.kda_recurrent(bits(qkv), g_np, beta_np, s0, 1, N, H, H, D, D)
    assert max_rel(o32.cpu().numpy(), o_32g) < 2e-3 and frob_rel(st.cpu().numpy(), o_stg) < 1e-2
    assert frob_rel(st.cpu().numpy(), o_st) < 1e-2, "state after prefill + decode, conv included, vs the oracle end to end"
    # ---- the reference's own kernels on the same inputs: per-token kernel with seqlen = 512, then 16 x seqlen = 1 ----
    if ref.available():
        cs_r, st_r = dev_bf16(cst0), dev(s0)
        qkv_r = torch.empty_like(qkv)
        out_r = torch.empty_like(out)
        ref.conv1d_update(x_pre.view(1, dim, T), cs_r, None, wd, None, qkv_r[:, :T], 1, dim, T, 4, 4, True, False)
        ref.kda_recurrent(qkv_r[:, :T], gd[:, :T], bd[:, :T], st_r, out_r[:, :T], 1, T, H, H, D, D, 1, None, True, False)
        for s in range(T, N):
            xs = xd[:, s].contiguous()
            ref.conv1d_update(xs.view(1, dim, 1), cs_r, None, wd, None, qkv_r[:, s:s + 1], 1, dim, 1, 4, 4, True, False)
            ref.kda_recurrent(qkv_r[:, s:s + 1], gd[:, s:s + 1].contiguous(), bd[:, s:s + 1].contiguous(), st_r,
                              out_r[:, s:s + 1], 1, 1, H, H, D, D, 1, None, True, False)
        torch.cuda.synchronize()
        assert np.array_equal(bits(qkv_r), bits(qkv)), "conv output: same bits as the reference kernel"
        assert np.array_equal(bits(cs_r), bits(cs))
        assert frob_rel(st.cpu().numpy(), st_r.cpu().numpy()) < 1e-2
        assert frob_rel(o_stg, st_r.cpu().numpy()) < 1e-2, "oracle pinned to the reference kernels"
        a, b = out.float().cpu().numpy(), out_r.float().cpu().numpy()
        assert max_rel(a, b) < 8e-3, "bf16 (round toward zero) outputs within one unit of the reference's"


def _kda_oracle(tr, total_rows_per_call):
    """oracle replay of one KDA layer of the trunk over the same sequence of calls"""
    ki, H, D, dim = tr.kda_in, tr.H, tr.D, tr.dim
    x32, f, b = (ki[k].cpu().numpy() for k in ("x32", "f", "b"))
    dtb, alog, lb = ki["dt_bias"].cpu().numpy(), ki["a_log"].cpu().numpy(), ki["lower_bound"]
    w = bits(ki["conv_w"])
    cst = np.zeros((1, dim, 4), dtype=np.uint16)
    st = np.zeros((1, 1, H, D, D), dtype=np.float32)
    recs, ys = [], []
    for n in total_rows_per_call:
        mixed, beta, g = orc.kda_prepare(np.ascontiguousarray(x32[0, :n]), np.ascontiguousarray(b[0, :n]),
                                         np.ascontiguousarray(f[0, :n]), dtb, alog, lb, n, dim, H, D)
        qkv, cst = orc.conv1d_update(mixed.reshape(1, dim, n), cst, w, None, 1, dim, n, 4, 4)
        rec16, rec32, st = orc.kda_recurrent(qkv, g.reshape(1, n, H, D), beta.reshape(1, n, H), st, 1, n, H, H, D, D)
        recs.append(rec32)
        ys.append(rec16)
    return recs, ys, st, cst


@pytest.mark.parametrize("fused", [True, False])
def test_cut_down_hybrid_stack_two_chunks_then_decode(fused):
    n_tok, chunk, steps, H = 8192, 4096, 16, 4
    tr = TrunkAttention(n_kda=2, n_mla=1, heads=H, batch=1, max_ctx=n_tok + 64, max_chunk=chunk, seed=5, fused=fused,
                        keep_outputs=True)
    tr.prefill(n_tok, chunk)
    for s in range(steps):
        tr.run_chunk(n_tok + s, 1)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    calls = [chunk, chunk] + [1] * steps
    # ---------------- KDA layers (both see the same inputs and start from zero: same results) ----------------
    recs, _, o_st, o_cst = _kda_oracle(tr, calls)
    for L in range(2):
        kept = tr.kept[("kda", L)]
        assert len(kept) == len(calls)
        for (rec, y), want32, n in zip(kept, recs, calls):
            got = rec.float().cpu().numpy().reshape(1, n, H, 128)
            assert max_rel(got, want32) < 6e-3, "bf16 round-toward-zero outputs vs the oracle's fp32 outputs"
        assert frob_rel(tr.rec_state[L].cpu().numpy(), o_st) < 1e-2
        assert np.array_equal(bits(tr.conv_state[L]), o_cst)
        # gated norm of the last decode step against the oracle on the GPU's own recurrence output
        rec, y = kept[-1]
        want_y = orc.gated_rms_norm(bits(rec).reshape(H, 128), bits(tr.kda_in["norm_w"]),
                                    tr.kda_in["gate_out"][:H].cpu().numpy(), H, 128, 1e-6, gate_act=1)
        assert np.abs(y.float().cpu().numpy() - synth.f16_bits_to_f32(want_y)).max() < 2e-3
    # ---------------- MLA layer: planes, then sampled rows of every call ----------------
    mi = tr.mla_in
    total = n_tok + steps
    ckv_o = np.zeros((tr.cap, 512), dtype=np.uint16)
    pool_o = np.zeros((tr.cap // 4, 128), dtype=np.uint16)
    ring_o = np.zeros((tr.ring_rows, 256), dtype=np.uint16)
    kv_pre, ln_w = mi["kv_pre"].cpu().numpy(), bits(mi["ln_w"])
    idx_k, idx_g = bits(mi["idx_k"]), bits(mi["idx_g"])
    kn_w, kn_b, ape = bits(mi["knorm_w"]), bits(mi["knorm_b"]), mi["ape"].cpu().numpy()
    pos = 0
    for n in calls:
        orc.mla_cache_append(np.ascontiguousarray(kv_pre[:n]), ln_w, ckv_o, pos, n, 1e-6)
        kn = orc.layernorm_f16(np.ascontiguousarray(idx_k[:n]), kn_w, kn_b, n, 128, 1e-5)
        orc.kpool_write(kn, np.ascontiguousarray(idx_g[:n]), ring_o, tr.ring_rows, pool_o, ape, pos, n)
        pos += n
    got_ckv, got_pool = bits(tr.ckv[0][0]), bits(tr.pool[0][0])
    f16 = synth.f16_bits_to_f32
    assert np.abs(f16(got_ckv[:total]) - f16(ckv_o[:total])).max() < 2e-3, "latent cache rows"
    assert np.abs(f16(got_pool[:total // 4]) - f16(pool_o[:total // 4])).max() < 4e-3, "pooled keys"
    kept = tr.kept[("mla", 0, 0)]
    assert len(kept) == len(calls)
    q_nope, q_idx, w_idx, kv_b = bits(mi["q_nope"]), bits(mi["q_idx"]), bits(mi["w"]), bits(mi["kv_b"])
    for ci, (pos, n, topk, raw, lat, oab) in enumerate(kept):
        rows = [0, 1, n // 2, n - 1] if n > 1 else [0]
        rows = sorted(set(rows))
        qp = np.array([pos + r for r in rows], dtype=np.int32)
        npools = (pos + n) // 4
        # the GPU's scores of these rows (the pooled keys of visible pools never change once written)
        sc = torch.empty(len(rows), npools, dtype=torch.float16, device="cuda")
        sel = torch.tensor(rows, device="cuda")
        hk.indexer_score(mi["q_idx"][sel].contiguous(), tr.pool[0][0], mi["w"][sel].contiguous(), dev(qp), sc, len(rows), npools)
        torch.cuda.synchronize()
        _, o_sc32 = orc.indexer_score(np.ascontiguousarray(q_idx[rows]), got_pool, np.ascontiguousarray(w_idx[rows]), qp,
                                      len(rows), npools)
        s_gpu = f16(bits(sc))
        finite = np.isfinite(o_sc32)
        assert np.array_equal(np.isfinite(s_gpu), finite) and np.abs(s_gpu[finite] - o_sc32[finite]).max() <= 4e-3
        want_topk = orc.dsa_topk(bits(sc), npools, len(rows), npools, min(512, npools), 512)
        got_topk = topk.cpu().numpy()[rows]
        assert np.array_equal(got_topk, want_topk), "pool selection, bit-exact on the GPU's fp16 scores (call %d)" % ci
        want_raw = orc.pool_expand(got_topk, qp, len(rows))
        got_raw = raw.cpu().numpy()[rows]
        assert np.array_equal(got_raw, want_raw)
        o_ql = orc.q_latent(np.ascontiguousarray(q_nope[rows]), kv_b, len(rows))
        _, o_lat32 = orc.mla_attend(o_ql, got_ckv, len(rows), 64, 0.0625, raw_idx=np.ascontiguousarray(got_raw), kidx=KIDX)
        g_lat = lat.float().cpu().numpy()[rows]
        assert max_rel(g_lat, o_lat32) < 2e-3, "sparse attention rows of call %d" % ci
        want_o = f16(orc.o_absorb(np.ascontiguousarray(bits(lat)[rows]), kv_b, len(rows)))
        assert max_rel(oab.float().cpu().numpy()[rows], want_o) < 2e-3


def test_decode_step_of_two_sequences_on_their_own_streams_equals_sequence_by_sequence():
    """batch 2: the MLA layers of a decode step run on one stream per sequence with single-row work buffers of their
    own (fused driver); the same stack run sequence by sequence on one stream (unfused driver: the reference's call
    sequence) must leave the same selections, attention rows, caches and states"""
    n_tok, chunk, steps, H = 1024, 512, 5, 4
    runs = []
    for fused in (True, False):
        tr = TrunkAttention(n_kda=2, n_mla=2, heads=H, batch=2, max_ctx=n_tok + 64, max_chunk=chunk, seed=9, fused=fused,
                            keep_outputs=True)
        tr.prefill(n_tok, chunk)
        for s in range(steps):
            tr.run_chunk(n_tok + s, 1)
        torch.cuda.synchronize()
        assert hk.read_device_status() == 0
        runs.append(tr)
    a, b = runs
    for seq in range(2):
        for L in range(2):
            assert torch.equal(a.ckv[seq][L], b.ckv[seq][L]) and torch.equal(a.pool[seq][L], b.pool[seq][L])
            ka, kb = a.kept[("mla", L, seq)], b.kept[("mla", L, seq)]
            assert len(ka) == len(kb) == 2 + steps
            for (pa, na, ta, ra, la, oa), (pb, nb, tb, rb, lb, ob) in zip(ka[-steps:], kb[-steps:]):
                assert (pa, na) == (pb, nb) and torch.equal(ta, tb) and torch.equal(ra, rb), "selection of a decoded token"
                assert max_rel(la.float().cpu().numpy(), lb.float().cpu().numpy()) < 2e-3
                assert max_rel(oa.float().cpu().numpy(), ob.float().cpu().numpy()) < 2e-3
    for L in range(2):
        assert frob_rel(a.rec_state[L].cpu().numpy(), b.rec_state[L].cpu().numpy()) < 1e-2
        assert torch.equal(a.conv_state[L], b.conv_state[L])
