"""GPU parity of the kernels either side of the KDA recurrence, through the C ABI: transpose + cast, gate
preparation, gated RMS norm, the fused cast + convolution and the chunked prefill that forms its own gates.
Checked against the CPU oracle and, when it was built, against the reference's own kernels compiled for
sm_100a (same arithmetic order and compiler flags: bit-exact)."""
import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bf16_ulp_diff, bits, dev, dev_bf16, dev_f16, max_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,F", [(64, 128), (37, 200), (1, 24576), (513, 96), (2048, 1536), (3, 7)])
def test_transpose_cast(S, F):
    x = synth.rng(S + F).standard_normal((S, F), dtype=np.float32)
    dx = dev(x)
    out = torch.zeros(F, S, dtype=torch.bfloat16, device="cuda")
    hk.kda_transpose_cast(out, dx, S, F)
    torch.cuda.synchronize()
    o_mixed, _, _ = orc.kda_prepare(x, None, None, None, None, 0.0, S, F, 1, 4)
    assert np.array_equal(bits(out), o_mixed)
    if ref.available():
        r = torch.zeros(F, S, dtype=torch.bfloat16, device="cuda")
        ref.kda_transpose_cast(r, dx, S, F)
        torch.cuda.synchronize()
        assert np.array_equal(bits(out), bits(r))


def _gate_outputs(fn, k, S, H, D):
    beta = torch.zeros(S, H, dtype=torch.bfloat16, device="cuda")
    g = torch.zeros(S, H, D, dtype=torch.float32, device="cuda")
    fn(dev(k["b"]), dev(k["f"]), dev(k["dt_bias"]), dev(k["a_log"]), k["lower_bound"], beta, g, S, H, D)
    torch.cuda.synchronize()
    return bits(beta), g.cpu().numpy()


@pytest.mark.parametrize("S,H,D", [(10, 3, 128), (257, 32, 128), (1, 64, 128), (33, 5, 6)])
def test_gate(S, H, D):
    k = synth.kda_raw_gates(S, H, D, seed=S)
    beta, g = _gate_outputs(hk.kda_gate, k, S, H, D)
    _, o_beta, o_g = orc.kda_prepare(None, k["b"], k["f"], k["dt_bias"], k["a_log"], k["lower_bound"], S, 1, H, D)
    assert bf16_ulp_diff(beta, o_beta).max() <= 1
    # the device exponential is the fast one (2 ulp) feeding a reciprocal: 1e-5 of the gate's range
    assert np.max(np.abs(g - o_g)) < 1e-5 * abs(k["lower_bound"])
    if ref.available():
        r_beta, r_g = _gate_outputs(ref.kda_gate, k, S, H, D)
        assert np.array_equal(beta, r_beta)
        assert np.array_equal(g, r_g), "same expression, same flags: bit-exact"


def test_prepare_is_both():
    S, F, H, D = 70, 3 * 2 * 128, 2, 128
    k = synth.kda_raw_gates(S, H, D, seed=9)
    x = synth.rng(10).standard_normal((S, F), dtype=np.float32)
    mixed = torch.zeros(F, S, dtype=torch.bfloat16, device="cuda")
    beta = torch.zeros(S, H, dtype=torch.bfloat16, device="cuda")
    g = torch.zeros(S, H, D, dtype=torch.float32, device="cuda")
    hk.kda_prepare(dev(x), dev(k["b"]), dev(k["f"]), dev(k["dt_bias"]), dev(k["a_log"]), k["lower_bound"], mixed, beta, g,
                   S, F, H, D)
    torch.cuda.synchronize()
    o_mixed, _, _ = orc.kda_prepare(x, None, None, None, None, 0.0, S, F, 1, 4)
    assert np.array_equal(bits(mixed), o_mixed)
    b2, g2 = _gate_outputs(hk.kda_gate, k, S, H, D)
    assert np.array_equal(bits(beta), b2) and np.array_equal(g.cpu().numpy(), g2)
    if ref.available():
        rm = torch.zeros(F, S, dtype=torch.bfloat16, device="cuda")
        rb = torch.zeros(S, H, dtype=torch.bfloat16, device="cuda")
        rg = torch.zeros(S, H, D, dtype=torch.float32, device="cuda")
        ref.kda_prepare(dev(x), dev(k["b"]), dev(k["f"]), dev(k["dt_bias"]), dev(k["a_log"]), k["lower_bound"], rm, rb, rg,
                        S, F, H, D)
        torch.cuda.synchronize()
        assert np.array_equal(bits(mixed), bits(rm)) and np.array_equal(bits(beta), bits(rb))
        assert np.array_equal(g.cpu().numpy(), rg.cpu().numpy())


def _f16_ulp(a_bits, b_bits):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + (x & 0x7FFF))
    return np.abs(key(a_bits) - key(b_bits))


@pytest.mark.parametrize("rows,dim,w_dt,y_dt,g_dt,w_groups,gate_first,gate_act", [
    (640, 128, "bf16", "f16", "f32", 1, False, 1),        # the KDA output gate (n*64 rows of one head)
    (1, 128, "bf16", "f16", "f32", 1, False, 1),
    (37, 128, "f32", "f32", "bf16", 1, False, 0),
    (50, 256, "f32", "f16", "bf16", 1, True, 0),
    (33, 64, "bf16", "f32", "f32", 4, False, 0),
    (9, 2048, "f32", "f16", "f32", 1, False, 1),          # one CTA per row
    (6, 4096 + 512, "bf16", "f32", "bf16", 3, True, 0),
])
def test_gated_rms_norm(rows, dim, w_dt, y_dt, g_dt, w_groups, gate_first, gate_act):
    r = synth.rng(rows + dim)
    x = synth.f32_to_bf16_bits(r.standard_normal((rows, dim), dtype=np.float32))
    w = (1 + 0.1 * r.standard_normal((w_groups, dim), dtype=np.float32)).astype(np.float32)
    g = (2 * r.standard_normal((rows, dim), dtype=np.float32)).astype(np.float32)
    w_np = synth.f32_to_bf16_bits(w) if w_dt == "bf16" else w
    g_np = synth.f32_to_bf16_bits(g) if g_dt == "bf16" else g
    dw = dev_bf16(w_np) if w_dt == "bf16" else dev(w_np)
    dg = dev_bf16(g_np) if g_dt == "bf16" else dev(g_np)
    dx = dev_bf16(x)
    ydtype = torch.float16 if y_dt == "f16" else torch.float32
    y = torch.zeros(rows, dim, dtype=ydtype, device="cuda")
    eps, cb = 1e-6, 0.25 if w_groups > 1 else 0.0
    hk.gated_rms_norm(dx, dw, y, dg, rows, dim, eps, cb, w_groups, gate_first, gate_act)
    torch.cuda.synchronize()
    o = orc.gated_rms_norm(x, w_np, g_np, rows, dim, eps, y_f32=(y_dt == "f32"), constant_bias=cb, w_groups=w_groups,
                           gate_first=gate_first, gate_act=gate_act)
    if y_dt == "f16":
        assert _f16_ulp(bits(y), o).max() <= 1
    else:
        assert max_rel(y.cpu().numpy(), o) < 1e-5
    if ref.available():
        yr = torch.zeros(rows, dim, dtype=ydtype, device="cuda")
        ref.gated_rms_norm(dx, dw, yr, dg, rows, dim, eps, cb, w_groups, gate_first, gate_act)
        torch.cuda.synchronize()
        assert torch.equal(y, yr), "same summation order as the reference kernel: bit-exact"


@pytest.mark.parametrize("dim,T,bsz", [(1536, 512, 1), (1536, 1, 1), (1536, 3, 2), (200, 37, 1), (12288, 130, 1), (64, 4099, 1)])
def test_cast_conv_equals_transpose_cast_then_conv(dim, T, bsz):
    r = synth.rng(dim + T)
    x = r.standard_normal((bsz, T, dim), dtype=np.float32)
    inp = synth.conv_inputs(T, dim, bsz=bsz, seed=dim + T)
    dx, dw = dev(x), dev_bf16(inp["weight"])
    # two-step path: per sequence transpose + cast, then the channel-major convolution
    mixed = torch.empty(bsz, dim, T, dtype=torch.bfloat16, device="cuda")
    for b in range(bsz):
        hk.kda_transpose_cast(mixed[b], dx[b], T, dim)
    st_a = dev_bf16(inp["state"])
    out_a = torch.empty(bsz, T, dim, dtype=torch.bfloat16, device="cuda")
    hk.cuda_causal_conv1d_update(mixed, st_a, None, dw, None, out_a, bsz, dim, T, 4, 4, True, False)
    st_b = dev_bf16(inp["state"])
    out_b = torch.zeros(bsz, T, dim, dtype=torch.bfloat16, device="cuda")
    hk.kda_cast_conv(dx, st_b, None, dw, None, out_b, bsz, dim, T, True)
    torch.cuda.synchronize()
    assert np.array_equal(bits(st_a), bits(st_b)), "window state"
    assert np.array_equal(bits(out_a), bits(out_b)), "fused cast + conv must equal the two-step path"
    # and the oracle on the rounded input
    o_out, o_st = orc.conv1d_update(bits(mixed), inp["state"], inp["weight"], None, bsz, dim, T, 4, 4)
    assert np.array_equal(bits(st_b), o_st)
    assert bf16_ulp_diff(bits(out_b), o_out).max() <= 1


@pytest.mark.parametrize("T,H", [(64, 2), (200, 3), (4096, 32)])
def test_chunked_prefill_gated_equals_gate_then_prefill(T, H):
    D = 128
    inp = synth.kda_inputs(T, H, D, seed=T + 1)
    k = synth.kda_raw_gates(T, H, D, seed=T)
    qkv = dev_bf16(inp["mixed_qkv"])
    f, b, dtb, al = dev(k["f"]), dev(k["b"]), dev(k["dt_bias"]), dev(k["a_log"])
    s0 = (0.1 * synth.rng(3).standard_normal((1, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    # two-step path
    beta = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    g = torch.empty(T, H, D, dtype=torch.float32, device="cuda")
    hk.kda_gate(b, f, dtb, al, k["lower_bound"], beta, g, T, H, D)
    st_a = dev(s0)
    out_a = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    path = hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, st_a, out_a, 1, T, H, H, D, D, 1, None, True, False)
    assert path == "chunked"
    # fused
    st_b = dev(s0)
    out_b = torch.zeros(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    hk.kda_chunked_prefill_gated(qkv, f, b, dtb, al, k["lower_bound"], st_b, out_b, 1, T, H)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    assert torch.equal(out_a, out_b), "gates formed inside the kernel must give the same output bits"
    assert torch.equal(st_a, st_b)
    if T <= 256:
        # against the oracle: gate restatement, then the token-by-token recurrence
        _, o_beta, o_g = orc.kda_prepare(None, k["b"], k["f"], k["dt_bias"], k["a_log"], k["lower_bound"], T, 1, H, D)
        _, o32, o_st = orc.kda_recurrent(inp["mixed_qkv"], o_g.reshape(1, T, H, D), o_beta.reshape(1, T, H), s0, 1, T, H, H, D, D)
        got = torch.empty(1, T, H, D, dtype=torch.float32, device="cuda")
        st_c = dev(s0)
        hk.kda_chunked_prefill_gated(qkv, f, b, dtb, al, k["lower_bound"], st_c, out_b, 1, T, H, out_f32=got)
        torch.cuda.synchronize()
        assert max_rel(got.cpu().numpy(), o32) < 2e-3          # the path's stated tolerance
        assert max_rel(st_c.cpu().numpy(), o_st) < 2e-3


@pytest.mark.parametrize("n,pos", [(1, 0), (1, 777), (37, 100), (4096, 32768)])
def test_mla_cache_append(n, pos):
    r = synth.rng(n + pos)
    kv = (3 * r.standard_normal((n, 512), dtype=np.float32)).astype(np.float32)
    lw = synth.f32_to_f16_bits((1 + 0.1 * r.standard_normal(512, dtype=np.float32)).astype(np.float32))
    rows = pos + n + 3
    cache0 = synth.f32_to_f16_bits(r.standard_normal((rows, 512), dtype=np.float32))
    ck, stage = dev_f16(cache0), torch.zeros(n, 512, dtype=torch.float16, device="cuda")
    hk.mla_cache_append(dev(kv), dev_f16(lw), ck, pos, n, 1e-6, ckv_new=stage)
    torch.cuda.synchronize()
    got = bits(ck)
    want = orc.mla_cache_append(kv, lw, cache0.copy(), pos, n, 1e-6)
    assert np.array_equal(got[:pos], cache0[:pos]) and np.array_equal(got[pos + n:], cache0[pos + n:]), "other rows untouched"
    assert _f16_ulp(got[pos:pos + n], want[pos:pos + n]).max() <= 1
    assert np.array_equal(bits(stage), got[pos:pos + n])
    if ref.available():
        y = torch.zeros(n, 512, dtype=torch.float16, device="cuda")
        ref.rms_norm(dev(kv), dev_f16(lw), y, n, 512, 1e-6)
        torch.cuda.synchronize()
        assert np.array_equal(bits(y), got[pos:pos + n]), "same summation order as the reference kernel: bit-exact"


@pytest.mark.parametrize("rows,dim", [(1, 128), (300, 128), (17, 96), (5, 1000)])
def test_layernorm_f16(rows, dim):
    r = synth.rng(rows + dim)
    x = synth.f32_to_f16_bits((2 * r.standard_normal((rows, dim), dtype=np.float32) + 0.5).astype(np.float32))
    w = synth.f32_to_f16_bits((1 + 0.1 * r.standard_normal(dim, dtype=np.float32)).astype(np.float32))
    b = synth.f32_to_f16_bits((0.1 * r.standard_normal(dim, dtype=np.float32)).astype(np.float32))
    dx, dw, db = dev_f16(x), dev_f16(w), dev_f16(b)
    y = torch.zeros(rows, dim, dtype=torch.float16, device="cuda")
    hk.layernorm_f16(dx, dw, db, y, rows, dim, 1e-5)
    torch.cuda.synchronize()
    want = orc.layernorm_f16(x, w, b, rows, dim, 1e-5)
    assert max_rel(synth.f16_bits_to_f32(bits(y)), synth.f16_bits_to_f32(want)) < 2e-3
    assert (_f16_ulp(bits(y), want) > 1).mean() < 1e-3
    if ref.available():
        yr = torch.zeros(rows, dim, dtype=torch.float16, device="cuda")
        ref.layernorm_f16(dx, dw, db, yr, rows, dim, 1e-5)
        torch.cuda.synchronize()
        assert torch.equal(y, yr)
    # in place, as the engine calls it (src/engine/runner.cpp:577)
    hk.layernorm_f16(dx, dw, db, dx, rows, dim, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(dx, y)


def test_mla_decode_prologue_equals_append_layernorm_kpool_in_turn():
    """hk_mla_decode_prologue (one launch per decoded token) against hk_mla_cache_append -> hk_layernorm_f16 ->
    hk_kpool_write on separate copies of the caches, 11 consecutive positions (three pools complete on the way):
    cache rows, normalised keys, ring rows, pooled keys and the position word are the same bits"""
    r = synth.rng(404)
    pos0, steps, ring_rows = 1021, 11, 64
    cap = pos0 + steps + 2
    lw = dev_f16(synth.f32_to_f16_bits((1 + 0.1 * r.standard_normal(512, dtype=np.float32)).astype(np.float32)))
    kw = dev_f16(synth.f32_to_f16_bits((1 + 0.1 * r.standard_normal(128, dtype=np.float32)).astype(np.float32)))
    kb = dev_f16(synth.f32_to_f16_bits((0.1 * r.standard_normal(128, dtype=np.float32)).astype(np.float32)))
    ape = dev((0.1 * r.standard_normal((4, 128), dtype=np.float32)).astype(np.float32))
    cache0 = synth.f32_to_f16_bits(r.standard_normal((cap, 512), dtype=np.float32))
    ring0 = synth.f32_to_f16_bits(r.standard_normal((ring_rows, 256), dtype=np.float32))
    pool0 = synth.f32_to_f16_bits(r.standard_normal((cap // 4 + 1, 128), dtype=np.float32))
    ck_a, ck_b = dev_f16(cache0), dev_f16(cache0)
    rg_a, rg_b = dev_f16(ring0), dev_f16(ring0)
    pl_a, pl_b = dev_f16(pool0), dev_f16(pool0)
    kn_a = torch.zeros(1, 128, dtype=torch.float16, device="cuda")
    kn_b = torch.zeros(1, 128, dtype=torch.float16, device="cuda")
    qp = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    for s in range(steps):
        pos = pos0 + s
        kv = dev((3 * r.standard_normal((1, 512), dtype=np.float32)).astype(np.float32))
        ik = dev_f16(synth.f32_to_f16_bits((2 * r.standard_normal((1, 128), dtype=np.float32) + 0.3).astype(np.float32)))
        ig = dev_f16(synth.f32_to_f16_bits(r.standard_normal((1, 128), dtype=np.float32)))
        hk.mla_cache_append(kv, lw, ck_a, pos, 1, 1e-6)
        hk.layernorm_f16(ik, kw, kb, kn_a, 1, 128, 1e-5)
        hk.kpool_write(kn_a, ig, rg_a, ring_rows, pl_a, ape, pos, 1)
        hk.mla_decode_prologue(kv, lw, ck_b, 1e-6, ik, kw, kb, kn_b, 1e-5, ig, rg_b, ring_rows, pl_b, ape, pos, q_pos_out=qp)
        torch.cuda.synchronize()
        assert torch.equal(kn_a, kn_b) and int(qp.item()) == pos, s
    assert torch.equal(ck_a, ck_b) and torch.equal(rg_a, rg_b) and torch.equal(pl_a, pl_b)
    assert not np.array_equal(bits(pl_b), pool0), "pools were completed on the way"
