"""GPU parity of the KDA kernels (short conv, recurrence) through the C ABI, against the CPU oracle
and, when it was built, against the reference's own kernels compiled for sm_100a."""
import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bf16_ulp_diff, bits, dev, dev_bf16, frob_rel, max_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu


def _run_conv(x, st, w, bsz, dim, T, K=4, act=True, history=False, state_size=None, use_ref=False):
    state_size = state_size or K
    dx, dst, dw = dev_bf16(x), dev_bf16(st), dev_bf16(w)
    out = torch.empty(bsz, T, dim, dtype=torch.bfloat16, device="cuda")
    fn = ref.conv1d_update if use_ref else hk.cuda_causal_conv1d_update
    fn(dx, dst, None, dw, None, out, bsz, dim, T, state_size, K, act, history)
    torch.cuda.synchronize()
    return bits(out), bits(dst)


@pytest.mark.parametrize("dim,T", [(1536, 512), (1536, 1), (1536, 3), (1536, 37), (256, 200), (192, 4099), (12288, 128)])
def test_conv_vs_oracle_and_reference(dim, T):
    inp = synth.conv_inputs(T, dim, seed=dim + T)
    o_out, o_st = orc.conv1d_update(inp["x"], inp["state"], inp["weight"], None, 1, dim, T, 4, 4)
    g_out, g_st = _run_conv(inp["x"], inp["state"], inp["weight"], 1, dim, T)
    assert np.array_equal(g_st, o_st), "window state must match exactly"
    ulp = bf16_ulp_diff(g_out, o_out)
    assert ulp.max() <= 1 and (ulp > 0).mean() < 2e-3  # exp approximation may flip a rounding
    if ref.available():
        r_out, r_st = _run_conv(inp["x"], inp["state"], inp["weight"], 1, dim, T, use_ref=True)
        assert np.array_equal(g_st, r_st)
        assert np.array_equal(g_out, r_out), "same arithmetic as the reference kernel: bit-exact"


def test_conv_history_and_generic_k():
    dim, T, K, S = 96, 9, 3, 7
    inp = synth.conv_inputs(T, dim, K=K, seed=5)
    st = synth.f32_to_bf16_bits(synth.rng(9).standard_normal((1, dim, S), dtype=np.float32))
    for history in (False, True):
        o_out, o_st = orc.conv1d_update(inp["x"], st, inp["weight"], None, 1, dim, T, S, K, True, history)
        g_out, g_st = _run_conv(inp["x"], st, inp["weight"], 1, dim, T, K=K, history=history, state_size=S)
        assert np.array_equal(g_st, o_st)
        assert bf16_ulp_diff(g_out, o_out).max() <= 1


def _run_rec(inp, state, bsz, T, H, D, stride=1, cw=True, hist=False, use_ref=False, force_recurrent=True):
    q, g, b = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"])
    st = dev(state)
    out = torch.empty(bsz, T, H, D, dtype=torch.bfloat16, device="cuda")
    o32 = torch.empty(bsz, T, H, D, dtype=torch.float32, device="cuda")
    if use_ref:
        ref.kda_recurrent(q, g, b, st, out, bsz, T, H, H, D, D, stride, None, cw, hist)
        o32 = None
    else:
        hk.cuda_recurrent_gated_delta_rule(q, g, b, st, out, bsz, T, H, H, D, D, stride, None, cw, hist,
                                           out_f32=o32, force_recurrent=force_recurrent)
    torch.cuda.synchronize()
    return bits(out), (None if o32 is None else o32.cpu().numpy()), st.cpu().numpy()


@pytest.mark.parametrize("T,H", [(1, 32), (16, 4), (70, 2), (1, 64)])
def test_recurrent_vs_oracle_and_reference(T, H):
    D = 128
    inp = synth.kda_inputs(T, H, D, seed=T)
    s0 = (0.1 * synth.rng(3).standard_normal((1, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    o_out, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, 1, T, H, H, D, D)
    g_out, g_32, g_st = _run_rec(inp, s0, 1, T, H, D)
    assert max_rel(g_32, o_32) < 2e-3 and max_rel(g_32, o_32) < 1e-4
    assert frob_rel(g_st, o_st) < 1e-5
    assert bf16_ulp_diff(g_out, o_out).max() <= 1
    if ref.available():
        r_out, _, r_st = _run_rec(inp, s0, 1, T, H, D, use_ref=True)
        assert frob_rel(g_st, r_st) < 1e-5
        assert bf16_ulp_diff(g_out, r_out).max() <= 1
        assert frob_rel(o_st, r_st) < 1e-5, "oracle pinned to the reference kernel"


@pytest.mark.parametrize("dim,cw,hist,steps", [(64, False, False, 7), (64, False, True, 7), (128, False, True, 1),
                                               (128, True, True, 7), (128, True, False, 7), (128, False, False, 1)])
def test_recurrent_determinism_suite_shapes(dim, cw, hist, steps):
    """the 12-config grid of the reference's bit-repeatability test (test_deterministic_reductions.cu:19-49):
    same synthetic inputs, here also checked for VALUE against the oracle, then 4 repeats byte-equal."""
    heads, stride = 2, (steps + 1 if hist else 1)
    n = steps * 3 * heads * dim
    i = np.arange(n, dtype=np.float32)
    qkv = synth.f32_to_bf16_bits(np.sin(i * np.float32(0.019))).reshape(1, steps, 3 * heads * dim)
    bi = np.arange(steps * heads, dtype=np.float32)
    beta = synth.f32_to_bf16_bits((0.3 + np.cos(bi) * 0.1).astype(np.float32)).reshape(1, steps, heads)
    ng = steps * heads * (dim if cw else 1)
    g = (-0.01 - (np.arange(ng) % 7) * 0.003).astype(np.float32)
    s0 = (np.sin(np.arange(stride * heads * dim * dim, dtype=np.float32) * np.float32(0.017)) * 0.2).astype(np.float32)
    s0 = s0.reshape(1, stride, heads, dim, dim)
    inp = {"mixed_qkv": qkv, "g": g, "beta": beta}
    o_out, o_32, o_st = orc.kda_recurrent(qkv, g, beta, s0, 1, steps, heads, heads, dim, dim, stride,
                                          None, cw, hist)
    first = None
    for rep in range(4):
        g_out, g_32, g_st = _run_rec(inp, s0, 1, steps, heads, dim, stride, cw, hist)
        if first is None:
            first = (g_out.copy(), g_st.copy())
            assert max_rel(g_32, o_32) < 1e-4
            assert frob_rel(g_st, o_st) < 1e-5
        assert np.array_equal(g_out, first[0]) and np.array_equal(g_st.view(np.uint32), first[1].view(np.uint32))
    if ref.available():
        r_out, _, r_st = _run_rec(inp, s0, 1, steps, heads, dim, stride, cw, hist, use_ref=True)
        assert frob_rel(g_st, r_st) < 1e-5
        assert bf16_ulp_diff(g_out, r_out).max() <= 1


def test_recurrent_slots_and_batch():
    T, H, D, bsz = 3, 4, 128, 3
    inp = synth.kda_inputs(T, H, D, bsz=bsz, seed=11)
    slots = np.array([2, 0, 3], dtype=np.int32)
    s0 = (0.1 * synth.rng(4).standard_normal((4, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    o_out, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, bsz, T, H, H, D, D, 1, slots)
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    out = torch.empty(bsz, T, H, D, dtype=torch.bfloat16, device="cuda")
    hk.cuda_recurrent_gated_delta_rule(q, g, b, st, out, bsz, T, H, H, D, D, 1, dev(slots), True, False)
    torch.cuda.synchronize()
    assert frob_rel(st.cpu().numpy(), o_st) < 1e-5
    assert np.array_equal(st.cpu().numpy()[1], s0[1]), "unused slot untouched"
    assert bf16_ulp_diff(bits(out), o_out).max() <= 1


def test_bad_arguments_are_rejected_before_launch():
    t = torch.zeros(16, device="cuda")
    with pytest.raises(hk.HeliosB200Error) as e:
        hk.cuda_recurrent_gated_delta_rule(t, t, t, t, t, 1, 1, 3, 4, 128, 128, 1, None, True, False)
    assert e.value.status == hk.HK_ERR_INVALID
    with pytest.raises(hk.HeliosB200Error) as e:
        hk.cuda_recurrent_gated_delta_rule(t, t, t, t, t, 1, 1, 4, 4, 96, 96, 1, None, False, False)
    assert e.value.status == hk.HK_ERR_UNSUPPORTED
    with pytest.raises(hk.HeliosB200Error):
        hk.cuda_causal_conv1d_update(t, t, None, t, None, t, 1, 64, 8, 2, 4, True, False)


# ------------------------------------------------------------------------------------------------
# chunked tensor-core prefill == the recurrence called with seqlen = T
# ------------------------------------------------------------------------------------------------
def _gate_like_reference(T, H, D, seed):
    """log-decay in the reference engine's range: lb * sigmoid(x), lb = -5 (src/engine/glue2.cu:347-360)"""
    x = synth.rng(seed).standard_normal((1, T, H, D), dtype=np.float32)
    return (-5.0 / (1.0 + np.exp(-x))).astype(np.float32)


@pytest.mark.parametrize("T,H,gate", [(64, 2, "config"), (65, 2, "config"), (127, 1, "config"), (128, 4, "config"),
                                      (200, 2, "config"), (512, 32, "config"), (256, 2, "reference"), (192, 2, "weak")])
def test_chunked_prefill_vs_oracle(T, H, gate):
    D = 128
    inp = synth.kda_inputs(T, H, D, seed=100 + T)
    if gate == "reference":
        inp["g"] = _gate_like_reference(T, H, D, 7)
    elif gate == "weak":
        inp["g"] = (inp["g"] * 0.02).astype(np.float32)      # long memory: state grows over many chunks
    s0 = (0.1 * synth.rng(3).standard_normal((1, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    o_out, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, 1, T, H, H, D, D)
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    o32 = torch.empty(1, T, H, D, dtype=torch.float32, device="cuda")
    path = hk.cuda_recurrent_gated_delta_rule(q, g, b, st, out, 1, T, H, H, D, D, 1, None, True, False, out_f32=o32)
    torch.cuda.synchronize()
    assert path == "chunked"
    assert hk.read_device_status() == 0
    e_out, e_st = max_rel(o32.cpu().numpy(), o_32), frob_rel(st.cpu().numpy(), o_st)
    print("chunked T=%d H=%d gate=%s: out max_rel %.2e, state frob %.2e" % (T, H, gate, e_out, e_st))
    assert e_out < 2e-3, "outputs within 2e-3 (max |a-b| / max |b|) of the recurrence"
    assert e_st < 1e-2, "state within 1e-2 relative Frobenius"
    # the rounded output is the round-toward-zero bf16 of the fp32 output
    want_bits = (o32.cpu().numpy().view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal(bits(out), want_bits)


def test_chunked_prefill_then_decode_continues_the_state():
    T, H, D, extra = 256, 4, 128, 16
    inp = synth.kda_inputs(T + extra, H, D, seed=9)
    s0 = np.zeros((1, 1, H, D, D), dtype=np.float32)
    _, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, 1, T + extra, H, H, D, D)
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    out = torch.empty(1, T + extra, H, D, dtype=torch.bfloat16, device="cuda")
    o32 = torch.empty(1, T + extra, H, D, dtype=torch.float32, device="cuda")
    hk.cuda_recurrent_gated_delta_rule(q[:, :T], g[:, :T], b[:, :T], st, out[:, :T], 1, T, H, H, D, D, 1, None, True,
                                       False, out_f32=o32[:, :T])
    for s in range(T, T + extra):
        hk.cuda_recurrent_gated_delta_rule(q[:, s:s + 1], g[:, s:s + 1], b[:, s:s + 1], st, out[:, s:s + 1], 1, 1, H, H,
                                           D, D, 1, None, True, False, out_f32=o32[:, s:s + 1])
    torch.cuda.synchronize()
    assert max_rel(o32.cpu().numpy(), o_32) < 2e-3
    assert frob_rel(st.cpu().numpy(), o_st) < 1e-2


def test_chunked_matches_recurrent_kernel_and_reference_kernel():
    T, H, D = 320, 3, 128
    inp = synth.kda_inputs(T, H, D, seed=12)
    s0 = (0.05 * synth.rng(5).standard_normal((1, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    _, c32, c_st = _run_rec(inp, s0, 1, T, H, D, force_recurrent=False)
    _, r32, r_st = _run_rec(inp, s0, 1, T, H, D, force_recurrent=True)
    assert max_rel(c32, r32) < 2e-3 and frob_rel(c_st, r_st) < 1e-2
    if ref.available():
        _, _, ref_st = _run_rec(inp, s0, 1, T, H, D, use_ref=True)
        assert frob_rel(c_st, ref_st) < 1e-2, "state vs the reference's own kernel run with seqlen = T"


def test_chunked_batch_and_slots():
    T, H, D, bsz = 130, 2, 128, 2
    inp = synth.kda_inputs(T, H, D, bsz=bsz, seed=14)
    slots = np.array([1, 0], dtype=np.int32)
    s0 = (0.1 * synth.rng(6).standard_normal((2, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    _, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, bsz, T, H, H, D, D, 1, slots)
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    out = torch.empty(bsz, T, H, D, dtype=torch.bfloat16, device="cuda")
    o32 = torch.empty(bsz, T, H, D, dtype=torch.float32, device="cuda")
    assert hk.cuda_recurrent_gated_delta_rule(q, g, b, st, out, bsz, T, H, H, D, D, 1, dev(slots), True, False,
                                              out_f32=o32) == "chunked"
    torch.cuda.synchronize()
    assert max_rel(o32.cpu().numpy(), o_32) < 2e-3 and frob_rel(st.cpu().numpy(), o_st) < 1e-2


@pytest.mark.parametrize("T,H,bsz", [(2100, 3, 1), (1500, 2, 2), (4096, 32, 1), (1200, 64, 1), (1100, 32, 3), (1100, 17, 3)])
def test_chunked_fused_launch_equals_two_kernel_form(T, H, bsz):
    """the persistent fused launch (chains + preparation workers through the L2 ring; T spans more chunks than the
    ring has slots, so slots are reused) against the two-kernel form on the same inputs: same bits; the short
    cases also against the oracle.  The last three cases have more than 48 chains: 32, 48 and 17 chain CTAs walk two,
    two and three chains each, one after the other."""
    D = 128
    inp = synth.kda_inputs(T, H, D, bsz=bsz, seed=200 + T)
    s0 = (0.1 * synth.rng(8).standard_normal((bsz, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    q, g, b = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"])
    res = []
    try:
        for form in (1, 0):
            hk.kda_chunked_set_form(form)
            st = dev(s0)
            out = torch.empty(bsz, T, H, D, dtype=torch.bfloat16, device="cuda")
            o32 = torch.empty(bsz, T, H, D, dtype=torch.float32, device="cuda")
            ws_bytes = hk.kda_chunked_workspace_bytes(bsz, T, H)
            assert hk.cuda_recurrent_gated_delta_rule(q, g, b, st, out, bsz, T, H, H, D, D, 1, None, True, False,
                                                      out_f32=o32) == "chunked"
            # a second call on the same workspace-sized buffer: the ring flags are reset by every call
            st2 = dev(s0)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
            for _ in range(2):
                st2.copy_(dev(s0))
                hk.cuda_recurrent_gated_delta_rule(q, g, b, st2, out, bsz, T, H, H, D, D, 1, None, True, False,
                                                   out_f32=o32, workspace=ws)
            torch.cuda.synchronize()
            assert hk.read_device_status() == 0
            assert np.array_equal(st.cpu().numpy(), st2.cpu().numpy())
            res.append((ws_bytes, o32.cpu().numpy(), st.cpu().numpy(), bits(out)))
    finally:
        hk.kda_chunked_set_form(0)
    assert res[1][0] < res[0][0], "the fused form needs the ring only"
    assert np.array_equal(res[0][1], res[1][1]) and np.array_equal(res[0][2], res[1][2])
    assert np.array_equal(res[0][3], res[1][3])
    if T * H * bsz <= 8192:
        _, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, bsz, T, H, H, D, D)
        assert max_rel(res[1][1], o_32) < 2e-3 and frob_rel(res[1][2], o_st) < 1e-2


@pytest.mark.parametrize("H,bsz", [(32, 1), (4, 2), (64, 3)])
def test_decode_step_with_conv_inside_equals_the_two_launch_sequence(H, bsz):
    """hk_kda_decode_step (conv + recurrence of one decoded token in one launch, value slices of a head as a cluster)
    against cuda_causal_conv1d_update followed by cuda_recurrent_gated_delta_rule on the same buffers, 6 tokens in a
    row with carried window and state: same bits everywhere; the first token also against the oracle"""
    D, steps = 128, 6
    dim = 3 * H * D
    r = synth.rng(77 + H)
    x = synth.f32_to_bf16_bits(r.standard_normal((steps, bsz, dim), dtype=np.float32))
    w = synth.f32_to_bf16_bits((0.1 * r.standard_normal((dim, 4), dtype=np.float32)).astype(np.float32))
    bias = synth.f32_to_bf16_bits((0.05 * r.standard_normal((dim,), dtype=np.float32)).astype(np.float32))
    cst0 = synth.f32_to_bf16_bits(r.standard_normal((bsz, dim, 4), dtype=np.float32))
    gates = synth.kda_gates(steps, H, D, bsz=bsz, seed=3)
    g_all, beta_all = dev(np.ascontiguousarray(gates["g"].transpose(1, 0, 2, 3))), dev_bf16(np.ascontiguousarray(gates["beta"].transpose(1, 0, 2)))
    s0 = (0.1 * r.standard_normal((bsz, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    xd, wd, bd = dev_bf16(x), dev_bf16(w), dev_bf16(bias)
    # two-launch sequence
    cs_a, st_a = dev_bf16(cst0), dev(s0)
    qkv_a = torch.empty(steps, bsz, 1, dim, dtype=torch.bfloat16, device="cuda")
    out_a = torch.empty(steps, bsz, 1, H, D, dtype=torch.bfloat16, device="cuda")
    # fused
    cs_b, st_b = dev_bf16(cst0), dev(s0)
    qkv_b = torch.empty(steps, bsz, dim, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty(steps, bsz, H, D, dtype=torch.bfloat16, device="cuda")
    o32_b = torch.empty(steps, bsz, H, D, dtype=torch.float32, device="cuda")
    for s in range(steps):
        hk.cuda_causal_conv1d_update(xd[s].reshape(bsz, dim, 1), cs_a, None, wd, bd, qkv_a[s], bsz, dim, 1, 4, 4, True, False)
        hk.cuda_recurrent_gated_delta_rule(qkv_a[s], g_all[s], beta_all[s], st_a, out_a[s], bsz, 1, H, H, D, D, 1, None, True, False)
        hk.kda_decode_step(xd[s], cs_b, wd, bd, g_all[s], beta_all[s], st_b, out_b[s], bsz, H, out_f32=o32_b[s], conv_out=qkv_b[s])
    torch.cuda.synchronize()
    assert np.array_equal(bits(qkv_a.reshape(steps, bsz, dim)), bits(qkv_b)), "convolved q|k|v"
    assert np.array_equal(bits(cs_a), bits(cs_b)), "rolling window"
    assert np.array_equal(st_a.cpu().numpy(), st_b.cpu().numpy()), "recurrent state"
    assert np.array_equal(bits(out_a.reshape(steps, bsz, H, D)), bits(out_b)), "outputs"
    # first token against the oracle (conv, then recurrence)
    qkv0, _ = orc.conv1d_update(np.ascontiguousarray(x[0]).reshape(bsz, dim, 1), cst0, w, bias, bsz, dim, 1, 4, 4)
    assert np.array_equal(qkv0.reshape(bsz, dim), bits(qkv_b[0])) or \
        bf16_ulp_diff(qkv0.reshape(bsz, dim), bits(qkv_b[0])).max() <= 1
    _, o_32, _ = orc.kda_recurrent(bits(qkv_b[0]).reshape(bsz, 1, dim), np.ascontiguousarray(gates["g"][:, :1]),
                                   np.ascontiguousarray(gates["beta"][:, :1]), s0, bsz, 1, H, H, D, D)
    assert max_rel(o32_b[0].cpu().numpy().reshape(bsz, 1, H, D), o_32) < 2e-3


@pytest.mark.parametrize("H,bsz,w_bf16,g_bf16,y_f16", [(32, 1, True, False, True), (4, 3, False, True, False), (64, 2, True, True, True)])
def test_decode_layer_in_one_launch_equals_the_five_call_sequence(H, bsz, w_bf16, g_bf16, y_f16):
    """hk_kda_decode_layer (cast, gate preparation, conv, recurrence, gated RMS norm of one decoded token in ONE launch)
    against kda_transpose_cast -> kda_gate -> cuda_causal_conv1d_update -> cuda_recurrent_gated_delta_rule ->
    gated_rms_norm on the same buffers, 5 tokens in a row with carried window and state: the same bits everywhere"""
    D, steps = 128, 5
    dim = 3 * H * D
    r = synth.rng(5 + H)
    x32 = dev(r.standard_normal((steps, bsz, dim), dtype=np.float32))
    raw = synth.kda_raw_gates(steps * bsz, H, D, seed=9)
    f = dev(raw["f"]).reshape(steps, bsz, H, D).contiguous()
    b = dev(raw["b"]).reshape(steps, bsz, H).contiguous()
    dtb, alog, lb = dev(raw["dt_bias"]), dev(raw["a_log"]), raw["lower_bound"]
    w = dev_bf16(synth.f32_to_bf16_bits((0.1 * r.standard_normal((dim, 4), dtype=np.float32)).astype(np.float32)))
    cst0 = synth.f32_to_bf16_bits(r.standard_normal((bsz, dim, 4), dtype=np.float32))
    s0 = (0.1 * r.standard_normal((bsz, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    nw = (1.0 + 0.1 * torch.randn(D, device="cuda"))
    nw = nw.to(torch.bfloat16) if w_bf16 else nw
    go = torch.randn(steps, bsz * H, D, device="cuda")
    go = go.to(torch.bfloat16) if g_bf16 else go
    ydt = torch.float16 if y_f16 else torch.float32
    cs_a, st_a, cs_b, st_b = dev_bf16(cst0), dev(s0), dev_bf16(cst0), dev(s0)
    x16 = torch.empty(bsz, dim, 1, dtype=torch.bfloat16, device="cuda")
    g = torch.empty(bsz, H, D, dtype=torch.float32, device="cuda")
    beta = torch.empty(bsz, H, dtype=torch.bfloat16, device="cuda")
    qkv = torch.empty(bsz, 1, dim, dtype=torch.bfloat16, device="cuda")
    out_a = torch.empty(steps, bsz, 1, H, D, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty(steps, bsz, H, D, dtype=torch.bfloat16, device="cuda")
    y_a = torch.empty(steps, bsz * H, D, dtype=ydt, device="cuda")
    y_b = torch.empty(steps, bsz * H, D, dtype=ydt, device="cuda")
    for s in range(steps):
        for q in range(bsz):
            hk.kda_transpose_cast(x16[q], x32[s, q:q + 1], 1, dim)
        hk.kda_gate(b[s], f[s], dtb, alog, lb, beta, g, bsz, H, D)
        hk.cuda_causal_conv1d_update(x16, cs_a, None, w, None, qkv, bsz, dim, 1, 4, 4, True, False)
        hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, st_a, out_a[s], bsz, 1, H, H, D, D, 1, None, True, False)
        hk.gated_rms_norm(out_a[s], nw, y_a[s], go[s], bsz * H, D, 1e-6, gate_act=1)
        hk.kda_decode_layer(x32[s], cs_b, w, None, f[s], b[s], dtb, alog, lb, st_b, out_b[s], nw, go[s], y_b[s], bsz, H,
                            epsilon=1e-6, gate_act=1)
    torch.cuda.synchronize()
    assert np.array_equal(bits(cs_a), bits(cs_b)), "rolling window"
    assert np.array_equal(st_a.cpu().numpy(), st_b.cpu().numpy()), "recurrent state"
    assert np.array_equal(bits(out_a.reshape(steps, bsz, H, D)), bits(out_b)), "recurrence outputs"
    assert torch.equal(y_a, y_b), "normalised outputs"
    assert torch.isfinite(y_b.float()).all()
