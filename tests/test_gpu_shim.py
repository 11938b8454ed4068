"""The C++ boundary on the GPU: the reference-named launchers of libhelios_b200.so (helios::aux::*, helios::glue::*),
called from C++ the way the engine's layer loop calls them, against the same work done through the hk_* C ABI by
ctypes - bit for bit; the reference's own repeatability test linked against this library; and the KDA state snapshot
in the engine's layout ([conv][rec] per layer ordinal, src/engine/runner.cpp:319-335) taken after a prefill by the
REFERENCE's kernels, restored, and continued by this library's decode."""
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bits, dev, dev_bf16, dev_f16, frob_rel, max_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_launchers_equal_the_c_abi_bit_for_bit():
    exe = os.path.join(ROOT, "oracle", "_ref", "shim_harness")
    if not os.path.exists(exe):
        pytest.skip("C++ harness not built (make -C oracle harness)")
    r = synth.rng(41)
    H, D, T = 4, 128, 265
    inp = synth.kda_inputs(T, H, D, seed=41)
    s0 = (0.1 * r.standard_normal((1, 1, H, D, D), dtype=np.float32)).astype(np.float32)
    cv = synth.conv_inputs(37, 1536, seed=41)
    sc = synth.f32_to_f16_bits(r.standard_normal((3, 1000), dtype=np.float32))
    sc[1, 100:140] = sc[1, 7]                                 # ties
    nx = synth.f32_to_bf16_bits(r.standard_normal((64, 128), dtype=np.float32))
    nw = synth.f32_to_bf16_bits(1.0 + 0.1 * r.standard_normal((128,), dtype=np.float32))
    ng = r.standard_normal((64, 128), dtype=np.float32)
    S, F = 33, 3 * H * D
    pq = r.standard_normal((S, F), dtype=np.float32)
    raw = synth.kda_raw_gates(S, H, D, seed=41)
    files = {"rec_qkv": inp["mixed_qkv"], "rec_g": inp["g"], "rec_beta": inp["beta"], "rec_state": s0,
             "conv_x": cv["x"], "conv_state": cv["state"], "conv_w": cv["weight"], "topk_scores": sc,
             "norm_x": nx, "norm_w": nw, "norm_g": ng, "prep_qkv": pq, "prep_b": raw["b"], "prep_f": raw["f"],
             "prep_dt_bias": raw["dt_bias"], "prep_a_log": raw["a_log"]}
    with tempfile.TemporaryDirectory() as d:
        for name, a in files.items():
            np.ascontiguousarray(a).tofile(os.path.join(d, name + ".bin"))
        res = subprocess.run([exe, d], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0 and "SHIM HARNESS DONE" in res.stdout, res.stdout[-1000:] + res.stderr[-2000:]

        def out(name, dtype, shape):
            return np.fromfile(os.path.join(d, "out_" + name + ".bin"), dtype=dtype).reshape(shape)

        got = {"rec_out": out("rec_out", np.uint16, (T, H, D)), "rec_state": out("rec_state", np.float32, (H, D, D)),
               "conv_out": out("conv_out", np.uint16, (37, 1536)), "conv_state": out("conv_state", np.uint16, (1536, 4)),
               "topk_idx": out("topk_idx", np.int32, (3, 512)), "norm_y": out("norm_y", np.uint16, (64, 128)),
               "prep_mixed": out("prep_mixed", np.uint16, (F, S)), "prep_beta": out("prep_beta", np.uint16, (S, H)),
               "prep_g": out("prep_g", np.float32, (S, H, D)), "prep2_mixed": out("prep2_mixed", np.uint16, (F, S)),
               "prep2_beta": out("prep2_beta", np.uint16, (S, H)), "prep2_g": out("prep2_g", np.float32, (S, H, D))}
    # ---- the same calls through the C ABI (Python wrappers): recurrence in three calls with the same dispatch ----
    q, g, b, st = dev_bf16(inp["mixed_qkv"]), dev(inp["g"]), dev_bf16(inp["beta"]), dev(s0)
    o = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    t0, paths = 0, []
    for n in (1, 64, 200):
        paths.append(hk.cuda_recurrent_gated_delta_rule(q[:, t0:t0 + n], g[:, t0:t0 + n], b[:, t0:t0 + n], st, o[:, t0:t0 + n], 1, n,
                                                        H, H, D, D, 1, None, True, False))
        t0 += n
    assert paths == ["recurrent", "chunked", "chunked"]
    torch.cuda.synchronize()
    assert np.array_equal(bits(o).reshape(T, H, D), got["rec_out"]) and np.array_equal(st.cpu().numpy().reshape(H, D, D), got["rec_state"])
    cs = dev_bf16(cv["state"])
    co = torch.empty(1, 37, 1536, dtype=torch.bfloat16, device="cuda")
    hk.cuda_causal_conv1d_update(dev_bf16(cv["x"]), cs, None, dev_bf16(cv["weight"]), None, co, 1, 1536, 37, 4, 4, True, False)
    idx = torch.empty(3, 512, dtype=torch.int32, device="cuda")
    hk.dsa_topk(dev_f16(sc), 1000, idx, 3, 1000, 512, 512)
    y = torch.empty(64, 128, dtype=torch.float16, device="cuda")
    hk.gated_rms_norm(dev_bf16(nx), dev_bf16(nw), y, dev(ng), 64, 128, 1e-6, gate_act=1)
    mixed = torch.empty(F, S, dtype=torch.bfloat16, device="cuda")
    beta = torch.empty(S, H, dtype=torch.bfloat16, device="cuda")
    gg = torch.empty(S, H, D, dtype=torch.float32, device="cuda")
    hk.kda_transpose_cast(mixed, dev(pq), S, F)
    hk.kda_gate(dev(raw["b"]), dev(raw["f"]), dev(raw["dt_bias"]), dev(raw["a_log"]), -5.0, beta, gg, S, H, D)
    torch.cuda.synchronize()
    assert np.array_equal(bits(co).reshape(37, 1536), got["conv_out"]) and np.array_equal(bits(cs).reshape(1536, 4), got["conv_state"])
    assert np.array_equal(idx.cpu().numpy(), got["topk_idx"])
    assert np.array_equal(idx.cpu().numpy(), orc.dsa_topk(sc, 1000, 3, 1000, 512, 512)), "and the oracle's selection"
    assert np.array_equal(bits(y), got["norm_y"])
    for k, t in (("prep_mixed", mixed), ("prep_beta", beta), ("prep2_mixed", mixed), ("prep2_beta", beta)):
        assert np.array_equal(bits(t), got[k]), k
    assert np.array_equal(gg.cpu().numpy(), got["prep_g"]) and np.array_equal(gg.cpu().numpy(), got["prep2_g"])
    # values, not only agreement: the recurrence against the oracle
    _, o_32, o_st = orc.kda_recurrent(inp["mixed_qkv"], inp["g"], inp["beta"], s0, 1, T, H, H, D, D)
    assert frob_rel(got["rec_state"].reshape(1, 1, H, D, D), o_st) < 1e-2


def test_reference_repeatability_binary_against_this_library():
    """The reference's own test/test_deterministic_reductions.cu (12 recurrence configurations, 16 repeats each,
    byte-identical state and output), built from the reference tree with the recurrence launcher taken from
    libhelios_b200.so."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_deterministic_reductions_on_b200")
    if not os.path.exists(exe):
        pytest.skip("reference test binary not built (make -C oracle reftest)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.count("PASS recurrence") == 12, r.stdout[-2000:] + r.stderr[-2000:]


def test_kda_snapshot_taken_from_reference_kernels_restores_into_this_library():
    """The engine snapshots the KDA state as, per KDA layer ordinal, [conv window bytes][recurrent state bytes]
    (src/engine/runner.cpp:319-335, sizes :1422-1424).  Two layers are prefilled (conv + recurrence) by the
    reference's own kernels, their planes are concatenated in that layout, copied into fresh planes (the restore),
    and 8 decode steps are run by this library; the result equals the oracle run end to end."""
    if not ref.available():
        pytest.skip("reference kernels not built (make -C oracle ref)")
    H, D, T, steps, n_layers = 8, 128, 300, 8, 2
    dim = 3 * H * D
    conv_bytes, rec_bytes = dim * 4 * 2, H * D * D * 4
    snap = torch.empty(n_layers * (conv_bytes + rec_bytes), dtype=torch.uint8, device="cuda")
    layers = []
    for L in range(n_layers):
        r = synth.rng(60 + L)
        x = synth.f32_to_bf16_bits(r.standard_normal((dim, T + steps), dtype=np.float32))
        w = synth.f32_to_bf16_bits((0.1 * r.standard_normal((dim, 4), dtype=np.float32)).astype(np.float32))
        gates = synth.kda_gates(T + steps, H, D, seed=60 + L)
        layers.append((x, w, gates))
        xd, wd, gd, bd = dev_bf16(x), dev_bf16(w), dev(gates["g"]), dev_bf16(gates["beta"])
        cs = torch.zeros(1, dim, 4, dtype=torch.bfloat16, device="cuda")
        st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
        qkv = torch.empty(1, T, dim, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
        ref.conv1d_update(xd[:, :T].contiguous().view(1, dim, T), cs, None, wd, None, qkv, 1, dim, T, 4, 4, True, False)
        ref.kda_recurrent(qkv, gd[:, :T].contiguous(), bd[:, :T].contiguous(), st, out, 1, T, H, H, D, D, 1, None, True, False)
        off = L * (conv_bytes + rec_bytes)
        snap[off:off + conv_bytes] = cs.view(torch.uint8).reshape(-1)          # snapshot: D2D copies into one buffer
        snap[off + conv_bytes:off + conv_bytes + rec_bytes] = st.view(torch.uint8).reshape(-1)
    torch.cuda.synchronize()
    host = snap.cpu()                                          # the engine keeps snapshots in pinned host memory
    for L, (x, w, gates) in enumerate(layers):
        off = L * (conv_bytes + rec_bytes)
        cs = host[off:off + conv_bytes].cuda().view(torch.bfloat16).view(1, dim, 4).clone()        # restore
        st = host[off + conv_bytes:off + conv_bytes + rec_bytes].cuda().view(torch.float32).view(1, 1, H, D, D).clone()
        xd, wd, gd, bd = dev_bf16(x), dev_bf16(w), dev(gates["g"]), dev_bf16(gates["beta"])
        o32 = torch.empty(steps, 1, H, D, dtype=torch.float32, device="cuda")
        out = torch.empty(steps, 1, H, D, dtype=torch.bfloat16, device="cuda")
        for s in range(steps):
            hk.kda_decode_step(xd[:, T + s].contiguous().view(1, dim), cs, wd, None, gd[:, T + s], bd[:, T + s], st, out[s], 1, H,
                               out_f32=o32[s])
        torch.cuda.synchronize()
        # oracle end to end: conv + recurrence over T + steps tokens from zero state
        o_qkv, o_cst = orc.conv1d_update(x.reshape(1, dim, T + steps), np.zeros((1, dim, 4), np.uint16), w, None, 1, dim, T + steps, 4, 4)
        _, o_32, o_st = orc.kda_recurrent(o_qkv, gates["g"], gates["beta"], np.zeros((1, 1, H, D, D), np.float32), 1, T + steps,
                                          H, H, D, D)
        assert np.array_equal(bits(cs), o_cst), "conv window after restore + decode"
        assert frob_rel(st.cpu().numpy(), o_st) < 1e-2
        assert max_rel(o32.cpu().numpy().reshape(1, steps, H, D), o_32[:, T:]) < 2e-3
