"""Generates tests/golden/reference_kernels.npz: outputs of the REFERENCE's own CUDA kernels
(oracle/_ref/libhelios_ref.so, built from the reference tree by `make -C oracle ref`) on small seeded
inputs.  Run on a machine with a GPU:

    python tests/golden/make_golden.py [output.npz]

Inputs are rebuilt from seeds by `cases()` below (also imported by the CPU test that checks the
oracle against these fixtures), so only the outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helios_glm53flash_b200 import synth  # noqa: E402


def cases():
    """name -> dict of numpy inputs (deterministic)"""
    c = {}
    # KDA recurrence: channelwise 128-dim (GLM shape, 2 heads, 24 tokens, non-zero initial state),
    # and head-wide decay at dim 64
    k = synth.kda_inputs(24, 2, 128, seed=41)
    k["state"] = (0.1 * synth.rng(42).standard_normal((1, 1, 2, 128, 128), dtype=np.float32)).astype(np.float32)
    c["kda_cw128"] = k
    k = synth.kda_inputs(9, 2, 64, seed=43)
    k["g"] = np.ascontiguousarray(k["g"][..., 0])
    k["state"] = (0.1 * synth.rng(44).standard_normal((1, 1, 2, 64, 64), dtype=np.float32)).astype(np.float32)
    c["kda_hw64"] = k
    c["conv"] = synth.conv_inputs(40, 64, seed=45)
    r = synth.rng(46)
    c["kpool"] = {"idx_k": synth.f32_to_f16_bits(r.uniform(-1, 1, (24, 128)).astype(np.float32)),
                  "idx_g": synth.f32_to_f16_bits((3 * r.uniform(-1, 1, (24, 128))).astype(np.float32)),
                  "ape": (2 * r.uniform(-1, 1, (4, 128))).astype(np.float32)}
    ix = synth.indexer_inputs(96, 3, seed=47)
    ix["q_pos"] = np.array([383, 200, 17], dtype=np.int32)
    c["indexer"] = ix
    sc = np.round(synth.rng(48).standard_normal((3, 700), dtype=np.float32) * 4) / 4
    sc[1, 20:] = -np.inf
    sc[2, 300:] = -np.inf
    c["topk"] = {"scores": synth.f32_to_f16_bits(sc)}
    ml = synth.mla_inputs(256, 4, seed=49, cache_std=0.5)
    rs = np.random.RandomState(50)
    ridx = rs.randint(0, 256, (2, 40)).astype(np.int32)
    ridx[:, 5::9] = -1
    ml["raw_idx"] = ridx
    c["mla"] = ml
    pidx = np.where(np.arange(2 * 512) % 5 == 0, -1, rs.randint(0, 40, 2 * 512)).astype(np.int32).reshape(2, 512)
    c["expand"] = {"pool_idx": pidx, "q_pos": np.array([150, 3], dtype=np.int32)}
    # KDA producers / consumer: gate preparation, transpose + cast, gated RMS norm (sigmoid gate, dim 128)
    gt = synth.kda_raw_gates(10, 3, 128, seed=51)
    gt["qkv"] = synth.rng(52).standard_normal((10, 72), dtype=np.float32)
    c["kda_prepare"] = gt
    r = synth.rng(53)
    c["gated_norm"] = {"x": synth.f32_to_bf16_bits(r.standard_normal((12, 128), dtype=np.float32)),
                       "w": synth.f32_to_bf16_bits((1 + 0.1 * r.standard_normal(128, dtype=np.float32)).astype(np.float32)),
                       "g": (2 * r.standard_normal((12, 128), dtype=np.float32)).astype(np.float32)}
    return c


def main(out_path):
    import torch
    import hk_ref as ref
    from gpu_util import bits, dev, dev_bf16, dev_f16
    assert ref.available(), "oracle/_ref/libhelios_ref.so missing"
    c = cases()
    g = {}
    for name, (dim, cw) in {"kda_cw128": (128, True), "kda_hw64": (64, False)}.items():
        k = c[name]
        T = k["mixed_qkv"].shape[1]
        st = dev(k["state"])
        out = torch.empty(1, T, 2, dim, dtype=torch.bfloat16, device="cuda")
        ref.kda_recurrent(dev_bf16(k["mixed_qkv"]), dev(k["g"]), dev_bf16(k["beta"]), st, out, 1, T, 2, 2, dim, dim, 1,
                          None, cw, False)
        torch.cuda.synchronize()
        g[name + "_out"] = bits(out)
        g[name + "_state"] = st.cpu().numpy()
    k = c["conv"]
    st = dev_bf16(k["state"])
    out = torch.empty(1, 40, 64, dtype=torch.bfloat16, device="cuda")
    ref.conv1d_update(dev_bf16(k["x"]), st, None, dev_bf16(k["weight"]), None, out, 1, 64, 40, 4, 4, True, False)
    torch.cuda.synchronize()
    g["conv_out"], g["conv_state"] = bits(out), bits(st)
    k = c["kpool"]
    ring = torch.zeros(32, 256, dtype=torch.float16, device="cuda")
    pk = torch.zeros(6, 128, dtype=torch.float16, device="cuda")
    dk_, dg_, da_ = dev_f16(k["idx_k"]), dev_f16(k["idx_g"]), dev(k["ape"])
    ref.kpool_write(dk_, dg_, ring, 32, pk, da_, 0, 10)          # a chunk that ends mid-pool
    ref.kpool_write(dk_[10:], dg_[10:], ring, 32, pk, da_, 10, 14)
    torch.cuda.synchronize()
    g["kpool_pk"] = bits(pk)
    k = c["indexer"]
    sc = torch.empty(3, 96, dtype=torch.float16, device="cuda")
    ref.indexer_score(dev_f16(k["q_idx"]), dev_f16(k["pool_k"]), dev_f16(k["w"]), dev(k["q_pos"]), sc, 3, 96)
    torch.cuda.synchronize()
    g["indexer_scores"] = bits(sc)
    k = c["topk"]
    idx = torch.empty(3, 72, dtype=torch.int32, device="cuda")
    ref.dsa_topk(dev_f16(k["scores"]), 700, idx, 3, 700, 64, 72, t_seq=700)
    torch.cuda.synchronize()
    g["topk_idx"] = idx.cpu().numpy()
    k = c["mla"]
    q, ck = dev_f16(k["q_lat"]), dev_f16(k["ckv"])
    lo = torch.empty(2, 64, 512, dtype=torch.float16, device="cuda")
    ref.mla_sparse_decode(q, ck, dev(k["raw_idx"]), 40, lo, 2)
    lo2 = torch.empty(4, 64, 512, dtype=torch.float16, device="cuda")
    ref.mla_dense_prefill(q, ck, lo2, 4, 100)
    torch.cuda.synchronize()
    g["mla_sparse_out"], g["mla_dense_out"] = bits(lo), bits(lo2)
    k = c["expand"]
    raw = torch.empty(2, 2052, dtype=torch.int32, device="cuda")
    ref.pool_expand_row(dev(k["pool_idx"]), dev(k["q_pos"]), raw, 2)
    torch.cuda.synchronize()
    g["expand_raw"] = raw.cpu().numpy()
    k = c["kda_prepare"]
    mixed = torch.empty(72, 10, dtype=torch.bfloat16, device="cuda")
    beta = torch.empty(10, 3, dtype=torch.bfloat16, device="cuda")
    gg = torch.empty(10, 3, 128, dtype=torch.float32, device="cuda")
    ref.kda_transpose_cast(mixed, dev(k["qkv"]), 10, 72)
    ref.kda_gate(dev(k["b"]), dev(k["f"]), dev(k["dt_bias"]), dev(k["a_log"]), k["lower_bound"], beta, gg, 10, 3, 128)
    torch.cuda.synchronize()
    g["prepare_mixed"], g["prepare_beta"], g["prepare_g"] = bits(mixed), bits(beta), gg.cpu().numpy()
    k = c["gated_norm"]
    y = torch.empty(12, 128, dtype=torch.float16, device="cuda")
    ref.gated_rms_norm(dev_bf16(k["x"]), dev_bf16(k["w"]), y, dev(k["g"]), 12, 128, 1e-6, gate_act=1)
    torch.cuda.synchronize()
    g["gated_norm_y"] = bits(y)
    np.savez_compressed(out_path, **g)
    print("wrote", out_path, {n: v.shape for n, v in g.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_kernels.npz"))
