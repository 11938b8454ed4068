"""The reference's own CUDA kernels, compiled for sm_100a from the reference tree (oracle/_ref/libhelios_ref.so),
timed on this GPU next to this library's kernels on the same buffers.  A script, not a pytest module:

    python tests/time_reference_kernels.py [--iters 10] [--case NAME ...]

One JSON line per case: median device time (CUDA events on the current stream, 2 warm-ups, 256 MB L2
flush before every timed call) of the reference kernel and of libhelios_b200, and their ratio.  Inputs
are seeded synthetic tensors with the shapes of the benchmark configurations.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def timed(torch, fn, iters, flush):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2] * 1e3          # microseconds


def cases(torch, hk, ref, synth):
    H, D = 32, 128
    bf = torch.bfloat16

    def bits16(a, dtype):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dtype).cuda()

    def kda(T):
        gates = synth.kda_gates(T, H, D, seed=1)
        g, beta = torch.from_numpy(gates["g"]).cuda(), bits16(gates["beta"], bf)
        qkv = torch.randn(1, T, 3 * H * D, device="cuda").to(bf)
        st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
        out = torch.empty(1, T, H, D, dtype=bf, device="cuda")
        ws = torch.empty(max(256, hk.kda_chunked_workspace_bytes(1, T, H)), dtype=torch.uint8, device="cuda")
        ours = lambda: hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, st, out, 1, T, H, H, D, D, 1, None, True, False, workspace=ws)
        theirs = lambda: ref.kda_recurrent(qkv, g, beta, st, out, 1, T, H, H, D, D, 1, None, True, False)
        return ours, theirs

    def conv(T):
        dim = 3 * H * D
        x = torch.randn(1, dim, T, device="cuda").to(bf)
        w = (0.1 * torch.randn(dim, 4, device="cuda")).to(bf)
        st = torch.zeros(1, dim, 4, dtype=bf, device="cuda")
        out = torch.empty(1, T, dim, dtype=bf, device="cuda")
        ours = lambda: hk.cuda_causal_conv1d_update(x, st, None, w, None, out, 1, dim, T, 4, 4, True, False)
        theirs = lambda: ref.conv1d_update(x, st, None, w, None, out, 1, dim, T, 4, 4, True, False)
        return ours, theirs

    def indexer(m):
        npools = 65536
        ix = synth.indexer_inputs(npools, m, seed=7)
        qi, pk, w = bits16(ix["q_idx"], torch.float16), bits16(ix["pool_k"], torch.float16), bits16(ix["w"], torch.float16)
        q_pos = torch.full((m,), 4 * npools - 1, dtype=torch.int32, device="cuda")
        sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")
        ours = lambda: hk.indexer_score(qi, pk, w, q_pos, sc, m, npools)
        theirs = lambda: ref.indexer_score(qi, pk, w, q_pos, sc, m, npools)
        return ours, theirs

    def topk():
        npools = 65536
        sc = torch.randn(1, npools, device="cuda").half()
        idx = torch.empty(1, 512, dtype=torch.int32, device="cuda")
        ours = lambda: hk.dsa_topk(sc, npools, idx, 1, npools, 512, 512)
        theirs = lambda: ref.dsa_topk(sc, npools, idx, 1, npools, 512, 512)
        return ours, theirs

    def sparse(m):
        L, kidx = 262144, 2052
        ck = torch.randn(L, 512, dtype=torch.float16, device="cuda")
        q = torch.randn(m, 64, 512, dtype=torch.float16, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(3)
        raw = torch.randint(0, L, (m, kidx), generator=g, device="cuda", dtype=torch.int32)
        lo = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
        ours = lambda: hk.mla_sparse_decode(q, ck, raw, kidx, lo, m)
        theirs = lambda: ref.mla_sparse_decode(q, ck, raw, kidx, lo, m)
        return ours, theirs

    def dense(qlen, pos):
        ck = torch.randn(pos + qlen, 512, dtype=torch.float16, device="cuda")
        q = torch.randn(qlen, 64, 512, dtype=torch.float16, device="cuda")
        lo = torch.empty(qlen, 64, 512, dtype=torch.float16, device="cuda")
        ours = lambda: hk.mla_dense_prefill(q, ck, lo, qlen, pos)
        theirs = lambda: ref.mla_dense_prefill(q, ck, lo, qlen, pos)
        return ours, theirs

    def absorb(n, which):
        kb = (0.05 * torch.randn(32768, 512, device="cuda")).half()
        if which == "q":
            qn = torch.randn(n, 64, 256, device="cuda").half()
            ql = torch.empty(n, 64, 512, dtype=torch.float16, device="cuda")
            return (lambda: hk.q_latent(qn, kb, ql, n)), (lambda: ref.q_latent_t(qn, kb, ql, n))
        lo = torch.randn(n, 64, 512, device="cuda").half()
        o = torch.empty(n, 64, 256, dtype=torch.float16, device="cuda")
        wt = torch.empty(64, 512, 256, dtype=torch.float16, device="cuda")
        ref.wuv_transpose(kb, wt)
        return (lambda: hk.o_absorb(lo, kb, o, n)), (lambda: ref.o_absorb_t(lo, wt, o, n))

    def glue(kind, T):
        F = 3 * H * D
        if kind == "transpose":
            x = torch.randn(T, F, device="cuda")
            dst = torch.empty(F, T, dtype=bf, device="cuda")
            return (lambda: hk.kda_transpose_cast(dst, x, T, F)), (lambda: ref.kda_transpose_cast(dst, x, T, F))
        raw = synth.kda_raw_gates(T, H, D, seed=2)
        f, b = torch.from_numpy(raw["f"]).cuda(), torch.from_numpy(raw["b"]).cuda()
        dtb, al, lb = torch.from_numpy(raw["dt_bias"]).cuda(), torch.from_numpy(raw["a_log"]).cuda(), raw["lower_bound"]
        if kind == "gate":
            beta = torch.empty(T, H, dtype=bf, device="cuda")
            g = torch.empty(T, H, D, dtype=torch.float32, device="cuda")
            return (lambda: hk.kda_gate(b, f, dtb, al, lb, beta, g, T, H, D)), (lambda: ref.kda_gate(b, f, dtb, al, lb, beta, g, T, H, D))
        x = torch.randn(T * H, D, device="cuda").to(bf)
        w = torch.ones(D, dtype=bf, device="cuda")
        y = torch.empty(T * H, D, dtype=torch.float16, device="cuda")
        return ((lambda: hk.gated_rms_norm(x, w, y, f, T * H, D, 1e-6, gate_act=1)),
                (lambda: ref.gated_rms_norm(x, w, y, f, T * H, D, 1e-6, gate_act=1)))

    return {
        "transpose_cast_32k": (lambda: glue("transpose", 32768), "transpose + cast, 32768 tokens x 12288 channels", 10),
        "gate_32k": (lambda: glue("gate", 32768), "gate preparation, 32768 tokens x 32 heads x 128", 10),
        "gated_norm_32k": (lambda: glue("norm", 32768), "gated RMS norm, 1048576 rows of 128", 10),
        "kda_prefill_32k": (lambda: kda(32768), "KDA layer prefill, T=32768, H=32, d=128 (reference: per-token recurrence)", 3),
        "kda_prefill_4k": (lambda: kda(4096), "KDA layer prefill, T=4096, H=32", 5),
        "kda_decode": (lambda: kda(1), "KDA decode step, H=32", 20),
        "conv_32k": (lambda: conv(32768), "short conv + SiLU, 12288 channels x 32768 tokens", 10),
        "indexer_m1": (lambda: indexer(1), "indexer scores, 1 row x 65536 pools", 20),
        "indexer_m256": (lambda: indexer(256), "indexer scores, 256 rows x 65536 pools", 5),
        "topk_65536": (topk, "top-512 of 65536 scores, 1 row", 20),
        "sparse_m1": (lambda: sparse(1), "sparse MLA decode, 1 row, 2052 gathered latents of 262144", 20),
        "sparse_m256": (lambda: sparse(256), "sparse MLA, 256 rows x 2052 gathered latents", 5),
        "dense_decode_32k": (lambda: dense(1, 32767), "dense MLA decode, 1 row over 32768 latents", 10),
        "dense_prefill_256": (lambda: dense(256, 32768), "dense causal MLA prefill, 256 rows after 32768", 3),
        "q_latent_4096": (lambda: absorb(4096, "q"), "absorbed query projection, 4096 rows x 64 heads (reference: q_latent_t)", 5),
        "o_absorb_4096": (lambda: absorb(4096, "o"), "absorbed output projection, 4096 rows x 64 heads (reference: o_absorb_t on transposed weights)", 5),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=0, help="override the per-case iteration count")
    ap.add_argument("--case", action="append", default=[])
    args = ap.parse_args()
    import torch
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import synth
    import hk_ref as ref
    if not ref.available():
        raise SystemExit("oracle/_ref/libhelios_ref.so is not built (make -C oracle ref)")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = cases(torch, hk, ref, synth)
    for name in (args.case or list(table)):
        build, desc, iters = table[name]
        ours, theirs = build()
        iters = args.iters or iters
        t_ref = timed(torch, theirs, iters, flush)
        t_ours = timed(torch, ours, iters, flush)
        print(json.dumps({"case": name, "desc": desc, "reference_kernel_us": t_ref, "this_library_us": t_ours,
                          "speedup": t_ref / t_ours, "iters": iters, "device_status": hk.read_device_status()}), flush=True)
        del ours, theirs
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
