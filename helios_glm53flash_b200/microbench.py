"""Per-kernel micro-benchmarks of libhelios_b200 on synthetic inputs.

    python -m helios_glm53flash_b200.microbench --case mla_dense_b8 [--iters 20] [--warmup 3]

Each case times one entry point with CUDA events on the current stream (median of --iters, L2 flushed
by a 256 MB write between iterations unless the working set exceeds L2 by itself) and prints one JSON
line with the time and the achieved algorithmic bandwidth.  The cases are small enough to be captured
under a profiler (a few hundred MB on the device).
"""
import argparse
import json

import numpy as np


def _bits16(t, dtype):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t).view(np.int16)).view(dtype).cuda()


def build_case(name):
    """returns (callable, algorithmic_bytes, needs_flush, description)"""
    import torch
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import synth
    H, D = 32, 128
    if name in ("kda_prefill_8k", "kda_prefill_32k", "kda_recurrent_512"):
        T = {"kda_prefill_8k": 8192, "kda_prefill_32k": 32768, "kda_recurrent_512": 512}[name]
        gates = synth.kda_gates(T, H, D, seed=1)
        g, beta = torch.from_numpy(gates["g"]).cuda(), _bits16(gates["beta"], torch.bfloat16)
        qkv = torch.randn(1, T, 3 * H * D, device="cuda").to(torch.bfloat16)
        st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
        out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(hk.kda_chunked_workspace_bytes(1, T, H), dtype=torch.uint8, device="cuda")
        force = name == "kda_recurrent_512"

        def fn():
            hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, st, out, 1, T, H, H, D, D, 1, None, True, False,
                                               workspace=ws, force_recurrent=force)
        return fn, T * H * 1538 + 2 * H * D * D * 4, T < 8192, "KDA prefill T=%d H=32 (chunked unless 'recurrent')" % T
    if name in ("conv_8k", "conv_32k"):
        T = 8192 if name == "conv_8k" else 32768
        dim = 3 * H * D
        x = torch.randn(1, dim, T, device="cuda").to(torch.bfloat16)
        w = (0.1 * torch.randn(dim, 4, device="cuda")).to(torch.bfloat16)
        st = torch.zeros(1, dim, 4, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(1, T, dim, dtype=torch.bfloat16, device="cuda")

        def fn():
            hk.cuda_causal_conv1d_update(x, st, None, w, None, out, 1, dim, T, 4, 4, True, False)
        return fn, 4 * dim * T, False, "short conv + SiLU, 12288 channels x %d tokens" % T
    if name in ("transpose_cast_32k", "gate_32k", "gated_norm_32k", "cast_conv_32k", "kda_prefill_gated_32k",
                "transpose_cast_4k", "gate_4k", "gated_norm_4k", "cast_conv_4k"):
        T = 4096 if name.endswith("_4k") else 32768
        F = 3 * H * D
        kind = name.rsplit("_", 1)[0]
        if kind == "transpose_cast":
            x = torch.randn(T, F, device="cuda")
            dst = torch.empty(F, T, dtype=torch.bfloat16, device="cuda")

            def fn():
                hk.kda_transpose_cast(dst, x, T, F)
            return fn, 6 * T * F, False, "transpose + cast, %d tokens x 12288 channels (fp32 in, bf16 out)" % T
        if kind == "cast_conv":
            x = torch.randn(1, T, F, device="cuda")
            w = (0.1 * torch.randn(F, 4, device="cuda")).to(torch.bfloat16)
            st = torch.zeros(1, F, 4, dtype=torch.bfloat16, device="cuda")
            out = torch.empty(1, T, F, dtype=torch.bfloat16, device="cuda")

            def fn():
                hk.kda_cast_conv(x, st, None, w, None, out, 1, F, T, True)
            return fn, 6 * T * F, False, "cast + short conv + SiLU from token-major fp32, %d tokens x 12288 channels" % T
        raw = synth.kda_raw_gates(T, H, D, seed=2)
        f, b = torch.from_numpy(raw["f"]).cuda(), torch.from_numpy(raw["b"]).cuda()
        dtb, al = torch.from_numpy(raw["dt_bias"]).cuda(), torch.from_numpy(raw["a_log"]).cuda()
        if kind == "gate":
            beta = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
            g = torch.empty(T, H, D, dtype=torch.float32, device="cuda")

            def fn():
                hk.kda_gate(b, f, dtb, al, raw["lower_bound"], beta, g, T, H, D)
            return fn, T * H * (8 * D + 6), False, "gate preparation, %d tokens x 32 heads x 128" % T
        if kind == "gated_norm":
            x = torch.randn(T * H, D, device="cuda").to(torch.bfloat16)
            w = torch.ones(D, dtype=torch.bfloat16, device="cuda")
            y = torch.empty(T * H, D, dtype=torch.float16, device="cuda")

            def fn():
                hk.gated_rms_norm(x, w, y, f, T * H, D, 1e-6, gate_act=1)
            return fn, T * H * D * 8, False, "gated RMS norm (sigmoid), %d rows of 128 (bf16 in, fp32 gate, fp16 out)" % (T * H)
        qkv = torch.randn(1, T, F, device="cuda").to(torch.bfloat16)
        st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
        out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(hk.kda_chunked_workspace_bytes(1, T, H), dtype=torch.uint8, device="cuda")

        def fn():
            hk.kda_chunked_prefill_gated(qkv, f, b, dtb, al, raw["lower_bound"], st, out, 1, T, H, workspace=ws)
        return fn, T * H * 1538 + 2 * H * D * D * 4, False, "KDA prefill with the gates formed in the kernel, T=%d H=32" % T
    if name == "kda_decode":
        kd = synth.kda_inputs(1, H, D, seed=5)
        q, g, b = _bits16(kd["mixed_qkv"], torch.bfloat16), torch.from_numpy(kd["g"]).cuda(), _bits16(kd["beta"], torch.bfloat16)
        st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
        o = torch.empty(1, 1, H, D, dtype=torch.bfloat16, device="cuda")

        def fn():
            hk.cuda_recurrent_gated_delta_rule(q, g, b, st, o, 1, 1, H, H, D, D, 1, None, True, False)
        return fn, 2 * H * D * D * 4 + H * 1538, True, "KDA decode step, 32 heads"
    if name in ("mla_dense_b1", "mla_dense_b8", "mla_dense_b1_simt"):
        B = 8 if name == "mla_dense_b8" else 1
        L = 32768
        ck = torch.randn(B * L, 512, dtype=torch.float16, device="cuda")
        qd = torch.randn(B, 64, 512, dtype=torch.float16, device="cuda")
        base = torch.from_numpy((np.arange(B) * L).astype(np.int64)).cuda()
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        lo = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(B, L)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, B * 64)), dtype=torch.uint8, device="cuda")

        def fn():
            hk.mla_dense_prefill(qd, ck, lo, B, 0, scale=512 ** -0.5, kv_base=base, kv_len=lens, n_split=ns,
                                 workspace=wsb, n_keys_hint=L)
        return fn, B * L * 1024, B == 1, "dense MLA decode, batch %d x 32768 latents, %d splits" % (B, ns)
    if name == "mla_prefill_256":
        qlen, pos = 256, 32768
        ck = torch.randn(pos + qlen, 512, dtype=torch.float16, device="cuda")
        qd = torch.randn(qlen, 64, 512, dtype=torch.float16, device="cuda")
        lo = torch.empty(qlen, 64, 512, dtype=torch.float16, device="cuda")

        def fn():
            hk.mla_dense_prefill(qd, ck, lo, qlen, pos, scale=512 ** -0.5, n_split=1)
        return fn, (pos + qlen) * 1024 + 2 * qlen * 65536, True, "dense causal MLA prefill, 256 rows after 32768"
    if name in ("indexer_262k", "indexer_prefill_256"):
        npools = 65536
        m = 1 if name == "indexer_262k" else 256
        ix = synth.indexer_inputs(npools, m, seed=7)
        qi, pk, w = _bits16(ix["q_idx"], torch.float16), _bits16(ix["pool_k"], torch.float16), _bits16(ix["w"], torch.float16)
        q_pos = torch.full((m,), 4 * npools - 1, dtype=torch.int32, device="cuda")
        sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")

        def fn():
            hk.indexer_score(qi, pk, w, q_pos, sc, m, npools)
        return fn, npools * 256 + m * npools * 2, True, "indexer scores, %d rows x 65536 pools" % m
    if name in ("q_latent_4096", "o_absorb_4096"):
        n = 4096
        kb = (0.05 * torch.randn(32768, 512, device="cuda")).half()
        if name == "q_latent_4096":
            qn = torch.randn(n, 64, 256, device="cuda").half()
            ql = torch.empty(n, 64, 512, dtype=torch.float16, device="cuda")

            def fn():
                hk.q_latent(qn, kb, ql, n)
        else:
            lo = torch.randn(n, 64, 512, device="cuda").half()
            o = torch.empty(n, 64, 256, dtype=torch.float16, device="cuda")

            def fn():
                hk.o_absorb(lo, kb, o, n)
        return fn, n * 64 * (256 + 512) * 2 + 64 * 256 * 512 * 2, True, "absorbed projection, 4096 rows x 64 heads (68.7 GFLOP)"
    if name == "topk_262k":
        npools = 65536
        sc = torch.randn(1, npools, device="cuda").half()
        idx = torch.empty(1, 512, dtype=torch.int32, device="cuda")

        def fn():
            hk.dsa_topk(sc, npools, idx, 1, npools, 512, 512)
        return fn, npools * 2, True, "top-512 of 65536 fp16 scores, one row"
    if name == "sparse_262k":
        L = 262144
        ck = torch.randn(L, 512, dtype=torch.float16, device="cuda")
        ql = torch.randn(1, 64, 512, dtype=torch.float16, device="cuda")
        raw = torch.randint(0, L, (1, 2052), dtype=torch.int32, device="cuda")
        lo = torch.empty(1, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(1, 2052)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, 64)), dtype=torch.uint8, device="cuda")

        def fn():
            hk.mla_sparse_decode(ql, ck, raw, 2052, lo, 1, n_split=ns, workspace=wsb)
        return fn, 2052 * 1024, True, "sparse MLA decode, 2052 gathered latents of 262144, %d splits" % ns
    raise SystemExit("unknown case " + name)


CASES = ["kda_prefill_8k", "kda_prefill_32k", "kda_recurrent_512", "conv_8k", "conv_32k", "kda_decode", "mla_dense_b1",
         "mla_dense_b8", "mla_prefill_256", "indexer_262k", "indexer_prefill_256", "topk_262k", "sparse_262k", "q_latent_4096", "o_absorb_4096",
         "transpose_cast_32k", "gate_32k", "gated_norm_32k", "cast_conv_32k", "kda_prefill_gated_32k", "transpose_cast_4k",
         "gate_4k", "gated_norm_4k", "cast_conv_4k"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, help="one of: " + ", ".join(CASES) + ", 'all', or 'tc05_issue' (cycles per tensor-core product by shape and issue form)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true",
                    help="capture the call in a CUDA graph and time its replay (no host launch latency in the figure)")
    args = ap.parse_args()
    import torch
    import helios_glm53flash_b200 as hk
    if args.case == "tc05_issue":
        # not a timing of a library call: SM clock ticks per tcgen05 product by shape and issue form
        for M, N in [(64, 16), (64, 48), (64, 96), (64, 128), (64, 256), (128, 32), (128, 64), (128, 128), (128, 256)]:
            row = {"case": "tc05_issue", "M": M, "N": N, "K": 16}
            for conv in (0, 1):
                for count in (32, 512):
                    hk.tc05_issue_probe(M, N, conv, count)
                    issue, done = hk.tc05_issue_probe(M, N, conv, count)
                    row["%s_burst%d_cycles_per_mma" % ("converged_warp" if conv else "single_thread", count)] = round(done / count, 1)
            print(json.dumps(row), flush=True)
        return
    for name in (CASES if args.case == "all" else [args.case]):
        fn, nbytes, flush, desc = build_case(name)
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        if args.graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            call = graph.replay
        else:
            call = fn
        ts = []
        for _ in range(args.iters):
            if buf is not None:
                buf.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            call()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        ms = ts[len(ts) // 2]
        print(json.dumps({"case": name + ("+graph" if args.graph else ""), "desc": desc, "us": ms * 1e3, "algorithmic_GBps": nbytes / (ms * 1e-3) / 1e9,
                          "device_status": hk.read_device_status()}), flush=True)
        del fn, buf
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
