#!/usr/bin/env python
"""Benchmark of the trunk-attention hot path on B200.

Headline workload (N = 1): one KDA layer prefill at 32,768 tokens, batch 1, 32 heads x 128 (d_k = d_v),
chunk 64, bf16 inputs, fp32 state - one step = short conv (+SiLU) over the 12,288 q|k|v channels
followed by the chunked gated-delta-rule prefill.  Synthetic inputs with the benchmark's value
distributions (helios_glm53flash_b200.synth); inputs are larger than L2, so no flush is needed
between steps.  With N > 1 every rank runs the same workload on its own sequence (weak scaling, no
collective on the data path); timing is device-side, max over ranks.

One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the reference's
algorithm (the reference has no CPU implementation of this path and is CUDA-only) on
the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

T_FULL, HEADS, DIM = 32768, 32, 128
CPU_SAMPLE_T = 32768
METRIC = "kda_prefill_tokens_per_s_at_32k_ctx"


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """one `nvidia-smi -lms` process sampling SM clocks and throttle reasons; samples are stamped on
    arrival so that the ones taken inside the timed region can be picked out"""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.thread = [], None, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "10"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.rows.append((time.time(), parts))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t_begin, t_end):
        inside = [r for ts, r in self.rows if t_begin <= ts <= t_end]
        note = "samples inside the timed region"
        if not inside:
            inside = [r for _, r in self.rows]
            note = "no sample fell inside the timed region; all samples of the run (warm-up included)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in inside if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in inside)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(inside[0][1]) if inside[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(inside), "note": note}


def cpu_baseline(steps=1, sample_t=CPU_SAMPLE_T):
    """oracle (CPU port of the reference algorithm) on a bounded sample: conv + recurrence over
    `sample_t` tokens of the same workload, all host threads"""
    import numpy as np
    import hk_oracle as orc
    from helios_glm53flash_b200 import synth
    dim = 3 * HEADS * DIM
    cv = synth.conv_inputs(sample_t, dim, seed=0)
    kd = synth.kda_gates(sample_t, HEADS, DIM, seed=0)
    state = np.zeros((1, 1, HEADS, DIM, DIM), dtype=np.float32)
    best = None
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        qkv, _ = orc.conv1d_update(cv["x"], cv["state"], cv["weight"], None, 1, dim, sample_t, 4, 4)
        orc.kda_recurrent(qkv, kd["g"], kd["beta"], state, 1, sample_t, HEADS, HEADS, DIM, DIM)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": sample_t / best, "unit": "tok/s", "cores": orc.threads(), "kind": "port",
            "sample": "conv + recurrence over %d of the 32768 tokens, 32 heads, best of %d; cost is linear in tokens"
                      % (sample_t, max(1, steps)), "seconds": best * (T_FULL / sample_t)}


def _reference_kernels_on_gpu(args):
    """the reference's own conv + recurrence kernels (its sm_86 sources compiled unchanged for sm_100a into
    oracle/_ref/libhelios_ref.so) on the full 32,768-token workload, device-timed; None when the library or a
    GPU is missing"""
    try:
        import torch
        import hk_ref
        if not (torch.cuda.is_available() and hk_ref.available()):
            return None
        hk_ref.lib()
    except Exception:
        return None
    import numpy as np
    from helios_glm53flash_b200 import synth
    T, H, D = T_FULL, HEADS, DIM
    dim = 3 * H * D
    cv = synth.conv_inputs(T, dim, seed=0)
    kd = synth.kda_gates(T, H, D, seed=0)

    def bits16(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).cuda()

    x, w = bits16(cv["x"]), bits16(cv["weight"])
    g, beta = torch.from_numpy(kd["g"]).cuda(), bits16(kd["beta"])
    conv_state = torch.zeros(1, dim, 4, dtype=torch.bfloat16, device="cuda")
    rec_state = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
    qkv = torch.empty(1, T, dim, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")

    def step():
        conv_state.zero_()
        rec_state.zero_()
        hk_ref.conv1d_update(x, conv_state, None, w, None, qkv, 1, dim, T, 4, 4, True, False)
        hk_ref.kda_recurrent(qkv, g, beta, rec_state, out, 1, T, H, H, D, D, 1, None, True, False)

    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / args.steps


def run_reference_arm(args, rank):
    """The reference has no CPU implementation of this path; what it has are its CUDA kernels, which compile for
    sm_100a as they are.  When that build (oracle/_ref) is present this arm times them on the GPU, every step the full
    workload; otherwise it times the CPU restatement, the full 32,768 tokens once per step for at most 3 steps, and
    prints the number of steps it really ran."""
    if rank != 0:
        return
    workload = "kda_prefill_32k: conv1d(K=4,SiLU) + gated delta rule, B=1, T=32768, H=32, d=128"
    ms = _reference_kernels_on_gpu(args)
    if ms is not None:
        value = T_FULL / (ms * 1e-3)
        line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16 in / fp32 state", "data": "synthetic",
                "config": {"workload": workload,
                           "note": "the reference's own per-token kernels (cuda_causal_conv1d_update + "
                                   "cuda_recurrent_gated_delta_rule, sm_86 sources compiled unchanged for sm_100a) on one GPU"},
                "cpu_baseline": {"value": value, "unit": "tok/s", "cores": 0, "kind": "reference",
                                 "sample": "full workload per step, reference CUDA kernels on the same GPU (the reference "
                                           "has no CPU path); rank 0 only"},
                "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return
    ran = max(1, min(args.steps, 3))
    cb = cpu_baseline(steps=ran, sample_t=T_FULL)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": ran, "warmup": 0, "ms_per_step": 1e3 * cb["seconds"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload,
                       "note": "reference kernels not built on this machine: CPU restatement (oracle), full workload per "
                               "step, best of the %d steps run" % ran},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)



# =====================================================================================================
# per-kernel cases (one entry point each, small enough for a profiler capture) and the reference's own
# kernels timed beside this library's on the same buffers
# =====================================================================================================
def _bits16(t, dtype):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t).view(np.int16)).view(dtype).cuda()


def build_kernel_case(name):
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
    if name in ("indexer_262k", "indexer_prefill_256", "indexer_prefill_1024x8192"):
        npools = 8192 if name.endswith("x8192") else 65536
        m = {"indexer_262k": 1, "indexer_prefill_256": 256}.get(name, 1024)
        ix = synth.indexer_inputs(npools, m, seed=7)
        qi, pk, w = _bits16(ix["q_idx"], torch.float16), _bits16(ix["pool_k"], torch.float16), _bits16(ix["w"], torch.float16)
        q_pos = torch.full((m,), 4 * npools - 1, dtype=torch.int32, device="cuda")
        sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")

        def fn():
            hk.indexer_score(qi, pk, w, q_pos, sc, m, npools)
        return fn, npools * 256 + m * npools * 2, True, "indexer scores, %d rows x %d pools, %.1f GFLOP" % (
            m, npools, m * npools * 32 * 128 * 2 / 1e9)
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
    if name in ("sparse_prefill_4096", "sparse_prefill_1024"):
        # the trunk's largest prefill stage: every row of a chunk attends its own 2,052 gathered rows of a 32,768-row
        # cache (32 MB: the gathers hit L2); bytes = gathered bytes, flops = 4 * 64 * 512 per (row, key)
        L, m = 32768, int(name.split("_")[-1])
        ck = torch.randn(L, 512, dtype=torch.float16, device="cuda")
        ql = torch.randn(m, 64, 512, dtype=torch.float16, device="cuda")
        pos = torch.arange(L - m, L, device="cuda").view(m, 1)
        raw = (torch.rand(m, 2052, device="cuda") * (pos + 1).float()).int().clamp_(max=L - 1)    # causal: rows <= position
        lo = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(m, 2052)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, m * 64)), dtype=torch.uint8, device="cuda")

        def fn():
            hk.mla_sparse_decode(ql, ck, raw, 2052, lo, m, n_split=ns, workspace=wsb)
        return fn, m * 2052 * 1024, False, "sparse MLA prefill, %d rows x 2052 gathered latents of 32768, %d split(s), %.1f GFLOP" % (
            m, ns, m * 2052 * 4 * 64 * 512 / 1e9)
    raise SystemExit("unknown case " + name)


KERNEL_CASES = ["kda_prefill_8k", "kda_prefill_32k", "kda_recurrent_512", "conv_8k", "conv_32k", "kda_decode", "mla_dense_b1",
         "mla_dense_b8", "mla_prefill_256", "indexer_262k", "indexer_prefill_256", "indexer_prefill_1024x8192", "topk_262k", "sparse_262k", "sparse_prefill_4096", "q_latent_4096", "o_absorb_4096",
         "transpose_cast_32k", "gate_32k", "gated_norm_32k", "cast_conv_32k", "kda_prefill_gated_32k", "transpose_cast_4k",
         "gate_4k", "gated_norm_4k", "cast_conv_4k"]




def run_kernel_cases(args):
    """`--kernel-case NAME` (or `all`): median device time of one entry point (CUDA events on the current stream, L2
    flushed by a 256 MB write between iterations unless the working set exceeds L2 by itself), one JSON line each"""
    import torch
    import helios_glm53flash_b200 as hk
    hk.load_library()
    names = KERNEL_CASES if args.kernel_case == "all" else [args.kernel_case]
    for name in names:
        fn, nbytes, flush, desc = build_kernel_case(name)
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
        for _ in range(max(args.warmup, 1)):
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
        print(json.dumps({"case": name + ("+graph" if args.graph else ""), "desc": desc, "us": ms * 1e3,
                          "algorithmic_GBps": nbytes / (ms * 1e-3) / 1e9, "device_status": hk.read_device_status()}), flush=True)
        del fn, buf
        torch.cuda.empty_cache()


def _timed_us(torch, fn, iters, flush):
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


def reference_kernel_cases(torch, hk, ref, synth):
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




def run_reference_kernel_cases(args):
    """`--case reference_kernels`: the reference's own CUDA kernels (oracle/_ref/libhelios_ref.so, its sources compiled
    for sm_100a) and this library's on the same buffers: median device time of each (2 warm-ups, 256 MB L2 flush before
    every timed call), one JSON line per case; `--kernel-case NAME` selects one"""
    import torch
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import synth
    import hk_ref as ref
    if not ref.available():
        print(json.dumps({"case": "reference_kernels", "unavailable": "oracle/_ref/libhelios_ref.so is not built (make -C oracle ref)"}))
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = reference_kernel_cases(torch, hk, ref, synth)
    for name in ([args.kernel_case] if args.kernel_case else list(table)):
        build, desc, iters = table[name]
        ours, theirs = build()
        t_ref = _timed_us(torch, theirs, iters, flush)
        t_ours = _timed_us(torch, ours, iters, flush)
        print(json.dumps({"case": name, "desc": desc, "reference_kernel_us": t_ref, "this_library_us": t_ours,
                          "speedup": t_ref / t_ours, "iters": iters, "device_status": hk.read_device_status()}), flush=True)
        del ours, theirs
        torch.cuda.empty_cache()


def run_trunk_case(args):
    """The whole hybrid trunk's attention path (34 KDA + 11 MLA layers, shapes of the benchmark configurations) on a
    synthetic sequence: prefill in 4,096-token chunks, then decode steps; device-timed.  Reports prefill tok/s, decode
    us per token and the share of every stage (CUDA events around each call, summed over layers and chunks)."""
    import torch
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200.trunk import TrunkAttention
    hk.load_library()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    ctx, B, chunk, steps = args.trunk_ctx, args.trunk_batch, 4096, args.trunk_decode
    tr = TrunkAttention(n_kda=34, n_mla=11, heads=HEADS, batch=B, max_ctx=ctx + steps + 64, max_chunk=chunk, seed=0, fused=True)
    tr.run_chunk(0, chunk)                                  # warm-up chunk (its rows are overwritten by the timed run)
    torch.cuda.synchronize()
    for st in tr.rec_state + tr.conv_state:
        st.zero_()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    tr.prefill(ctx, chunk, timed=True)
    e1.record()
    shares = tr.stage_shares()
    for s in range(steps):
        tr.run_chunk(ctx + s, 1)
    e2.record()
    torch.cuda.synchronize()
    status = hk.read_device_status()
    pre_ms, dec_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
    tot = sum(shares.values())
    # The same decode step as ONE replayed CUDA graph (all launches of the 45 layers at one position; a replay repeats
    # that position, so the work per replay is that of one token at this context): what an engine that captures its
    # decode step sees, without the host's launch cost.
    graph_us = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            tr.run_chunk(ctx + steps, 1)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                tr.run_chunk(ctx + steps, 1)
            side.synchronize()
            for _ in range(3):
                graph.replay()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(max(steps, 8)):
                graph.replay()
            g1.record()
            side.synchronize()
            graph_us = 1e3 * g0.elapsed_time(g1) / max(steps, 8)
        status = status or hk.read_device_status()
    except Exception as exc:   # a capture that fails must not cost the prefill figures
        graph_us = "capture failed: %s" % str(exc)[:200]
    line = {"metric": "trunk_attention_prefill_tokens_per_s", "value": B * ctx / (pre_ms * 1e-3), "unit": "tok/s", "n_gpus": 1,
            "higher_is_better": True, "data": "synthetic", "dtype": "bf16 / fp16 in, fp32 accumulate + state",
            "config": {"workload": "34 KDA + 11 MLA attention layers in the engine's call order, %d sequence(s) x %d tokens, "
                                   "prefill in %d-token chunks, then %d decode steps" % (B, ctx, chunk, steps)},
            "prefill_ms": pre_ms, "prefill_ms_per_chunk": pre_ms / (ctx / chunk),
            "decode_us_per_token_host_launched": 1e3 * dec_ms / max(steps, 1),
            "decode_us_per_token_graph_replay": graph_us,
            "stage_share_of_prefill": {k: v / tot for k, v in sorted(shares.items(), key=lambda kv: -kv[1])},
            "stage_ms_total": {k: v for k, v in sorted(shares.items(), key=lambda kv: -kv[1])},
            "device_status": status}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=T_FULL, help="sequence length (default: the benchmark's 32768)")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / MLA side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--case", default="kda_prefill", choices=["kda_prefill", "trunk", "reference_kernels"],
                    help="kda_prefill: the headline line (default).  trunk: the 34 KDA + 11 MLA attention stack in the engine's "
                         "call order, prefill in 4,096-token chunks then decode (one GPU; its own JSON line).  reference_kernels: "
                         "the reference's own kernels timed beside this library's, one JSON line per kernel")
    ap.add_argument("--kernel-case", default=None,
                    help="time ONE entry point on a small case (median of --iters) and print its JSON line; 'all' runs every "
                         "case.  With --case reference_kernels: the one comparison to run")
    ap.add_argument("--iters", type=int, default=20, help="timed calls of --kernel-case")
    ap.add_argument("--graph", action="store_true", help="--kernel-case: time the replay of a CUDA graph of the call")
    ap.add_argument("--trunk-ctx", type=int, default=32768, help="tokens prefetched by --case trunk (the full configuration is 262144)")
    ap.add_argument("--trunk-batch", type=int, default=1, help="sequences of --case trunk (the batched configuration is 8 x 32768)")
    ap.add_argument("--trunk-decode", type=int, default=64, help="decode steps after the prefill of --case trunk")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.case == "trunk":
        if rank == 0:
            run_trunk_case(args)
        return
    if args.case == "reference_kernels":
        if rank == 0:
            run_reference_kernel_cases(args)
        return
    if args.kernel_case:
        if rank == 0:
            run_kernel_cases(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import synth
    hk.load_library()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL may print a version banner on stdout when the communicator comes up; stdout carries exactly
        # one JSON line, so the banner goes to stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    T, H, D = args.tokens, HEADS, DIM
    dim = 3 * H * D
    steps, warmup = args.steps, max(args.warmup, 3)
    # ---- inputs: pinned host copies (for the end-to-end leg) and device-resident copies ----
    cv = synth.conv_inputs(T, dim, seed=rank)
    kd = synth.kda_gates(T, H, D, seed=rank)

    def pin_bits(a, dtype):
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dtype)
        return t.pin_memory()

    h_x = pin_bits(cv["x"], torch.bfloat16)
    h_w = pin_bits(cv["weight"], torch.bfloat16)
    h_g = torch.from_numpy(kd["g"]).pin_memory()
    h_beta = pin_bits(kd["beta"], torch.bfloat16)
    del cv, kd
    d_x, d_w, d_g, d_beta = h_x.cuda(), h_w.cuda(), h_g.cuda(), h_beta.cuda()
    conv_state = torch.zeros(1, dim, 4, dtype=torch.bfloat16, device="cuda")
    rec_state = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
    qkv = torch.empty(1, T, dim, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    h_out = torch.empty(1, T, H, D, dtype=torch.bfloat16).pin_memory()
    ws = torch.empty(hk.kda_chunked_workspace_bytes(1, T, H), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()

    def step(x=d_x, g=d_g, beta=d_beta, ev=None):
        conv_state.zero_()
        rec_state.zero_()
        if ev:
            ev[0].record(stream)
        hk.cuda_causal_conv1d_update(x, conv_state, None, d_w, None, qkv, 1, dim, T, 4, 4, True, False)
        if ev:
            ev[1].record(stream)
        path = hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, rec_state, out, 1, T, H, H, D, D, 1, None, True, False,
                                                  workspace=ws)
        if ev:
            ev[2].record(stream)
        return path

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None   # started early: nvidia-smi needs a moment to come up
    for _ in range(warmup):
        path = step()
    barrier()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin = time.time()
    e0.record(stream)
    for i in range(steps):
        step(ev=evs[i])
    e1.record(stream)
    barrier()
    t_end = time.time()
    ms_total = e0.elapsed_time(e1)
    clocks = None
    if sampler:
        clocks = sampler.summary(t_begin, t_end)
        if clocks.get("samples", 0) < 3 or "no sample" in clocks.get("note", ""):
            # the timed region was shorter than a few sampling periods: the same loop runs on, untimed, for 0.4 s
            t_c0 = time.time()
            while time.time() - t_c0 < 0.4:
                for _ in range(10):
                    step()
                torch.cuda.synchronize()
            clocks = sampler.summary(t_c0 + 0.05, time.time())
            clocks["note"] = "timed region of %.0f ms too short to sample: the same step loop continued untimed for 0.4 s, samples from there" % ms_total
        sampler.stop()
    conv_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / steps
    kda_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / steps
    assert hk.read_device_status() == 0, "a bounded device wait expired"

    # ---- end to end through the host-facing call: pinned host inputs in, result back to the host ----
    # The sequence is cut into segments; a copy-in stream, the compute stream and a copy-out stream form
    # a pipeline (the conv window and the recurrent state carry from one segment to the next, so the
    # result is the one-launch result).  Every step moves all inputs and the whole output over PCIe.
    e2e_steps = max(2, min(steps, 5))
    hg2, hb2 = torch.empty_like(d_g), torch.empty_like(d_beta)
    seg = 4096 if T % 4096 == 0 and T > 4096 else T
    n_seg = T // seg
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_done = [torch.cuda.Event() for _ in range(n_seg)]
    comp_done = [torch.cuda.Event() for _ in range(n_seg)]
    g3, b3 = hg2.view(1, T, H, D), hb2.view(1, T, H)
    hg3, hb3 = h_g.view(1, T, H, D), h_beta.view(1, T, H)
    # the conv input is channel-major [dim][tokens]: the host hands over one [dim][segment] block per segment
    hx_seg = [h_x.view(dim, T)[:, i * seg:(i + 1) * seg].contiguous().pin_memory() for i in range(n_seg)]
    x_seg = [torch.empty(1, dim, seg, dtype=torch.bfloat16, device="cuda") for _ in range(n_seg)]

    def e2e_step(first):
        conv_state.zero_()
        rec_state.zero_()
        for i in range(n_seg):
            sl = slice(i * seg, (i + 1) * seg)
            with torch.cuda.stream(s_in):
                if not first:
                    s_in.wait_event(comp_done[i])            # the previous step has consumed this segment
                x_seg[i].view(dim, seg).copy_(hx_seg[i], non_blocking=True)
                g3[:, sl].copy_(hg3[:, sl], non_blocking=True)
                b3[:, sl].copy_(hb3[:, sl], non_blocking=True)
                in_done[i].record(s_in)
            stream.wait_event(in_done[i])
            hk.cuda_causal_conv1d_update(x_seg[i], conv_state, None, d_w, None, qkv[:, sl], 1, dim, seg, 4, 4, True, False)
            hk.cuda_recurrent_gated_delta_rule(qkv[:, sl], g3[:, sl], b3[:, sl], rec_state, out[:, sl], 1, seg, H, H, D, D,
                                               1, None, True, False, workspace=ws)
            comp_done[i].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[i])
                h_out[:, sl].copy_(out[:, sl], non_blocking=True)
        stream.wait_stream(s_out)

    e2e_step(True)                                            # untimed: also checks the pipelined result
    torch.cuda.synchronize()
    seg_out = h_out.clone()
    step()
    torch.cuda.synchronize()
    e2e_diff = (seg_out.cuda().float() - out.float()).abs()
    e2e_matches = {"max_abs_diff": float(e2e_diff.max()), "mismatching_fraction": float((e2e_diff > 0).float().mean()),
                   "first_bad_token": int((e2e_diff.view(T, -1).amax(dim=1) > 0).float().argmax())}
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(e2e_steps):
        e2e_step(False)
    e3.record(stream)
    barrier()
    e2e_ms = e2.elapsed_time(e3) / e2e_steps
    h2d = h_x.numel() * 2 + h_g.numel() * 4 + h_beta.numel() * 2
    d2h = h_out.numel() * 2

    t = torch.tensor([ms_total, e2e_ms, conv_ms, kda_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, conv_ms, kda_ms = [float(v) for v in t.cpu()]
    ms_step = ms_total / steps

    multi = None
    if world > 1:
        multi = multi_gpu_measurements(hk, synth, torch, dist, np, rank, local_rank, world, kda_ms)
    extras = {}
    if rank == 0 and not args.no_extras:
        extras = side_measurements(hk, synth, torch, np, local_rank)

    if rank == 0:
        peaks, peak_kind = _peaks()
        # dominant kernel pair = the chunked KDA prefill (prep + scan launches): algorithmic bytes per
        # token-head 1538 B (q,k,v bf16 + g f32 + beta + out bf16) plus the fp32 state in and out
        alg_bytes = T * H * 1538 + 2 * H * D * D * 4
        achieved = alg_bytes / (kda_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * T / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 in / fp16 tensor-core operands / fp32 accumulate+state", "data": "synthetic",
            "config": {"workload": "kda_prefill_32k: conv1d(K=4,SiLU) over 12288 channels + chunked gated delta rule, "
                                   "B=1 per GPU, T=%d, H=32, d_k=d_v=128, chunk 64, zero initial state" % T,
                       "l2": "inputs (%.0f MB) exceed L2; no flush between steps" % ((h2d) / 1e6),
                       "parallelism": "independent sequence per GPU (no data-path collective)", "path": path},
            "kernel_ms": {"conv1d": conv_ms, "kda_chunked_prefill": kda_ms},
            "roofline": {"bound": "hbm", "kernel": "kda_fused_kernel (chunk preparation + chain scan in one persistent launch)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         # dram__bytes_read + dram__bytes_write of the fused kernel from the ncu capture of the T = 8,192
                         # case (574 MB), scaled by the chunk count: traffic is linear in T
                         "traffic": 574.8e6 * (T / 8192.0), "traffic_source": "ncu dram bytes of kda_fused_kernel at T = 8192, scaled by T / 8192",
                         "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": alg_bytes,
                         "tensor_tflops_dense_chunk_math": (T // 64) * H * 11.71e6 / (kda_ms * 1e-3) / 1e12},
            "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "pipeline": "%d segments of %d tokens on copy-in / compute / copy-out streams" % (n_seg, seg),
                    "equals_one_launch_result": e2e_matches},
            "gpu_launches": 2 * steps,
            "clocks": clocks,
            "extras": extras,
        }
        if multi is not None:
            line["multi_gpu"] = multi
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(steps=3)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def multi_gpu_measurements(hk, synth, torch, dist, np, rank, local_rank, world, kda_ms_32_heads):
    """The partitions of the path across the GPUs of one node, device-timed, max over ranks:
      * split-KV decode over a 262,144-token latent cache (batch 1 and batch 8): every rank attends its slice, the
        partials are combined by peer loads over NVLink; against the same decode on one GPU (rank 0's own time);
      * the sparse form of it for one sequence (indexer scores of the local pools, selection exchanged between the
        ranks, attention over the selected rows of the local slice), against the one-GPU chain;
      * KDA prefill sharded by heads (32 / N heads per GPU, same 32,768 tokens): strong scaling of the headline step;
      * MLA dense decode of 8 sequences x 32,768 tokens sharded by sequences (8 / N per GPU); the tensor-core kernel
        keeps all 64 heads of a sequence on one GPU (heads are its accumulator lanes);
      * SM clocks of every rank, sampled on its own GPU while its split-KV loop runs."""
    from helios_glm53flash_b200 import splitkv
    res = {"n_gpus": world}
    H, D, T = HEADS, DIM, T_FULL

    def max_over_ranks(v):
        t = torch.tensor([float(v)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def graph_time(fn, iters=30, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return g, a.elapsed_time(b) / iters

    # ---- split-KV decode at 262,144 tokens of context ----
    L, scale = 262144, 512 ** -0.5
    sampler = ClockSampler(local_rank)
    t_clk0 = time.time()
    for m in (1, 8):
        gen = torch.Generator(device="cuda").manual_seed(4321 + m)            # same cache and queries on every rank
        q = torch.randn(m, 64, 512, generator=gen, device="cuda", dtype=torch.float32).half()
        b0, e0 = splitkv.shard_tokens(L, rank, world)
        # this rank's slice of every sequence, concatenated (a rank never holds the other ranks' rows)
        shard = torch.randn(m * (e0 - b0), 512, device="cuda", dtype=torch.float16)
        shard_base = torch.arange(m, device="cuda", dtype=torch.int64) * (e0 - b0)
        out = torch.zeros(m, 64, 512, dtype=torch.float16, device="cuda")
        dec = splitkv.SplitKVDecoder(m, max_wait_ms=2000)
        g, ms = graph_time(lambda: dec.step(q, shard, e0 - b0, out, scale, kv_base=shard_base))
        ms = max_over_ranks(ms)
        status = hk.read_device_status()
        # the same decode on one GPU (the whole cache of every sequence on this rank), rank 0's own time
        ms1 = 0.0
        if rank == 0:
            full = torch.randn(m * L, 512, device="cuda", dtype=torch.float16)
            base1 = torch.arange(m, device="cuda", dtype=torch.int64) * L
            len1 = torch.full((m,), L, dtype=torch.int32, device="cuda")
            ns = hk.mla_auto_splits(m, L)
            ws1 = torch.empty(max(256, hk.mla_partial_bytes(ns, m * 64)), dtype=torch.uint8, device="cuda")
            ref = torch.empty_like(out)
            fn1 = lambda: hk.mla_dense_prefill(q, full, ref, m, 0, scale=scale, kv_base=base1, kv_len=len1, n_split=ns,
                                               workspace=ws1, n_keys_hint=L)
            for _ in range(3):
                fn1()
            torch.cuda.synchronize()
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                fn1()
            g1.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(30):
                g1.replay()
            b.record()
            torch.cuda.synchronize()
            ms1 = a.elapsed_time(b) / 30
            del full, g1
        ms1 = max_over_ranks(ms1)
        # the library baseline for the exchange: the same local partial, then ncclAllGather of the partial sets and
        # the local combine over the gathered sets (host-launched: a collective cannot sit in this graph replay loop
        # together with the bounded waits; so the figure includes NCCL's launch cost, as an engine would see it)
        rows_ = m * 64
        pad_ = ((rows_ * 4 + 255) // 256) * 256
        set_bytes = 2 * pad_ + rows_ * 512 * 4
        mine = torch.empty(set_bytes, dtype=torch.uint8, device="cuda")
        allsets = torch.empty(world * set_bytes, dtype=torch.uint8, device="cuda")
        pm = mine[:rows_ * 4].view(torch.float32)
        plv = mine[pad_:pad_ + rows_ * 4].view(torch.float32)
        pa = mine[2 * pad_:].view(torch.float32)
        base_all = allsets.data_ptr()
        tm = torch.tensor([base_all + r_ * set_bytes for r_ in range(world)], dtype=torch.int64, device="cuda")
        tl = tm + pad_
        ta = tm + 2 * pad_
        lens_ = torch.full((m,), e0 - b0, dtype=torch.int32, device="cuda")
        ns_ = hk.mla_auto_splits(m, max(1, e0 - b0))
        wsn = torch.empty(max(256, hk.mla_partial_bytes(ns_, rows_)), dtype=torch.uint8, device="cuda")
        out_n = torch.zeros_like(out)

        def nccl_step():
            hk.mla_dense_partial_ws(q, shard, shard_base, lens_, 0, pm, plv, pa, m, e0 - b0, scale=scale, n_split=ns_, workspace=wsn)
            dist.all_gather_into_tensor(allsets, mine)
            hk.lse_combine_ptrs(tm, tl, ta, world, rows_, out_n)
        for _ in range(5):
            nccl_step()
        torch.cuda.synchronize()
        dist.barrier()
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for _ in range(30):
            nccl_step()
        b_.record()
        torch.cuda.synchronize()
        ms_nccl = max_over_ranks(a_.elapsed_time(b_) / 30)
        agree = float((out_n.float() - out.float()).abs().max())
        res["splitkv_decode_262k_b%d" % m] = {
            "us_per_step": ms * 1e3, "one_gpu_us_per_step": ms1 * 1e3, "speedup_vs_one_gpu": ms1 / ms,
            "efficiency": ms1 / ms / world, "aggregate_hbm_gbs": m * L * 1024 / (ms * 1e-3) / 1e9,
            "exchange": dec.form, "device_status": status,
            "nccl_allgather_baseline_us_per_step": ms_nccl * 1e3, "nccl_baseline_max_abs_diff": agree}
        del mine, allsets, wsn
        del g
        dec.close()
        del shard
        torch.cuda.empty_cache()
    # ---- SPARSE split-KV decode of one 262,144-token sequence: pools and cache rows split over the ranks, selection
    # exchanged (512 candidates per rank), attention over the selected rows of the local slice, partials combined ----
    if world <= 8:
        gen = torch.Generator(device="cuda").manual_seed(99)
        P = L // 4
        q = torch.randn(1, 64, 512, generator=gen, device="cuda", dtype=torch.float32).half()
        q_idx = torch.randn(1, 32, 128, generator=gen, device="cuda", dtype=torch.float32).half()
        w_idx = torch.rand(1, 32, generator=gen, device="cuda", dtype=torch.float32).half()
        q_pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
        prange, rrange = splitkv.shard_pools(L, rank, world)
        pool_l = (torch.randn(prange[1] - prange[0], 128, device="cuda") * 0.5).half()
        ckv_l = torch.randn(rrange[1] - rrange[0], 512, device="cuda", dtype=torch.float16)
        out = torch.zeros(1, 64, 512, dtype=torch.float16, device="cuda")
        dec = splitkv.SplitKVDecoder(1, max_wait_ms=2000, sparse=True)
        g, ms = graph_time(lambda: dec.step_sparse(q, q_idx, w_idx, q_pos, pool_l, prange, ckv_l, rrange, out, scale))
        ms = max_over_ranks(ms)
        status = hk.read_device_status()
        ms1 = 0.0
        if rank == 0:
            pool_f = (torch.randn(P, 128, device="cuda") * 0.5).half()
            ckv_f = torch.randn(L, 512, device="cuda", dtype=torch.float16)
            sc = torch.empty(1, P, dtype=torch.float16, device="cuda")
            topk = torch.empty(1, 512, dtype=torch.int32, device="cuda")
            raw = torch.empty(1, 2052, dtype=torch.int32, device="cuda")
            ref = torch.empty_like(out)
            ns = hk.mla_auto_splits(1, 2052)
            ws1 = torch.empty(max(256, hk.mla_partial_bytes(ns, 64)), dtype=torch.uint8, device="cuda")

            def chain():
                hk.indexer_score(q_idx, pool_f, w_idx, q_pos, sc, 1, P)
                hk.dsa_topk(sc, P, topk, 1, P, 512, 512)
                hk.pool_expand_row(topk, q_pos, raw, 1)
                hk.mla_sparse_decode(q, ckv_f, raw, 2052, ref, 1, scale=scale, n_split=ns, workspace=ws1)
            for _ in range(3):
                chain()
            torch.cuda.synchronize()
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                chain()
            g1.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(30):
                g1.replay()
            b.record()
            torch.cuda.synchronize()
            ms1 = a.elapsed_time(b) / 30
            del pool_f, ckv_f, g1
        ms1 = max_over_ranks(ms1)
        res["splitkv_sparse_decode_262k_b1"] = {
            "us_per_step": ms * 1e3, "one_gpu_us_per_step": ms1 * 1e3, "speedup_vs_one_gpu": ms1 / ms,
            "note": "latency-bound on one GPU already (16.8 MB of pooled keys + 2.1 MB of selected rows per step): the split "
                    "buys cache capacity per GPU, not time", "device_status": status}
        del g
        dec.close()
        del pool_l, ckv_l
        torch.cuda.empty_cache()
    t_clk1 = time.time()
    sampler.stop()
    clk = sampler.summary(t_clk0, t_clk1)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons")})
    res["per_rank_clocks_during_splitkv"] = gathered

    # ---- KDA prefill sharded by heads: 32 / N heads on every GPU, the same 32,768 tokens ----
    if H % world == 0:
        Hl = H // world
        kd = synth.kda_gates(T, Hl, D, seed=rank)
        g_l, beta_l = torch.from_numpy(kd["g"]).cuda(), torch.from_numpy(kd["beta"].view(np.int16)).view(torch.bfloat16).cuda()
        qkv_l = torch.randn(1, T, 3 * Hl * D, device="cuda").to(torch.bfloat16)
        st_l = torch.zeros(1, 1, Hl, D, D, dtype=torch.float32, device="cuda")
        out_l = torch.empty(1, T, Hl, D, dtype=torch.bfloat16, device="cuda")
        ws_l = torch.empty(hk.kda_chunked_workspace_bytes(1, T, Hl), dtype=torch.uint8, device="cuda")

        def kda_step():
            st_l.zero_()
            hk.cuda_recurrent_gated_delta_rule(qkv_l, g_l, beta_l, st_l, out_l, 1, T, Hl, Hl, D, D, 1, None, True, False,
                                               workspace=ws_l)
        for _ in range(3):
            kda_step()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            kda_step()
        b.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(a.elapsed_time(b) / 10)
        res["kda_prefill_32k_head_sharded"] = {
            "heads_per_gpu": Hl, "ms": ms, "tokens_per_s": T / (ms * 1e-3), "ms_32_heads_on_one_gpu": kda_ms_32_heads,
            "speedup": kda_ms_32_heads / ms, "efficiency": kda_ms_32_heads / ms / world,
            "note": "one chain per head: with few heads per GPU the step is bound by the 512-chunk chain, not by the SMs"}
        del qkv_l, g_l, out_l, ws_l
        torch.cuda.empty_cache()

    # ---- MLA dense decode, 8 sequences x 32,768 tokens, sharded by sequences: two alternating sets of caches
    #      (together larger than L2), a timed region = 10 replays of a graph that decodes both ----
    B, L2 = 8, 32768
    if B % world == 0:
        Bl = B // world
        n_sets = 2 if Bl * L2 * 1024 * 2 > (160 << 20) else 4
        cks = [torch.randn(Bl * L2, 512, dtype=torch.float16, device="cuda") for _ in range(n_sets)]
        qd = torch.randn(Bl, 64, 512, dtype=torch.float16, device="cuda")
        base = torch.arange(Bl, device="cuda", dtype=torch.int64) * L2
        lens = torch.full((Bl,), L2, dtype=torch.int32, device="cuda")
        lo = torch.empty(Bl, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(Bl, L2)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, Bl * 64)), dtype=torch.uint8, device="cuda")

        def mla_step():
            for ck in cks:
                hk.mla_dense_prefill(qd, ck, lo, Bl, 0, scale=scale, kv_base=base, kv_len=lens, n_split=ns, workspace=wsb,
                                     n_keys_hint=L2)
        for _ in range(3):
            mla_step()
        torch.cuda.synchronize()
        gm = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gm):
            mla_step()
        ts = []
        for _ in range(5):
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                gm.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / (10 * n_sets))
        ms = max_over_ranks(sorted(ts)[len(ts) // 2])
        res["mla_dense_decode_32k_b8_sequence_sharded"] = {
            "sequences_per_gpu": Bl, "us_per_layer": ms * 1e3, "aggregate_hbm_gbs": B * L2 * 1024 / (ms * 1e-3) / 1e9,
            "l2": "%d alternating cache sets of %d MB per GPU, 10 graph replays per timed region" % (n_sets, Bl * L2 * 1024 >> 20)}
    return res


FIGURE_CLOCKS = {}      # label -> SM clock summary sampled while that figure's launch chain ran for 0.3 s


def _time_loop(torch, fns, iters=10, warm=2, flush=None, sustain_ms=2.0, label=None, gpu_index=0):
    """median device time, in ms, of ONE pass over the callables of `fns` run back to back.  The chain is
    captured in a CUDA graph after the warm-up and replays are timed, so host launch latency is not in the
    figure; a timed region holds as many replays as fill about `sustain_ms` (a decode loop keeps the GPU
    busy: a single short launch after an idle gap would be timed at idle clocks)."""
    for _ in range(warm):
        for f in fns:
            f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()

    def once(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    reps = max(1, min(200, int(sustain_ms / max(once(1), 1e-3) + 0.999)))
    ts = sorted(once(reps) for _ in range(iters))
    if label is not None:
        # the clock record of this figure: the same chain replayed for 0.3 s with the 10 ms sampler running
        sampler = ClockSampler(gpu_index)
        t0 = time.time()
        while time.time() - t0 < 0.3:
            for _ in range(20):
                graph.replay()
            torch.cuda.synchronize()
        t1 = time.time()
        sampler.stop()
        FIGURE_CLOCKS[label] = sampler.summary(t0 + 0.05, t1)
    return ts[len(ts) // 2]


def side_measurements(hk, synth, torch, np, gpu_index=0):
    """Decode-side figures.  Each is the median device time of a chain of launches over DISTINCT
    per-layer buffers (34 KDA layers, 11 MLA layers, as in the hybrid trunk), divided by the number of
    layers; L2 is flushed (256 MB write) before every timed region unless the buffers exceed L2 on their
    own.  A timed region repeats the chain until it lasts about 2 ms (see _time_loop)."""
    from gpu_util import dev, dev_bf16, dev_f16
    res = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    H, D = HEADS, DIM
    # ---- KDA decode step: 34 layers, each with its own 2 MiB fp32 state and its own conv window; the step includes
    #      the short convolution: one fused launch per layer, and the reference's two-launch sequence beside it ----
    n_kda = 34
    dimc = 3 * H * D
    kd = synth.kda_inputs(1, H, D, seed=5)
    g, b = dev(kd["g"]), dev_bf16(kd["beta"])
    xdec = torch.randn(1, dimc, device="cuda").to(torch.bfloat16)
    wdec = (0.1 * torch.randn(dimc, 4, device="cuda")).to(torch.bfloat16)
    sts = [torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda") for _ in range(n_kda)]
    css = [torch.zeros(1, dimc, 4, dtype=torch.bfloat16, device="cuda") for _ in range(n_kda)]
    qkv1 = torch.empty(1, 1, dimc, dtype=torch.bfloat16, device="cuda")
    o = torch.empty(1, 1, H, D, dtype=torch.bfloat16, device="cuda")
    fns = [(lambda st=st, cs=cs: hk.kda_decode_step(xdec, cs, wdec, None, g, b, st, o, 1, H)) for st, cs in zip(sts, css)]
    ms = _time_loop(torch, fns, flush=flush, label="kda_decode", gpu_index=gpu_index) / n_kda
    res["kda_decode_us_per_layer"] = ms * 1e3
    res["kda_decode_hbm_gbs"] = (2 * H * D * D * 4 + H * 1538) / (ms * 1e-3) / 1e9

    def two_launch(st, cs):
        hk.cuda_causal_conv1d_update(xdec.view(1, dimc, 1), cs, None, wdec, None, qkv1, 1, dimc, 1, 4, 4, True, False)
        hk.cuda_recurrent_gated_delta_rule(qkv1, g, b, st, o, 1, 1, H, H, D, D, 1, None, True, False)
    fns = [(lambda st=st, cs=cs: two_launch(st, cs)) for st, cs in zip(sts, css)]
    res["kda_decode_two_launch_us_per_layer"] = 1e3 * _time_loop(torch, fns, flush=flush) / n_kda
    # the whole layer of a decoded token, from the projections' fp32 row to the gated, normalised fp16 activations: one
    # launch (hk_kda_decode_layer), and the reference's five-call sequence (cast, gate, conv, recurrence, gated norm)
    rawg = synth.kda_raw_gates(1, H, D, seed=4)
    f1, b1 = dev(rawg["f"]), dev(rawg["b"])
    dtb1, alog1, lb1 = dev(rawg["dt_bias"]), dev(rawg["a_log"]), rawg["lower_bound"]
    x32d = torch.randn(1, dimc, device="cuda")
    nw1 = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    go1 = torch.randn(H, D, device="cuda")
    y1 = torch.empty(H, D, dtype=torch.float16, device="cuda")
    o1 = torch.empty(1, H, D, dtype=torch.bfloat16, device="cuda")
    g1, bt1 = torch.empty(1, H, D, device="cuda"), torch.empty(1, H, dtype=torch.bfloat16, device="cuda")
    x16d = torch.empty(dimc, 1, dtype=torch.bfloat16, device="cuda")
    fns = [(lambda st=st, cs=cs: hk.kda_decode_layer(x32d, cs, wdec, None, f1, b1, dtb1, alog1, lb1, st, o1, nw1, go1, y1, 1, H))
           for st, cs in zip(sts, css)]
    res["kda_decode_layer_one_launch_us_per_layer"] = 1e3 * _time_loop(torch, fns, flush=flush, label="kda_decode_layer",
                                                                       gpu_index=gpu_index) / n_kda

    def five_calls(st, cs):
        hk.kda_transpose_cast(x16d, x32d, 1, dimc)
        hk.kda_gate(b1, f1, dtb1, alog1, lb1, bt1, g1, 1, H, D)
        hk.cuda_causal_conv1d_update(x16d.view(1, dimc, 1), cs, None, wdec, None, qkv1, 1, dimc, 1, 4, 4, True, False)
        hk.cuda_recurrent_gated_delta_rule(qkv1, g1, bt1, st, o, 1, 1, H, H, D, D, 1, None, True, False)
        hk.gated_rms_norm(o, nw1, y1, go1, H, D, 1e-6, gate_act=1)
    fns = [(lambda st=st, cs=cs: five_calls(st, cs)) for st, cs in zip(sts, css)]
    res["kda_decode_layer_five_call_sequence_us_per_layer"] = 1e3 * _time_loop(torch, fns, flush=flush) / n_kda
    del sts, css
    # ---- dense MLA decode over 32K latent caches: 11 layers (B=1), 2 alternating layers (B=8) ----
    L = 32768
    for B, n_layers in ((1, 11), (8, 2)):
        cks = [torch.randn(B * L, 512, dtype=torch.float16, device="cuda") for _ in range(n_layers)]
        qd = torch.randn(B, 64, 512, dtype=torch.float16, device="cuda")
        base = dev((np.arange(B) * L).astype(np.int64))
        lens = dev(np.full(B, L, dtype=np.int32))
        lo = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(B, L)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, B * 64)), dtype=torch.uint8, device="cuda")
        fns = [(lambda ck=ck: hk.mla_dense_prefill(qd, ck, lo, B, 0, scale=512 ** -0.5, kv_base=base, kv_len=lens,
                                                   n_split=ns, workspace=wsb, n_keys_hint=L)) for ck in cks]
        ms = _time_loop(torch, fns, flush=flush if B * L * 1024 * n_layers < (200 << 20) else None,
                        label="mla_dense_decode_32k_b%d" % B, gpu_index=gpu_index) / n_layers
        res["mla_dense_decode_32k_b%d_us_per_layer" % B] = ms * 1e3
        res["mla_dense_decode_32k_b%d_hbm_gbs" % B] = B * L * 1024 / (ms * 1e-3) / 1e9
        res["mla_dense_decode_32k_b%d_splits" % B] = ns
        del cks
    # ---- indexer -> top-512 -> expand -> sparse MLA at 262,144 tokens of context, 11 layers ----
    npools, L, n_mla = 65536, 262144, 11
    ix = synth.indexer_inputs(npools, 1, seed=7)
    qi, w = dev_f16(ix["q_idx"]), dev_f16(ix["w"])
    pks = [torch.randn(npools, 128, dtype=torch.float16, device="cuda") for _ in range(n_mla)]
    ckvs = [torch.randn(L, 512, dtype=torch.float16, device="cuda") for _ in range(n_mla)]
    q_pos = dev(np.array([L - 1], dtype=np.int32))
    sc = torch.empty(1, npools, dtype=torch.float16, device="cuda")
    idx = torch.empty(1, 512, dtype=torch.int32, device="cuda")
    raw = torch.empty(1, 2052, dtype=torch.int32, device="cuda")
    ql = torch.randn(1, 64, 512, dtype=torch.float16, device="cuda")
    lo = torch.empty(1, 64, 512, dtype=torch.float16, device="cuda")
    ns = hk.mla_auto_splits(1, 2052)
    wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, 64)), dtype=torch.uint8, device="cuda")
    f_score = [(lambda pk=pk: hk.indexer_score(qi, pk, w, q_pos, sc, 1, npools)) for pk in pks]
    ms = _time_loop(torch, f_score, flush=flush, label="indexer_score_262k", gpu_index=gpu_index) / n_mla
    res["indexer_score_262k_us_per_layer"] = ms * 1e3
    res["indexer_score_262k_hbm_gbs"] = npools * 256 / (ms * 1e-3) / 1e9
    f_topk = [lambda: hk.dsa_topk(sc, npools, idx, 1, npools, 512, 512)] * n_mla
    res["topk512_262k_us_per_layer"] = 1e3 * _time_loop(torch, f_topk, flush=flush, label="topk512_262k", gpu_index=gpu_index) / n_mla
    hk.pool_expand_row(idx, q_pos, raw, 1)
    f_sparse = [(lambda ck=ck: hk.mla_sparse_decode(ql, ck, raw, 2052, lo, 1, n_split=ns, workspace=wsb)) for ck in ckvs]
    ms = _time_loop(torch, f_sparse, flush=flush, label="mla_sparse_decode_262k", gpu_index=gpu_index) / n_mla
    res["mla_sparse_decode_262k_us_per_layer"] = ms * 1e3
    res["mla_sparse_decode_262k_hbm_gbs"] = 2052 * 1024 / (ms * 1e-3) / 1e9

    def chain(pk, ck):
        hk.indexer_score(qi, pk, w, q_pos, sc, 1, npools)
        hk.dsa_topk(sc, npools, idx, 1, npools, 512, 512)
        hk.pool_expand_row(idx, q_pos, raw, 1)
        hk.mla_sparse_decode(ql, ck, raw, 2052, lo, 1, n_split=ns, workspace=wsb)
    f_chain = [(lambda pk=pk, ck=ck: chain(pk, ck)) for pk, ck in zip(pks, ckvs)]
    res["dsa_sparse_mla_decode_262k_us_per_layer"] = 1e3 * _time_loop(torch, f_chain, flush=flush, label="dsa_sparse_mla_decode_262k",
                                                                        gpu_index=gpu_index) / n_mla

    def chain2(pk, ck):       # the same step with the selection in two launches (scorer, top-k with the expansion inside)
        hk.indexer_select(qi, pk, w, q_pos, sc, idx, raw, 1, npools)
        hk.mla_sparse_decode(ql, ck, raw, 2052, lo, 1, n_split=ns, workspace=wsb)
    f_chain2 = [(lambda pk=pk, ck=ck: chain2(pk, ck)) for pk, ck in zip(pks, ckvs)]
    res["dsa_sparse_mla_decode_262k_fused_selection_us_per_layer"] = 1e3 * _time_loop(
        torch, f_chain2, flush=flush, label="dsa_sparse_mla_decode_262k_fused_selection", gpu_index=gpu_index) / n_mla
    del pks, ckvs, f_sparse, f_chain, f_chain2
    torch.cuda.empty_cache()
    # ---- one KDA layer of the 32K prefill from the projections' fp32 outputs to the gated, normalised fp16
    #      activations: the reference's call sequence (transpose+cast, gate, conv, recurrence, gated norm) and the
    #      fused form (cast+conv, prefill that forms its own gates, gated norm).  Buffers exceed L2. ----
    T, F = T_FULL, 3 * H * D
    raw_g = synth.kda_raw_gates(T, H, D, seed=2)
    f_raw, b_raw = dev(raw_g["f"]), dev(raw_g["b"])
    dtb, alog, lb = dev(raw_g["dt_bias"]), dev(raw_g["a_log"]), raw_g["lower_bound"]
    x32 = torch.randn(1, T, F, device="cuda")
    g_out = torch.randn(T * H, D, device="cuda")
    w_conv = (0.1 * torch.randn(F, 4, device="cuda")).to(torch.bfloat16)
    w_norm = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    mixed = torch.empty(F, T, dtype=torch.bfloat16, device="cuda")
    conv_out = torch.empty(1, T, F, dtype=torch.bfloat16, device="cuda")
    beta = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    gate = torch.empty(T, H, D, dtype=torch.float32, device="cuda")
    cst = torch.zeros(1, F, 4, dtype=torch.bfloat16, device="cuda")
    rst = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
    rec = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    y16 = torch.empty(T * H, D, dtype=torch.float16, device="cuda")
    ws = torch.empty(hk.kda_chunked_workspace_bytes(1, T, H), dtype=torch.uint8, device="cuda")

    def layer_two_step():
        hk.kda_transpose_cast(mixed, x32, T, F)
        hk.kda_gate(b_raw, f_raw, dtb, alog, lb, beta, gate, T, H, D)
        hk.cuda_causal_conv1d_update(mixed, cst, None, w_conv, None, conv_out, 1, F, T, 4, 4, True, False)
        hk.cuda_recurrent_gated_delta_rule(conv_out, gate, beta, rst, rec, 1, T, H, H, D, D, 1, None, True, False, workspace=ws)
        hk.gated_rms_norm(rec, w_norm, y16, g_out, T * H, D, 1e-6, gate_act=1)

    def layer_fused():
        hk.kda_cast_conv(x32, cst, None, w_conv, None, conv_out, 1, F, T, True)
        hk.kda_chunked_prefill_gated(conv_out, f_raw, b_raw, dtb, alog, lb, rst, rec, 1, T, H, workspace=ws)
        hk.gated_rms_norm(rec, w_norm, y16, g_out, T * H, D, 1e-6, gate_act=1)

    ms2 = _time_loop(torch, [layer_two_step], iters=5, sustain_ms=0.0)
    ms1 = _time_loop(torch, [layer_fused], iters=5, sustain_ms=0.0)
    res["kda_layer_prefill_32k_reference_call_sequence_ms"] = ms2
    res["kda_layer_prefill_32k_fused_ms"] = ms1
    res["kda_layer_prefill_32k_fused_tokens_per_s"] = T / (ms1 * 1e-3)
    res["clocks_per_figure"] = dict(FIGURE_CLOCKS)
    return res


if __name__ == "__main__":
    main()
