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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

T_FULL, HEADS, DIM = 32768, 32, 128
CPU_SAMPLE_T = 16384
METRIC = "kda_prefill_tokens_per_s_at_32k_ctx"


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler(threading.Thread):
    """samples nvidia-smi clocks and throttle reasons while the timed region runs"""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag:
            try:
                o = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True, timeout=5).stdout.strip()
                if o:
                    self.rows.append([x.strip() for x in o.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(self.rows[0][1]) if self.rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.rows)}


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
                      % (sample_t, max(1, steps)), "seconds": best}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cb = cpu_baseline(steps=max(1, min(args.steps, 3)))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * T_FULL / cb["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "kda_prefill_32k: conv1d(K=4,SiLU) + gated delta rule, B=1, T=32768, H=32, d=128",
                       "note": "reference path is CUDA-only; this arm is its CPU restatement (oracle) on a bounded sample"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=T_FULL, help="sequence length (default: the benchmark's 32768)")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / MLA side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

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

    for _ in range(warmup):
        path = step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(steps):
        step(ev=evs[i])
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    sampler.stop_flag = True
    conv_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / steps
    kda_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / steps
    assert hk.read_device_status() == 0, "a bounded device wait expired"

    # ---- end to end through the host-facing call: pinned host inputs in, result back to the host ----
    e2e_steps = max(2, min(steps, 5))
    hx2, hg2, hb2 = torch.empty_like(d_x), torch.empty_like(d_g), torch.empty_like(d_beta)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(e2e_steps):
        hx2.copy_(h_x, non_blocking=True)
        hg2.copy_(h_g, non_blocking=True)
        hb2.copy_(h_beta, non_blocking=True)
        step(hx2, hg2, hb2)
        h_out.copy_(out, non_blocking=True)
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

    extras = {}
    if rank == 0 and not args.no_extras:
        extras = side_measurements(hk, synth, torch, np)

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
            "kernel_ms": {"conv1d": conv_ms, "kda_chunked_prefill(prep+scan)": kda_ms},
            "roofline": {"bound": "hbm", "kernel": "kda_chunk_prep_kernel + kda_chunk_scan_kernel",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": None, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": alg_bytes,
                         "tensor_tflops_dense_chunk_math": (T // 64) * H * 11.71e6 / (kda_ms * 1e-3) / 1e12},
            "e2e": {"value": world * T / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": 3 * steps,
            "clocks": sampler.summary(),
            "extras": extras,
        }
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(steps=1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _time_cuda(torch, fn, iters=20, warm=3, flush=None):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def side_measurements(hk, synth, torch, np):
    """decode-side figures at 32K / 262K context (median kernel time, L2 flushed between iterations)"""
    from gpu_util import dev, dev_bf16, dev_f16
    res = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    H, D = HEADS, DIM
    # KDA decode step, one layer (state 2 MiB in + out)
    kd = synth.kda_inputs(1, H, D, seed=5)
    q, g, b = dev_bf16(kd["mixed_qkv"]), dev(kd["g"]), dev_bf16(kd["beta"])
    st = torch.zeros(1, 1, H, D, D, dtype=torch.float32, device="cuda")
    o = torch.empty(1, 1, H, D, dtype=torch.bfloat16, device="cuda")
    ms = _time_cuda(torch, lambda: hk.cuda_recurrent_gated_delta_rule(q, g, b, st, o, 1, 1, H, H, D, D, 1, None, True, False), flush=flush)
    res["kda_decode_us_per_layer"] = ms * 1e3
    res["kda_decode_hbm_gbs"] = (2 * H * D * D * 4 + H * 1538) / (ms * 1e-3) / 1e9
    # dense MLA decode over a 32K latent cache
    for B in (1, 8):
        L = 32768
        ml = synth.mla_inputs(L * B, B, seed=6)
        qd, ck = dev_f16(ml["q_lat"]), dev_f16(ml["ckv"])
        base = dev((np.arange(B) * L).astype(np.int64))
        lens = dev(np.full(B, L, dtype=np.int32))
        lo = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
        ns = hk.mla_auto_splits(B, L)
        wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, B * 64)), dtype=torch.uint8, device="cuda")
        ms = _time_cuda(torch, lambda: hk.mla_dense_prefill(qd, ck, lo, B, 0, scale=512 ** -0.5, kv_base=base, kv_len=lens,
                                                            n_split=ns, workspace=wsb, n_keys_hint=L), flush=flush)
        res["mla_dense_decode_32k_b%d_us" % B] = ms * 1e3
        res["mla_dense_decode_32k_b%d_hbm_gbs" % B] = B * L * 1024 / (ms * 1e-3) / 1e9
    # indexer -> top-512 -> expand -> sparse MLA at 262,144 tokens of context
    npools, L = 65536, 262144
    ix = synth.indexer_inputs(npools, 1, seed=7)
    qi, pk, w = dev_f16(ix["q_idx"]), dev_f16(ix["pool_k"]), dev_f16(ix["w"])
    q_pos = dev(np.array([L - 1], dtype=np.int32))
    sc = torch.empty(1, npools, dtype=torch.float16, device="cuda")
    idx = torch.empty(1, 512, dtype=torch.int32, device="cuda")
    raw = torch.empty(1, 2052, dtype=torch.int32, device="cuda")
    ckv = torch.randn(L, 512, dtype=torch.float16, device="cuda")
    ql = torch.randn(1, 64, 512, dtype=torch.float16, device="cuda")
    lo = torch.empty(1, 64, 512, dtype=torch.float16, device="cuda")
    ns = hk.mla_auto_splits(1, 2052)
    wsb = torch.empty(max(256, hk.mla_partial_bytes(ns, 64)), dtype=torch.uint8, device="cuda")
    ms = _time_cuda(torch, lambda: hk.indexer_score(qi, pk, w, q_pos, sc, 1, npools), flush=flush)
    res["indexer_score_262k_us"] = ms * 1e3
    res["indexer_score_262k_hbm_gbs"] = npools * 256 / (ms * 1e-3) / 1e9
    res["topk512_262k_us"] = 1e3 * _time_cuda(torch, lambda: hk.dsa_topk(sc, npools, idx, 1, npools, 512, 512), flush=flush)
    hk.pool_expand_row(idx, q_pos, raw, 1)
    ms = _time_cuda(torch, lambda: hk.mla_sparse_decode(ql, ckv, raw, 2052, lo, 1, n_split=ns, workspace=wsb), flush=flush)
    res["mla_sparse_decode_262k_us"] = ms * 1e3
    res["mla_sparse_decode_262k_hbm_gbs"] = 2052 * 1024 / (ms * 1e-3) / 1e9
    return res


if __name__ == "__main__":
    main()
