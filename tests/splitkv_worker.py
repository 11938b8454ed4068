"""Worker of tests/test_gpu_multigpu.py: split-KV MLA decode over N GPUs, one rank per GPU, started by

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29600 tests/splitkv_worker.py [--ctx 262144] [--iters 20] [--form heads|all]

Checks the N-GPU result against the single-GPU dense kernel on the whole cache (every rank builds the
same seeded cache) and times the step (device events, max over ranks).  Also exercises the bounded wait:
in one extra step rank 1 withholds its flag and the other ranks' combine must time out cleanly."""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=262144)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded per step, each with its own cache of --ctx rows")
    ap.add_argument("--form", default=None, choices=[None, "heads", "all"], help="exchange form (default: heads when 64 % ranks == 0)")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import splitkv
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    L, m, scale = args.ctx, args.batch, 512 ** -0.5
    g = torch.Generator(device="cuda").manual_seed(1234)          # same caches and queries on every rank
    ckv = torch.randn(m * L, 512, generator=g, device="cuda", dtype=torch.float16)     # sequence s = rows [s L, (s+1) L)
    q = torch.randn(m, 64, 512, generator=g, device="cuda", dtype=torch.float32).half()
    b, e = splitkv.shard_tokens(L, rank, world)
    # this rank's slice of every sequence, concatenated; row s of the batch starts at s (e - b)
    shard = torch.cat([ckv[s * L + b:s * L + e] for s in range(m)]).contiguous()
    shard_base = (torch.arange(m, device="cuda", dtype=torch.int64) * (e - b))
    full_base = (torch.arange(m, device="cuda", dtype=torch.int64) * L)
    full_len = torch.full((m,), L, dtype=torch.int32, device="cuda")
    dec = splitkv.SplitKVDecoder(m, max_wait_ms=2000, form=args.form)
    out = torch.zeros(m, 64, 512, dtype=torch.float16, device="cuda")
    ref = torch.zeros_like(out)
    hk.mla_dense_prefill(q, ckv, ref, m, 0, scale=scale, kv_base=full_base, kv_len=full_len, n_keys_hint=L)   # single-GPU answer
    dec.step(q, shard, e - b, out, scale, kv_base=shard_base)
    torch.cuda.synchronize()
    err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    status = hk.read_device_status()
    # timing: (1) steps launched from the host one by one, (2) one step captured in a CUDA graph and
    # replayed (the step number lives on the device, so replays stay in lock step across the ranks)
    for _ in range(3):
        dec.step(q, shard, e - b, out, scale, kv_base=shard_base)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        dec.step(q, shard, e - b, out, scale, kv_base=shard_base)
    e1.record()
    torch.cuda.synchronize()
    t_host = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
    dist.all_reduce(t_host, op=dist.ReduceOp.MAX)
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dec.step(q, shard, e - b, out, scale, kv_base=shard_base)
    dec.epoch += args.iters + 3 - 1          # host mirror of the device step counter after the replays below
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(args.iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err = max(err, float((out.float() - ref.float()).abs().max() / ref.float().abs().max()))
    # single-GPU time of the same decode for reference (rank 0 only matters)
    ns = hk.mla_auto_splits(m, L)
    ws = torch.empty(max(256, hk.mla_partial_bytes(ns, m * 64)), dtype=torch.uint8, device="cuda")
    for _ in range(3):
        hk.mla_dense_prefill(q, ckv, ref, m, 0, scale=scale, kv_base=full_base, kv_len=full_len, n_split=ns, workspace=ws, n_keys_hint=L)
    torch.cuda.synchronize()
    g1 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g1):
        hk.mla_dense_prefill(q, ckv, ref, m, 0, scale=scale, kv_base=full_base, kv_len=full_len, n_split=ns, workspace=ws, n_keys_hint=L)
    g1.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        g1.replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = e0.elapsed_time(e1) / args.iters
    # failure injection on the host side of the protocol: rank 1 withholds its flag for one step
    timeout_seen = None
    if world > 1:
        dec.max_wait_ms = 100
        out2 = torch.full_like(out, 3.0)
        dec.step(q, shard, e - b, out2, scale, signal=(rank != 1), kv_base=shard_base)
        torch.cuda.synchronize()
        timeout_seen = hk.read_device_status() == hk.HK_ERR_TIMEOUT and bool((out2 == 3.0).all())
        dist.barrier()
        # recovery: after a timeout the group re-synchronises on the host, then steps again
        dec.resync()
        dec.max_wait_ms = 2000
        dec.step(q, shard, e - b, out, scale, kv_base=shard_base)
        torch.cuda.synchronize()
        err = max(err, float((out.float() - ref.float()).abs().max() / ref.float().abs().max()))
    flags = [err < 2e-3, status == 0, timeout_seen in (None, True), hk.read_device_status() == 0]
    if not all(flags):
        print(f"rank {rank}: err={err:.3e} first_status={status} timeout_seen={timeout_seen} checks={flags}",
              file=sys.stderr, flush=True)
    ok = torch.tensor([int(all(flags))], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"test": "splitkv_decode", "form": dec.form, "n_gpus": world, "ctx": L, "batch": m, "max_rel_err": err,
                          "us_per_step": float(t) * 1e3, "us_per_step_host_launched": float(t_host) * 1e3,
                          "single_gpu_us": t1 * 1e3,
                          "hbm_gbs_aggregate": m * L * 1024 / (float(t) * 1e-3) / 1e9,
                          "timeout_path_ok": timeout_seen, "all_ranks_ok": bool(ok.item())}), flush=True)
    dec.close()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
