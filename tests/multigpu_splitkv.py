"""Split-KV MLA decode over N GPUs (run with torchrun, one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29600 tests/multigpu_splitkv.py [--ctx 262144] [--iters 20]

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
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import splitkv
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    L, m, scale = args.ctx, 1, 512 ** -0.5
    g = torch.Generator(device="cuda").manual_seed(1234)          # same cache and query on every rank
    ckv = torch.randn(L, 512, generator=g, device="cuda", dtype=torch.float32).half()
    q = torch.randn(m, 64, 512, generator=g, device="cuda", dtype=torch.float32).half()
    b, e = splitkv.shard_tokens(L, rank, world)
    shard = ckv[b:e].contiguous()
    dec = splitkv.SplitKVDecoder(m, max_wait_ms=2000)
    out = torch.zeros(m, 64, 512, dtype=torch.float16, device="cuda")
    ref = torch.zeros_like(out)
    hk.mla_dense_prefill(q, ckv, ref, m, L - 1, scale=scale)      # single-GPU answer on the whole cache
    dec.step(q, shard, e - b, out, scale)
    torch.cuda.synchronize()
    err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    status = hk.read_device_status()
    # timing
    for _ in range(3):
        dec.step(q, shard, e - b, out, scale)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        dec.step(q, shard, e - b, out, scale)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # single-GPU time of the same decode for reference (rank 0 only matters)
    ns = hk.mla_auto_splits(m, L)
    ws = torch.empty(max(256, hk.mla_partial_bytes(ns, m * 64)), dtype=torch.uint8, device="cuda")
    for _ in range(3):
        hk.mla_dense_prefill(q, ckv, ref, m, L - 1, scale=scale, n_split=ns, workspace=ws)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        hk.mla_dense_prefill(q, ckv, ref, m, L - 1, scale=scale, n_split=ns, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    t1 = e0.elapsed_time(e1) / args.iters
    # failure injection on the host side of the protocol: rank 1 withholds its flag for one step
    timeout_seen = None
    if world > 1:
        dec.max_wait_ms = 100
        out2 = torch.full_like(out, 3.0)
        dec.step(q, shard, e - b, out2, scale, signal=(rank != 1))
        torch.cuda.synchronize()
        timeout_seen = hk.read_device_status() == hk.HK_ERR_TIMEOUT and bool((out2 == 3.0).all())
        dist.barrier()
        # recovery: the withheld epoch is published late, the next step works again
        if rank == 1:
            hk.peer_signal(dec.flag_ptrs, world, rank, dec.epoch)
        torch.cuda.synchronize()
        dist.barrier()
        dec.max_wait_ms = 2000
        dec.step(q, shard, e - b, out, scale)
        torch.cuda.synchronize()
        err = max(err, float((out.float() - ref.float()).abs().max() / ref.float().abs().max()))
    flags = [err < 2e-3, status == 0, timeout_seen in (None, True), hk.read_device_status() == 0]
    if not all(flags):
        print(f"rank {rank}: err={err:.3e} first_status={status} timeout_seen={timeout_seen} checks={flags}",
              file=sys.stderr, flush=True)
    ok = torch.tensor([int(all(flags))], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"test": "splitkv_decode", "n_gpus": world, "ctx": L, "max_rel_err": err,
                          "us_per_step": float(t) * 1e3, "single_gpu_us": t1 * 1e3,
                          "hbm_gbs_aggregate": L * 1024 / (float(t) * 1e-3) / 1e9,
                          "timeout_path_ok": timeout_seen, "all_ranks_ok": bool(ok.item())}), flush=True)
    dec.close()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
