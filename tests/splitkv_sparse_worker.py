"""Worker of tests/test_gpu_multigpu.py: SPARSE split-KV MLA decode of one sequence over N GPUs, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29620 tests/splitkv_sparse_worker.py [--ctx 262144] [--iters 20] [--rows 1]

Every rank builds the same seeded cache, pooled indexer keys and queries, keeps only its slice for the N-GPU step, and
checks against the one-GPU chain on the whole sequence (indexer scores -> top-512 -> expansion -> sparse attention):
the selected pools must be identical, the attention output equal within the attention tolerance.  Times the step
(device events, max over ranks) and exercises the bounded wait of the candidate exchange."""
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
    ap.add_argument("--rows", type=int, default=1, help="query rows of the step (the last --rows positions of the sequence)")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    import helios_glm53flash_b200 as hk
    from helios_glm53flash_b200 import splitkv
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    L, m, scale = args.ctx, args.rows, 512 ** -0.5
    P = L // 4
    g = torch.Generator(device="cuda").manual_seed(4321)
    ckv = torch.randn(L, 512, generator=g, device="cuda", dtype=torch.float16)
    pool = (torch.randn(P, 128, generator=g, device="cuda", dtype=torch.float32) * 0.5).half()
    q_lat = torch.randn(m, 64, 512, generator=g, device="cuda", dtype=torch.float32).half()
    q_idx = torch.randn(m, 32, 128, generator=g, device="cuda", dtype=torch.float32).half()
    w = torch.rand(m, 32, generator=g, device="cuda", dtype=torch.float32).half()
    q_pos = torch.arange(L - m, L, dtype=torch.int32, device="cuda")

    # the one-GPU chain on the whole sequence
    sc = torch.empty(m, P, dtype=torch.float16, device="cuda")
    topk = torch.empty(m, 512, dtype=torch.int32, device="cuda")
    raw = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
    ref = torch.zeros(m, 64, 512, dtype=torch.float16, device="cuda")
    ns = hk.mla_auto_splits(m, 2052)
    ws = torch.empty(max(256, hk.mla_partial_bytes(ns, m * 64)), dtype=torch.uint8, device="cuda")

    def one_gpu():
        hk.indexer_score(q_idx, pool, w, q_pos, sc, m, P)
        hk.dsa_topk(sc, P, topk, m, P, min(512, P), 512)
        hk.pool_expand_row(topk, q_pos, raw, m)
        hk.mla_sparse_decode(q_lat, ckv, raw, 2052, ref, m, scale=scale, n_split=ns, workspace=ws)

    one_gpu()
    torch.cuda.synchronize()
    prange, rrange = splitkv.shard_pools(L, rank, world)
    pool_shard = pool[prange[0]:prange[1]].contiguous()
    ckv_shard = ckv[rrange[0]:rrange[1]].contiguous()
    dec = splitkv.SplitKVDecoder(m, max_wait_ms=2000, sparse=True)
    out = torch.zeros(m, 64, 512, dtype=torch.float16, device="cuda")

    def step(**kw):
        dec.step_sparse(q_lat, q_idx, w, q_pos, pool_shard, prange, ckv_shard, rrange, out, scale, **kw)

    def rel():
        return float((out.float() - ref.float()).abs().max() / ref.float().abs().max())

    step()
    torch.cuda.synchronize()
    same_sel = bool(torch.equal(dec.sel_pools, topk))
    err, status = rel(), hk.read_device_status()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    t_host = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
    dist.all_reduce(t_host, op=dist.ReduceOp.MAX)
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
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
    err = max(err, rel())
    same_sel = same_sel and bool(torch.equal(dec.sel_pools, topk))
    # the one-GPU chain, replayed from a graph as well
    g1 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g1):
        one_gpu()
    g1.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        g1.replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = e0.elapsed_time(e1) / args.iters
    timeout_seen = None
    if world > 1:
        # rank 1 withholds its candidate flag for one step: the others' selection must give up cleanly
        dec.max_wait_ms = 100
        step(signal_candidates=(rank != 1))
        torch.cuda.synchronize()
        timeout_seen = hk.read_device_status() == hk.HK_ERR_TIMEOUT
        dist.barrier()
        dec.resync()
        dec.max_wait_ms = 2000
        out.zero_()
        step()
        torch.cuda.synchronize()
        err = max(err, rel())
        same_sel = same_sel and bool(torch.equal(dec.sel_pools, topk))
    flags = [err < 2e-3, status == 0, same_sel, timeout_seen in (None, True), hk.read_device_status() == 0]
    if not all(flags):
        print(f"rank {rank}: err={err:.3e} first_status={status} same_sel={same_sel} timeout_seen={timeout_seen} checks={flags}",
              file=sys.stderr, flush=True)
    ok = torch.tensor([int(all(flags))], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"test": "splitkv_sparse_decode", "n_gpus": world, "ctx": L, "rows": m, "max_rel_err": err,
                          "selection_identical": same_sel, "us_per_step": float(t) * 1e3,
                          "us_per_step_host_launched": float(t_host) * 1e3, "single_gpu_us": t1 * 1e3,
                          "timeout_path_ok": timeout_seen, "all_ranks_ok": bool(ok.item())}), flush=True)
    dec.close()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
