"""Multi-process host logic of split-KV decode on CPU: two gloo ranks each attend their slice of the
cache with the oracle, exchange the (m, l, acc) partials and merge them; the merged result must equal
un-split attention.  Also the failure path on the host: a rank that never contributes is detected by
a short timeout instead of a hang."""
import os
import sys

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def _worker(rank, world, port, fail_rank, ret):
    import datetime
    import hk_oracle as orc
    from helios_glm53flash_b200 import splitkv, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        L, m = 1001, 2
        inp = synth.mla_inputs(L, m, seed=3, cache_std=0.5)
        b, e = splitkv.shard_tokens(L, rank, world)
        _, _, part = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=np.full(m, b, np.int64),
                                    kv_len=np.full(m, e - b, np.int32), partial=True)
        if rank == fail_rank:
            ret[rank] = "left"          # this rank leaves between steps without contributing
            return
        gathered = [None] * world
        try:
            dist.all_gather_object(gathered, part)
        except Exception as ex:        # the peers learn of the missing rank through the group timeout
            ret[rank] = "timeout:" + type(ex).__name__
            return
        merged = splitkv.merge_partials_numpy(gathered)
        _, full = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=np.zeros(m, np.int64),
                                 kv_len=np.full(m, L, np.int32))
        ret[rank] = float(np.max(np.abs(merged.reshape(m, 64, 512) - full)))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(world, fail_rank, port):
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive()
    return dict(ret)


def test_two_ranks_merge_equals_unsplit_attention():
    ret = _run(2, -1, 29531)
    assert set(ret) == {0, 1}
    assert all(isinstance(v, float) and v < 1e-5 for v in ret.values()), ret


def test_missing_rank_is_reported_not_hung():
    ret = _run(2, 1, 29532)
    assert ret[1] == "left"
    assert isinstance(ret[0], str) and ret[0].startswith("timeout"), ret


def test_shard_and_region_layout():
    from helios_glm53flash_b200 import splitkv
    for n, w in [(262144, 8), (1001, 2), (7, 8)]:
        spans = [splitkv.shard_tokens(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n and all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
    lay = splitkv.region_layout(64, 8)
    for par in (0, 1):
        assert all(lay[k + str(par)] % 256 == 0 for k in ("m", "l", "acc"))
    assert lay["m0"] >= 256 and lay["m1"] == lay["acc0"] + 64 * 2048      # two partial sets, one per step parity
    assert lay["total"] == lay["acc1"] + 64 * 2048


def _sparse_worker(rank, world, port, ret):
    """gloo rank of the sparse split-KV selection: local top-k of the own pools with the oracle, candidates gathered,
    selection over the candidates in ascending global index (the host statement of hk_dsa_select_splitkv)"""
    import datetime
    import hk_oracle as orc
    from helios_glm53flash_b200 import splitkv, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        n_tokens, m, k = 4 * 1500 + 3, 2, 512
        P = n_tokens // 4
        r = synth.rng(11)                                          # the same scores on every rank
        sc = np.round(r.standard_normal((m, P), dtype=np.float32) * 4) / 4     # coarse: many exact ties at the threshold
        sc[:, P // 2:] = np.where(r.random((m, P - P // 2)) < 0.25, -np.inf, sc[:, P // 2:])
        bits = synth.f32_to_f16_bits(sc)
        (p0, p1), _ = splitkv.shard_pools(n_tokens, rank, world)
        local = np.ascontiguousarray(bits[:, p0:p1])
        idx = orc.dsa_topk(local, p1 - p0, m, p1 - p0, min(k, p1 - p0), 512)       # local selection, -1 padded
        cand = []
        for row in range(m):
            sel = np.sort(idx[row][idx[row] >= 0])                  # ascending local index
            cand.append((sel + p0, local[row][sel]))
        gathered = [None] * world
        dist.all_gather_object(gathered, cand)
        got = np.full((m, 512), -1, dtype=np.int32)
        for row in range(m):
            gidx = np.concatenate([g[row][0] for g in gathered])    # rank by rank = ascending global index
            gsc = np.concatenate([g[row][1] for g in gathered])
            assert np.all(np.diff(gidx) > 0)
            pos = orc.dsa_topk(gsc.reshape(1, -1), gsc.size, 1, gsc.size, min(k, gsc.size), 512)[0]
            got[row] = np.where(pos >= 0, gidx[np.maximum(pos, 0)], -1)
        want = orc.dsa_topk(bits, P, m, P, k, 512)
        ret[rank] = bool(np.array_equal(got, want))
    finally:
        dist.destroy_process_group()


def test_sparse_selection_over_rank_slices_equals_whole_row_selection_on_cpu():
    """the property the GPU kernels rely on, with two gloo ranks and the oracle's top-k: the union of the ranks' local
    selections contains the whole-row selection, and selecting among the candidates in ascending global index breaks
    ties as the whole-row selection does"""
    world, port = 2, 29655
    ret = mp.Manager().dict()
    mp.spawn(_sparse_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_pools_partitions_pools_and_rows():
    from helios_glm53flash_b200 import splitkv
    for n_tokens in (4, 7, 1000, 1003, 262144):
        for world in (1, 2, 3, 8):
            prev_p, prev_r = 0, 0
            for rank in range(world):
                (p0, p1), (r0, r1) = splitkv.shard_pools(n_tokens, rank, world)
                assert p0 == prev_p and r0 == prev_r and r0 == 4 * p0 and p1 >= p0
                assert r1 == (n_tokens if rank == world - 1 else 4 * p1)
                prev_p, prev_r = p1, r1
            assert prev_p == n_tokens // 4 and prev_r == n_tokens
