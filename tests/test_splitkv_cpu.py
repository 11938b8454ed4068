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
