"""Multi-GPU paths, run as child processes (one rank per GPU, torchrun) when the machine has at least two GPUs:
split-KV MLA decode in both exchange forms - result against the single-GPU kernel on the whole cache, a withheld
signal that must end in a clean timeout on every rank (host-made failure, bounded device waits), and the
re-synchronisation after it.  NVLS is off in the children; the kernels use plain peer loads and stores."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_worker(n, port, extra, script="splitkv_worker.py"):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", script)] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-4000:]
    return json.loads(lines[-1])


@pytest.mark.parametrize("form,batch", [("heads", 1), ("heads", 3), ("all", 2)])
def test_splitkv_decode_two_gpus(form, batch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run_worker(2, 29611 + batch, ["--ctx", "20000", "--iters", "5", "--batch", str(batch), "--form", form])
    assert res["all_ranks_ok"] and res["form"] == form and res["max_rel_err"] < 2e-3 and res["timeout_path_ok"] is True, res


@pytest.mark.parametrize("rows,ctx", [(1, 30001), (3, 6002)])
def test_sparse_splitkv_decode_two_gpus(rows, ctx):
    """one sequence, pools and cache rows split over two GPUs: the selection must equal the one-GPU selection exactly,
    the attention output within tolerance; a withheld candidate flag ends in a clean timeout on every rank"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run_worker(2, 29640 + rows, ["--ctx", str(ctx), "--iters", "5", "--rows", str(rows)], script="splitkv_sparse_worker.py")
    assert res["all_ranks_ok"] and res["selection_identical"] and res["max_rel_err"] < 2e-3 and res["timeout_path_ok"] is True, res
