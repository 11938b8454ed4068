"""The allocation-free sparse MLA decode entry point (hk_mla_sparse_static), called through the C ABI.

Who needs it: hosts that cannot allocate device memory at call time (an engine that hands out all of
its memory from a start-up arena and whose launchers have no scratch parameter).  The split-KV
partials then sit in a fixed array inside the library instead of a caller buffer.  The check is that
it returns what the ordinary entry point (caller-provided workspace) returns, on two calls in a row -
the second with other inputs and another split count, so stale contents of the shared array would
show.  The file name sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import hk_oracle as orc
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max |a-b| / max |b|, the tolerance of the attention tests


def _f16_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.float16).cuda()


def _max_rel(a, b):
    a, b = a.float().cpu().numpy().astype(np.float64), b.float().cpu().numpy().astype(np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    lib = hk.load_library()
    assert lib.hk_mla_sparse_static_max_slots() == 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # third call: m = 2 rows x 32 splits = all 64 slots of the built-in array (the sizing is an exact fit)
    for call, (m, kidx, T, n_split, seed) in enumerate([(1, 2052, 16384, 0, 3), (2, 700, 4096, 7, 4), (2, 1900, 8192, 32, 5)]):
        inp = synth.mla_inputs(T, m, seed=seed, cache_std=0.5)
        rs = np.random.RandomState(seed)
        ridx = rs.randint(0, T, (m, kidx)).astype(np.int32)
        ridx[:, 5::11] = -1
        q, c, r = _f16_dev(inp["q_lat"]), _f16_dev(inp["ckv"]), torch.from_numpy(ridx).cuda()
        # existing entry point, caller-provided workspace
        want = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
        hk.mla_sparse_decode(q, c, r, kidx, want, m, scale=0.0625, n_split=n_split)
        # new entry point, straight through the C ABI: no workspace argument, nothing allocated
        got = torch.full((m, 64, 512), 7.0, dtype=torch.float16, device="cuda")
        st = lib.hk_mla_sparse_static(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(c.data_ptr()),
                                      ctypes.c_void_p(r.data_ptr()), kidx, ctypes.c_void_p(got.data_ptr()), m,
                                      ctypes.c_float(0.0625), n_split, stream)
        assert st == hk.HK_OK, hk.status_string(st)
        torch.cuda.synchronize()
        assert hk.read_device_status() == 0
        err = _max_rel(got, want)
        assert err < TOL, "call %d: %.3e" % (call, err)
        # and against the CPU oracle, so that the two CUDA entry points are not only compared with each other
        _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, raw_idx=ridx, kidx=kidx)
        g32 = got.float().cpu().numpy().astype(np.float64)
        err_o = float(np.max(np.abs(g32 - o32)) / np.max(np.abs(o32)))
        assert err_o < TOL, "call %d vs oracle: %.3e" % (call, err_o)


def test_static_scratch_entry_rejects_oversized_requests():
    lib = hk.load_library()
    t = torch.zeros(65 * 64 * 512, dtype=torch.float16, device="cuda")
    idx = torch.zeros(65 * 8, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(idx.data_ptr()), 8,
            ctypes.c_void_p(t.data_ptr()))
    assert lib.hk_mla_sparse_static(*args, 65, ctypes.c_float(0.0625), 1, stream) == hk.HK_ERR_WORKSPACE
    assert lib.hk_mla_sparse_static(*args, 2, ctypes.c_float(0.0625), 33, stream) == hk.HK_ERR_WORKSPACE
    torch.cuda.synchronize()
