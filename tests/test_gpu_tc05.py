"""The tcgen05 / TMEM helper layer: a GEMM through every operand layout and instruction shape the
kernels use, checked against torch fp32 matmul, plus the reference's own parity binary."""
import os
import subprocess

import numpy as np
import pytest
import torch

import helios_glm53flash_b200 as hk

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("M,N,K,b_layout", [(128, 32, 128, 0), (128, 256, 128, 0), (128, 64, 64, 1), (128, 32, 128, 1),
                                            (128, 16, 128, 0), (128, 128, 16, 1), (128, 256, 64, 1), (128, 64, 64, 2), (128, 64, 128, 3),
                                            # 128-byte-swizzle operands (bit 2: A, bit 3: B), K-major and MN-major
                                            (64, 64, 64, 0x8), (64, 48, 128, 0x8), (128, 32, 128, 0x4), (128, 32, 128, 0xc),
                                            (128, 64, 64, 0x6), (128, 64, 48, 0x6), (128, 64, 64, 0x9), (128, 128, 64, 0xf),
                                            # bit 10: issued by a converged warp with an elected lane (tc::mma_f16_if)
                                            (128, 32, 128, 0x400), (128, 256, 128, 0x400), (64, 48, 128, 0x408), (64, 64, 64, 0x408),
                                            (128, 64, 48, 0x406), (128, 128, 64, 0x40f)])
def test_tc05_gemm_matches_fp32_matmul(M, N, K, b_layout):
    g = torch.Generator(device="cpu").manual_seed(M + N + K + b_layout)
    a = torch.randn(M, K, generator=g).half()
    b = torch.randn(N, K, generator=g).half()
    want = a.float() @ b.float().t()
    b_in = b if (b_layout & 1) == 0 else b.t().contiguous()
    a_in = a if (b_layout & 2) == 0 else a.t().contiguous()
    d, status = hk.tc05_selftest(a_in.cuda(), b_in.cuda(), M, N, K, b_layout)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    d = d.cpu()
    got = d[:M] if M == 128 else d[[(r // 16) * 32 + r % 16 for r in range(64)]]   # M = 64: row r sits in lane 32 (r / 16) + r % 16
    assert torch.allclose(got, want, atol=2e-2, rtol=1e-3), float((got - want).abs().max())


def test_reference_parity_binary_against_this_library():
    """The reference's own kernel parity test (src/cuda/attn/test/test_attn_parity.cpp), compiled
    from the reference tree and linked against libhelios_b200.so through the helios::attn shim."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_attn_parity_on_b200")
    if not os.path.exists(exe):
        pytest.skip("reference test binary not built (make -C oracle reftest)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:])
    assert "ATTN PARITY: ALL PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
