"""No-GPU checks of the boundary: the shared library loads, exports every symbol the public header
declares (and nothing the header does not), the reference-named C++ launchers are exported, and the
Python host layer refuses to compute without a device."""
import os
import re
import subprocess

import pytest

import helios_glm53flash_b200 as hk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from helios_glm53flash_b200 import build as hk_build
    return hk_build.build()


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "helios_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_exactly_the_header(built):
    out = subprocess.check_output(["nm", "-D", "--defined-only", built], text=True)
    exported = sorted(l.split()[-1] for l in out.splitlines() if " T " in l and l.split()[-1].startswith("hk_"))
    declared = _header_symbols()
    assert exported == declared
    assert sorted(hk.SIGNATURES) == declared, "ctypes table covers the whole header"


def test_library_loads_and_answers_without_a_gpu(built):
    lib = hk.load_library()
    assert lib.hk_abi_version() == 1
    assert hk.status_string(0) == "ok" and "workspace" in hk.status_string(hk.HK_ERR_WORKSPACE)
    assert lib.hk_mla_partial_bytes(4, 128) >= 4 * 128 * 2056
    assert lib.hk_kda_chunked_workspace_bytes(1, 512, 32) > 0


def test_reference_named_launchers_are_exported(built):
    out = subprocess.check_output(["nm", "-DC", "--defined-only", built], text=True)
    for name in ["helios::aux::cuda_recurrent_gated_delta_rule(", "helios::aux::cuda_causal_conv1d_update(",
                 "helios::aux::dsa_topk(", "helios::attn::kpool_write(", "helios::attn::indexer_score(",
                 "helios::attn::pool_expand_row(", "helios::attn::mla_sparse_decode(",
                 "helios::attn::mla_dense_prefill(", "helios::attn::q_latent_t(", "helios::attn::o_absorb_t(",
                 "helios::attn::o_absorb(", "helios::attn::wuv_transpose(", "helios::aux::gated_rms_norm(",
                 "helios::glue::kda_transpose_cast(", "helios::glue::kda_gate(", "helios::glue::kda_prepare(", "helios::glue::layernorm_f16("]:
        assert name in out, name


def test_no_cpu_path():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    t = torch.zeros(4)
    with pytest.raises(RuntimeError):
        hk.dsa_topk(t, 4, t, 1, 4, 1, 1)


def test_product_does_not_reference_the_oracle():
    pkg = os.path.join(ROOT, "helios_glm53flash_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "liboracle" not in text and "hk_oracle" not in text and "oracle/" not in text, f


def test_host_only_answers_of_the_abi(built):
    """entry points that compute on the host: sizes, layouts and the dispatch rule (no device needed)"""
    from helios_glm53flash_b200 import splitkv
    lib = hk.load_library()
    # candidate area of the sparse split-KV selection: 256 B of flags + two sets of (int32 index, fp16 score) x 512 x ranks x rows
    for m, g in ((1, 1), (1, 8), (3, 2), (8, 8)):
        assert lib.hk_dsa_select_region_bytes(m, g) == 256 + 2 * m * g * 512 * 6
    assert lib.hk_dsa_select_region_bytes(1, 9) == 0 and lib.hk_dsa_select_region_bytes(0, 2) == 0
    lay = splitkv.region_layout(64, 2, cand_bytes=lib.hk_dsa_select_region_bytes(1, 2))
    assert lay["cand"] % 256 == 0 and lay["total"] == lay["cand"] + lib.hk_dsa_select_region_bytes(1, 2)
    # the dispatch rule of the recurrence launcher: chunked path for channelwise decay, no history, 128-wide heads, >= 64 tokens
    rule = lambda seqlen, dk, dv, cw, hist: lib.hk_kda_dispatch_is_chunked(seqlen, 32, 32, dk, dv, 1, cw, hist)
    assert rule(64, 128, 128, 1, 0) == 1 and rule(32768, 128, 128, 1, 0) == 1
    assert rule(63, 128, 128, 1, 0) == 0 and rule(1, 128, 128, 1, 0) == 0
    assert rule(4096, 128, 128, 1, 1) == 0 and rule(4096, 128, 128, 0, 0) == 0 and rule(4096, 64, 64, 1, 0) == 0
    # static no-allocation entry: 64 (split, row) slots
    assert lib.hk_mla_sparse_static_max_slots() == 64
