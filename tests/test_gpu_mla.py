"""GPU parity of absorbed MLA (sparse gather / dense causal, decode / prefill rows), the split-KV
partials and the log-sum-exp combine, through the C ABI."""
import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bits, dev, dev_f16, max_rel, sum_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max |a-b| / max |b| for attention outputs


def _sparse_case(m, kidx, T, scale, seed, holes=True, std=0.5):
    inp = synth.mla_inputs(T, m, seed=seed, cache_std=std)
    r = np.random.RandomState(seed)
    ridx = r.randint(0, T, (m, kidx)).astype(np.int32)
    if holes:
        ridx[:, 3::7] = -1
    return inp, ridx


@pytest.mark.parametrize("m,kidx,T,scale,n_split", [
    (1, 64, 512, 0.0625, 1), (3, 300, 2048, 0.0625, 0), (1, 2052, 8192, 0.0625, 0), (2, 2052, 8192, 512 ** -0.5, 5),
    (1, 7, 64, 0.0625, 3), (5, 130, 1000, 0.0625, 2)])
def test_sparse_vs_oracle_and_reference(m, kidx, T, scale, n_split):
    inp, ridx = _sparse_case(m, kidx, T, scale, seed=kidx)
    o16, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, scale, raw_idx=ridx, kidx=kidx)
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_sparse_decode(q, c, dev(ridx), kidx, out, m, scale=scale, n_split=n_split)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    g = synth.f16_bits_to_f32(bits(out))
    assert max_rel(g, o32) < TOL and sum_rel(g, o32) < 3e-3
    if ref.available() and scale == 0.0625:
        out2 = torch.empty_like(out)
        ref.mla_sparse_decode(q, c, dev(ridx), kidx, out2, m)
        torch.cuda.synchronize()
        rr = synth.f16_bits_to_f32(bits(out2))
        assert max_rel(g, rr) < TOL, "within 2e-3 of the reference's own kernel"
        assert sum_rel(rr, o32) < 3e-3, "oracle pinned to the reference kernel"


def test_sparse_all_skipped_row_gives_zeros_and_duplicates_count_twice():
    m, kidx, T = 2, 16, 64
    inp, ridx = _sparse_case(m, kidx, T, 0.0625, seed=1, holes=False)
    ridx[0, :] = -1
    ridx[1, :] = np.array([5, 5, 9, -1] * 4, dtype=np.int32)
    o16, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, raw_idx=ridx, kidx=kidx)
    out = torch.full((m, 64, 512), 3.0, dtype=torch.float16, device="cuda")
    hk.mla_sparse_decode(dev_f16(inp["q_lat"]), dev_f16(inp["ckv"]), dev(ridx), kidx, out, m)
    torch.cuda.synchronize()
    g = synth.f16_bits_to_f32(bits(out))
    assert (g[0] == 0).all()
    assert max_rel(g[1], o32[1]) < TOL


@pytest.mark.parametrize("qlen,pos_start,scale,n_split", [(16, 0, 0.0625, 1), (1, 4095, 0.0625, 0), (1, 32767, 512 ** -0.5, 0),
                                                          (4, 1000, 0.0625, 3), (33, 100, 0.0625, 0)])
def test_dense_vs_oracle_and_reference(qlen, pos_start, scale, n_split):
    T = pos_start + qlen
    inp = synth.mla_inputs(T, qlen, seed=qlen + pos_start, cache_std=0.5)
    o16, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], qlen, 64, scale, pos_start=pos_start)
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    out = torch.empty(qlen, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(q, c, out, qlen, pos_start, scale=scale, n_split=n_split)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    g = synth.f16_bits_to_f32(bits(out))
    assert max_rel(g, o32) < TOL and sum_rel(g, o32) < 3e-3
    if ref.available() and scale == 0.0625 and T <= 8192:
        out2 = torch.empty_like(out)
        ref.mla_dense_prefill(q, c, out2, qlen, pos_start)
        torch.cuda.synchronize()
        rr = synth.f16_bits_to_f32(bits(out2))
        assert max_rel(g, rr) < TOL
        assert sum_rel(rr, o32) < 3e-3


def test_dense_batched_decode_over_concatenated_caches():
    B, L = 4, 777
    inp = synth.mla_inputs(B * L, B, seed=8, cache_std=0.5)
    base = (np.arange(B) * L).astype(np.int64)
    lens = np.array([L, L - 5, 1, 300], dtype=np.int32)
    o16, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], B, 64, 0.0625, kv_base=base, kv_len=lens)
    out = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(dev_f16(inp["q_lat"]), dev_f16(inp["ckv"]), out, B, 0, kv_base=dev(base), kv_len=dev(lens),
                         n_keys_hint=L)
    torch.cuda.synchronize()
    assert max_rel(synth.f16_bits_to_f32(bits(out)), o32) < TOL


def test_partials_and_combine_vs_oracle():
    m, L, S = 2, 900, 3
    inp = synth.mla_inputs(L, m, seed=21, cache_std=0.5)
    rows = m * 64
    cuts = [0, 250, 251, L]
    pm = torch.empty(S, rows, dtype=torch.float32, device="cuda")
    pl = torch.empty(S, rows, dtype=torch.float32, device="cuda")
    pa = torch.empty(S, rows, 512, dtype=torch.float32, device="cuda")
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    o_parts = []
    for s in range(S):
        base = np.full(m, cuts[s], dtype=np.int64)
        lens = np.full(m, cuts[s + 1] - cuts[s], dtype=np.int32)
        hk.mla_dense_partial(q, c, dev(base), dev(lens), 0, pm[s], pl[s], pa[s], m)
        o_parts.append(orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=base, kv_len=lens, partial=True)[2])
    out = torch.empty(rows, 512, dtype=torch.float16, device="cuda")
    hk.lse_combine(pm, pl, pa, S, rows, out)
    torch.cuda.synchronize()
    # the partial of each split, renormalised, equals the oracle's partial
    for s in range(S):
        om, ol, oa = o_parts[s]
        gm, gl, ga = pm[s].cpu().numpy(), pl[s].cpu().numpy(), pa[s].cpu().numpy()
        w = np.exp(gm - om)
        assert np.allclose(gl * w, ol, rtol=2e-3)
        assert max_rel(ga * w[:, None], oa) < TOL
    full16, full32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=np.zeros(m, np.int64),
                                    kv_len=np.full(m, L, np.int32))
    g = synth.f16_bits_to_f32(bits(out)).reshape(m, 64, 512)
    assert max_rel(g, full32) < TOL
    # oracle combine of the GPU partials gives the same
    c16, c32 = orc.lse_combine(pm.cpu().numpy(), pl.cpu().numpy(), pa.cpu().numpy(), S, rows)
    assert max_rel(g.reshape(rows, 512), c32) < 1e-3


def test_combine_edge_cases_and_pointer_variant():
    rows, S = 6, 4
    r = synth.rng(5)
    pm = r.standard_normal((S, rows), dtype=np.float32)
    pl = (1 + r.random((S, rows))).astype(np.float32)
    pa = r.standard_normal((S, rows, 512), dtype=np.float32)
    pm[:, 0] = -np.inf                    # a row where every split is empty -> zeros
    pm[1, 2] = -np.inf; pl[1, 2] = 0; pa[1, 2] = 0   # one empty split
    c16, c32 = orc.lse_combine(pm, pl, pa, S, rows)
    dm, dl, da = dev(pm), dev(pl), dev(pa)
    out = torch.empty(rows, 512, dtype=torch.float16, device="cuda")
    hk.lse_combine(dm, dl, da, S, rows, out)
    out2 = torch.empty_like(out)
    pm_ptrs = torch.tensor([dm[s].data_ptr() for s in range(S)], dtype=torch.int64, device="cuda")
    pl_ptrs = torch.tensor([dl[s].data_ptr() for s in range(S)], dtype=torch.int64, device="cuda")
    pa_ptrs = torch.tensor([da[s].data_ptr() for s in range(S)], dtype=torch.int64, device="cuda")
    hk.lse_combine_ptrs(pm_ptrs, pl_ptrs, pa_ptrs, S, rows, out2)
    torch.cuda.synchronize()
    g = synth.f16_bits_to_f32(bits(out))
    assert (g[0] == 0).all()
    assert max_rel(g, c32) < 1e-3
    assert np.array_equal(bits(out), bits(out2))


@pytest.mark.parametrize("m", [2, 131])
def test_absorbed_projections_vs_oracle(m):
    """tensor-core batched GEMMs (row tiles of 128: m = 131 leaves a ragged second tile) against the oracle;
    both weight layouts of the output projection"""
    r = synth.rng(9)
    qn = synth.f32_to_f16_bits(r.uniform(-1, 1, (m, 64, 256)).astype(np.float32))
    kb = synth.f32_to_f16_bits((0.3 * r.uniform(-1, 1, (32768, 512))).astype(np.float32))
    lo = synth.f32_to_f16_bits(r.uniform(-1, 1, (m, 64, 512)).astype(np.float32))
    dq, dkb, dlo = dev_f16(qn), dev_f16(kb), dev_f16(lo)
    ql = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    o1 = torch.empty(m, 64, 256, dtype=torch.float16, device="cuda")
    o2 = torch.empty_like(o1)
    wt = torch.empty(64, 512, 256, dtype=torch.float16, device="cuda")
    hk.q_latent(dq, dkb, ql, m)
    hk.o_absorb(dlo, dkb, o1, m)
    hk.wuv_transpose(dkb, wt)
    hk.o_absorb_t(dlo, wt, o2, m)
    torch.cuda.synchronize()
    f = synth.f16_bits_to_f32
    assert sum_rel(f(bits(ql)), f(orc.q_latent(qn, kb, m))) < 2e-3
    want_o = f(orc.o_absorb(lo, kb, m))
    assert sum_rel(f(bits(o1)), want_o) < 2e-3 and sum_rel(f(bits(o2)), want_o) < 2e-3


def test_peer_combine_on_one_gpu_and_bounded_wait_times_out_cleanly():
    """the cross-GPU combine path with every 'peer' on this GPU: flags set by hk_peer_signal release the
    wait; a slot that nothing sets makes the bounded wait expire - the kernel returns, the status word
    says so, the output is untouched and the context stays usable"""
    m, L, S = 1, 640, 2
    inp = synth.mla_inputs(L, m, seed=31, cache_std=0.5)
    rows = m * 64
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    pm = torch.empty(S, rows, dtype=torch.float32, device="cuda")
    pl = torch.empty(S, rows, dtype=torch.float32, device="cuda")
    pa = torch.empty(S, rows, 512, dtype=torch.float32, device="cuda")
    for s, (b, e) in enumerate([(0, 300), (300, L)]):
        hk.mla_dense_partial(q, c, dev(np.full(m, b, np.int64)), dev(np.full(m, e - b, np.int32)), 0, pm[s], pl[s], pa[s], m)
    flags = torch.zeros(S, dtype=torch.int32, device="cuda")
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")
    flag_ptrs = ptr([flags, flags])
    out = torch.full((rows, 512), 5.0, dtype=torch.float16, device="cuda")
    # only "rank 0" signals: slot 1 never arrives -> timeout after 50 ms, nothing written
    hk.peer_signal(flag_ptrs[:1], 1, 0, 1)
    hk.lse_combine_peers(ptr(list(pm)), ptr(list(pl)), ptr(list(pa)), S, rows, out, flags, 1, max_wait_ms=50)
    torch.cuda.synchronize()
    assert hk.read_device_status() == hk.HK_ERR_TIMEOUT
    assert (out == 5.0).all()
    # now both signal (as rank 0 and rank 1 of a 2-rank group whose flag arrays are this one array)
    hk.peer_signal(flag_ptrs, 2, 0, 2)
    hk.peer_signal(flag_ptrs, 2, 1, 2)
    hk.lse_combine_peers(ptr(list(pm)), ptr(list(pl)), ptr(list(pa)), S, rows, out, flags, 2, max_wait_ms=1000)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    _, full32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=np.zeros(m, np.int64),
                               kv_len=np.full(m, L, np.int32))
    assert max_rel(synth.f16_bits_to_f32(bits(out)).reshape(m, 64, 512), full32) < TOL


def test_enable_peer_access_is_idempotent_and_rejects_bad_devices():
    """own device: nothing to enable; a device index that does not exist: HK_ERR_INVALID; every other
    visible GPU: enabled (or already enabled), twice in a row"""
    cur = torch.cuda.current_device()
    hk.enable_peer_access(cur)
    with pytest.raises(Exception):
        hk.enable_peer_access(torch.cuda.device_count() + 3)
    for d in range(torch.cuda.device_count()):
        if d != cur and torch.cuda.can_device_access_peer(cur, d):
            hk.enable_peer_access(d)
            hk.enable_peer_access(d)


@pytest.mark.parametrize("m,L,n_split", [(1, 3000, 7), (2, 1111, 0), (1, 40, 1)])
def test_partial_with_local_splits_equals_one_split_partial(m, L, n_split):
    """hk_mla_dense_partial_ws: the splits over this GPU's SMs, merged on the GPU, give one partial set
    that normalises to the dense result (and to the oracle)"""
    inp = synth.mla_inputs(L, m, seed=33, cache_std=0.5)
    rows = m * 64
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    base, lens = dev(np.zeros(m, np.int64)), dev(np.full(m, L, np.int32))
    pm = torch.empty(rows, dtype=torch.float32, device="cuda")
    pl = torch.empty(rows, dtype=torch.float32, device="cuda")
    pa = torch.empty(rows, 512, dtype=torch.float32, device="cuda")
    hk.mla_dense_partial_ws(q, c, base, lens, 0, pm, pl, pa, m, L, n_split=n_split)
    out = torch.empty(rows, 512, dtype=torch.float16, device="cuda")
    hk.lse_combine(pm, pl, pa, 1, rows, out)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    full16, full32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=np.zeros(m, np.int64),
                                    kv_len=np.full(m, L, np.int32))
    g = synth.f16_bits_to_f32(bits(out)).reshape(m, 64, 512)
    assert max_rel(g, full32) < TOL


def test_exchange_region_alloc_view_and_free():
    """library-owned exchange region: zeroed, viewable as torch tensors, writable by kernels, freed"""
    region, handle = hk.peer_region_alloc(4096)
    assert len(handle) == 64 and region.data_ptr() % 256 == 0
    v = region.as_tensor(256, 1024, torch.float32)
    assert v.shape == (256,) and float(v.abs().sum()) == 0.0
    v.fill_(2.0)
    torch.cuda.synchronize()
    assert float(region.as_tensor(0, 4096, torch.uint8).float().sum()) > 0
    hk.peer_region_free(region)


def _planted_cache(L, m, seed, plant):
    """cache ~ N(0, 0.5) with keys planted as scaled copies of one head's query: (position, row, head, gain).
    A planted key's logit for its head is scale * gain * |q|^2 (about scale * gain * 512), far above
    the others' (about 0.7 sigma at scale 1/16), so the running maximum of that head jumps when the tile
    holding the planted key arrives."""
    inp = synth.mla_inputs(L, m, seed=seed, cache_std=0.5)
    ckv = synth.f16_bits_to_f32(inp["ckv"]).copy()
    q = synth.f16_bits_to_f32(inp["q_lat"])
    for pos, row, head, gain in plant:
        ckv[pos] = gain * q[row, head]
    inp["ckv"] = synth.f32_to_f16_bits(ckv)
    return inp


@pytest.mark.parametrize("n_split", [1, 3])
def test_dense_running_max_jumps_late_in_the_key_range(n_split):
    """peaked logits: several heads meet their (much larger) maximum many key tiles into the range, one of
    them twice with growing gains, so the accumulated output is rescaled in flight (jumps of 20+ log2 units)"""
    L, m = 1500, 2
    plant = [(700, 0, 3, 0.5), (1203, 0, 3, 1.0), (333, 0, 40, 0.6), (1450, 1, 63, 0.75), (97, 1, 0, 0.4),
             (610, 1, 17, 0.5)]
    inp = _planted_cache(L, m, 51, plant)
    base, lens = np.zeros(m, np.int64), np.full(m, L, np.int32)
    _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=base, kv_len=lens)
    out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(dev_f16(inp["q_lat"]), dev_f16(inp["ckv"]), out, m, 0, kv_base=dev(base), kv_len=dev(lens),
                         n_split=n_split, n_keys_hint=L)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    g = synth.f16_bits_to_f32(bits(out))
    assert max_rel(g, o32) < TOL and sum_rel(g, o32) < 3e-3
    # the planted heads are dominated by their planted key: a wrong rescale would show there first
    for _, row, head, _ in plant:
        assert max_rel(g[row, head], o32[row, head]) < TOL


@pytest.mark.parametrize("n_split", [1, 2])
def test_sparse_leading_tiles_fully_masked_and_late_maximum(n_split):
    """a gathered row whose first 100 indices are holes (two whole key tiles contribute nothing, the first live
    key arrives at tile 2) plus a planted maximum near the end; a second row that is live from the start"""
    T, m, kidx = 4096, 2, 400
    plant = [(3000, 0, 7, 0.6), (3001, 0, 50, 0.9), (123, 1, 9, 0.5)]
    inp = _planted_cache(T, m, 52, plant)
    r = np.random.RandomState(5)
    ridx = r.randint(0, T, (m, kidx)).astype(np.int32)
    ridx[0, :100] = -1
    ridx[0, 350] = 3000
    ridx[0, 390] = 3001
    ridx[1, 200] = 123
    ridx[1, 5::9] = -1
    _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, raw_idx=ridx, kidx=kidx)
    out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_sparse_decode(dev_f16(inp["q_lat"]), dev_f16(inp["ckv"]), dev(ridx), kidx, out, m, n_split=n_split)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    g = synth.f16_bits_to_f32(bits(out))
    assert max_rel(g, o32) < TOL and sum_rel(g, o32) < 3e-3
    for _, row, head, _ in plant:
        assert max_rel(g[row, head], o32[row, head]) < TOL


def test_dense_large_logit_scale():
    """cache ~ N(0, 4): logits of 10+ log2 units per sigma, maxima move by more than the lazy-rescale
    threshold in most tiles"""
    L, m = 2000, 1
    inp = synth.mla_inputs(L, m, seed=53, cache_std=4.0)
    base, lens = np.zeros(m, np.int64), np.full(m, L, np.int32)
    _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=base, kv_len=lens)
    for n_split in (1, 4):
        out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
        hk.mla_dense_prefill(dev_f16(inp["q_lat"]), dev_f16(inp["ckv"]), out, m, 0, kv_base=dev(base), kv_len=dev(lens),
                             n_split=n_split, n_keys_hint=L)
        torch.cuda.synchronize()
        assert hk.read_device_status() == 0
        g = synth.f16_bits_to_f32(bits(out))
        assert max_rel(g, o32) < TOL and sum_rel(g, o32) < 3e-3


def test_cache_row_count_bounds_gathered_and_dense_reads():
    """with the cache's row count given, gathered row numbers at or beyond it count as holes (nothing past the
    buffer is read) and a causal call that would run past the end is refused on the host"""
    T, m, kidx = 600, 2, 96
    inp = synth.mla_inputs(T, m, seed=61, cache_std=0.5)
    r = np.random.RandomState(3)
    ridx = r.randint(0, T, (m, kidx)).astype(np.int32)
    bad = ridx.copy()
    bad[:, 1::5] = T + r.randint(0, 1000, bad[:, 1::5].shape)        # beyond the cache
    holes = ridx.copy()
    holes[:, 1::5] = -1
    _, o32 = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, raw_idx=holes, kidx=kidx)
    q, c = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    for n_split in (1, 2):
        out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
        hk.mla_sparse_decode(q, c, dev(bad), kidx, out, m, n_split=n_split)        # ckv_rows = 600 from the tensor
        torch.cuda.synchronize()
        assert max_rel(synth.f16_bits_to_f32(bits(out)), o32) < TOL
    out = torch.empty(4, 64, 512, dtype=torch.float16, device="cuda")
    q4 = torch.zeros(4, 64, 512, dtype=torch.float16, device="cuda")
    with pytest.raises(hk.HeliosB200Error) as e:
        hk.mla_dense_prefill(q4, c, out, 4, T - 2)                                  # rows T-2 .. T+1 would be needed
    assert e.value.status == hk.HK_ERR_INVALID
    # per-row ranges are cut at the end of the cache on the device
    base, lens = np.array([T - 100, 0], dtype=np.int64), np.array([400, 50], dtype=np.int32)
    cut = np.array([100, 50], dtype=np.int32)
    _, o32d = orc.mla_attend(inp["q_lat"], inp["ckv"], m, 64, 0.0625, kv_base=base, kv_len=cut)
    out = torch.empty(m, 64, 512, dtype=torch.float16, device="cuda")
    hk.mla_dense_prefill(q, c, out, m, 0, kv_base=dev(base), kv_len=dev(lens), n_keys_hint=400)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    assert max_rel(synth.f16_bits_to_f32(bits(out)), o32d) < TOL


def test_split_decode_replayed_from_a_graph_sees_each_replays_partials():
    """The combine is a programmatic dependent of the partial kernel: in a replayed graph it must read the partials
    of THAT replay (the cache changes between replays), not lines of an earlier one."""
    B, L = 4, 2000
    inp = synth.mla_inputs(B * L, B, seed=31, cache_std=0.5)
    base, lens = dev((np.arange(B) * L).astype(np.int64)), dev(np.full(B, L, dtype=np.int32))
    q, ckv = dev_f16(inp["q_lat"]), dev_f16(inp["ckv"])
    out = torch.empty(B, 64, 512, dtype=torch.float16, device="cuda")
    run = lambda: hk.mla_dense_prefill(q, ckv, out, B, 0, kv_base=base, kv_len=lens, n_keys_hint=L)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        run()                                                   # scratch is sized before the capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
    torch.cuda.synchronize()
    for rep in range(3):
        ckv.copy_(torch.roll(ckv, 977 * (rep + 1), 0))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        got = out.clone()
        run()
        torch.cuda.synchronize()
        assert torch.equal(got, out), rep
    host = bits(ckv)
    o16, o32 = orc.mla_attend(inp["q_lat"], host, B, 64, 0.0625, kv_base=(np.arange(B) * L).astype(np.int64),
                              kv_len=np.full(B, L, dtype=np.int32))
    assert max_rel(synth.f16_bits_to_f32(bits(out)), o32) < TOL
