"""GPU parity of the DSA indexer path (pooled keys, scores, top-k, expansion) through the C ABI."""
import numpy as np
import pytest
import torch

import hk_oracle as orc
import hk_ref as ref
from gpu_util import bits, dev, dev_bf16, dev_f16, sum_rel
import helios_glm53flash_b200 as hk
from helios_glm53flash_b200 import synth

pytestmark = pytest.mark.gpu
NEG_INF = 0xFC00


def _kpool_inputs(n_tok, seed=0):
    r = synth.rng(seed + 404)
    ik = synth.f32_to_f16_bits(r.uniform(-1, 1, (n_tok, 128)).astype(np.float32))
    ig = synth.f32_to_f16_bits((3 * r.uniform(-1, 1, (n_tok, 128))).astype(np.float32))
    ape = (2 * r.uniform(-1, 1, (4, 128))).astype(np.float32)
    return ik, ig, ape


def _gpu_kpool(ik, ig, ape, calls, raw_rows, npools, fn=None):
    fn = fn or hk.kpool_write
    dik, dig, dape = dev_f16(ik), dev_f16(ig), dev(ape)
    ring = torch.zeros(raw_rows, 256, dtype=torch.float16, device="cuda")
    pk = torch.zeros(npools, 128, dtype=torch.float16, device="cuda")
    for (src0, pos, n) in calls:
        fn(dik[src0:], dig[src0:], ring, raw_rows, pk, dape, pos, n)
    torch.cuda.synchronize()
    return bits(pk)


def _cpu_kpool(ik, ig, ape, calls, raw_rows, npools):
    ring = np.zeros((raw_rows, 256), dtype=np.uint16)
    pk = np.zeros((npools, 128), dtype=np.uint16)
    for (src0, pos, n) in calls:
        orc.kpool_write(np.ascontiguousarray(ik[src0:]), np.ascontiguousarray(ig[src0:]), ring, raw_rows, pk, ape, pos, n)
    return pk


def test_kpool_write_values_split_invariance_and_ring_wrap():
    """the three kpool cases of the reference's parity test (test_attn_parity.cpp:112-207)"""
    np_, tmax = 64, 256
    ik, ig, ape = _kpool_inputs(np_ * 4)
    full = [(0, 0, np_ * 4)]
    g = _gpu_kpool(ik, ig, ape, full, tmax, np_)
    o = _cpu_kpool(ik, ig, ape, full, tmax, np_)
    assert sum_rel(synth.f16_bits_to_f32(g), synth.f16_bits_to_f32(o)) < 2e-3
    assert (g != o).mean() < 0.02  # a few last-bit differences from the approximate exp at most
    # split invariance: 16 tokens as 1x16, 4x4, 16x1 calls are bit-identical
    base = _gpu_kpool(ik, ig, ape, [(0, 0, 16)], tmax, np_)
    by4 = _gpu_kpool(ik, ig, ape, [(i, i, 4) for i in range(0, 16, 4)], tmax, np_)
    by1 = _gpu_kpool(ik, ig, ape, [(i, i, 1) for i in range(16)], tmax, np_)
    assert np.array_equal(base, by4) and np.array_equal(base, by1)
    assert (base[:4] != 0).all()
    # ring wrap: positions 12..27 through a 20-row ring equal the full plane; earlier pools untouched
    plane = _gpu_kpool(ik, ig, ape, [(0, 12, 16)], tmax, np_)
    ring = _gpu_kpool(ik, ig, ape, [(0, 12, 16)], 20, np_)
    assert np.array_equal(plane, ring)
    assert (ring[:3] == 0).all() and (ring[3:7] != 0).any()
    if ref.available():
        r = _gpu_kpool(ik, ig, ape, full, tmax, np_, fn=ref.kpool_write)
        assert np.array_equal(g, r), "same arithmetic as the reference kernel"


def _score_case(m, npools, q_pos, bf16=False, seed=0):
    inp = synth.indexer_inputs(npools, m, seed=seed, bf16=bf16)
    cast = dev_bf16 if bf16 else dev_f16
    sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")
    hk.indexer_score(cast(inp["q_idx"]), cast(inp["pool_k"]), cast(inp["w"]), dev(q_pos), sc, m, npools)
    torch.cuda.synchronize()
    assert hk.read_device_status() == 0
    return inp, bits(sc)


@pytest.mark.parametrize("m,npools,bf16", [(1, 128, False), (2, 64, False), (3, 600, False), (48, 600, False),
                                           (1, 4096, True), (9, 1000, True), (1, 65536, False),
                                           (45, 1100, True), (37, 300, False), (130, 5000, False), (32, 129, False)])
def test_indexer_score_vs_oracle_and_reference(m, npools, bf16):
    q_pos = np.array([min(npools * 4 - 1, 900 + 37 * r) if m > 1 else npools * 4 - 1 for r in range(m)], dtype=np.int32)
    inp, g = _score_case(m, npools, q_pos, bf16, seed=m + npools)
    o16, o32 = orc.indexer_score(inp["q_idx"], inp["pool_k"], inp["w"], q_pos, m, npools, bf16=bf16, acc64=True)
    assert np.array_equal(g == NEG_INF, o16 == NEG_INF), "visibility mask must match exactly"
    fin = o16 != NEG_INF
    gv, ov = synth.f16_bits_to_f32(g)[fin], o32[fin]
    assert np.sum(np.abs(gv - ov)) / np.sum(np.abs(ov) + 1e-6) < 3e-3     # reference test criterion
    assert np.max(np.abs(gv - ov)) <= 4e-3 * max(1.0, np.max(np.abs(ov)) / 4)
    if ref.available() and not bf16:
        sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")
        ref.indexer_score(dev_f16(inp["q_idx"]), dev_f16(inp["pool_k"]), dev_f16(inp["w"]), dev(q_pos), sc, m, npools)
        torch.cuda.synchronize()
        r = bits(sc)
        assert np.array_equal(r == NEG_INF, g == NEG_INF)
        rv = synth.f16_bits_to_f32(r)[fin]
        # both round an fp32 sum to fp16: at most one fp16 ulp apart (summation order differs)
        assert np.max(np.abs(rv - gv)) <= 4e-3 * max(1.0, np.max(np.abs(ov)) / 4)
        assert (r != g).mean() < 0.2


def test_indexer_legacy_matches_tensor_core_kernel():
    m, npools = 5, 300
    q_pos = np.array([1199, 3, 500, 777, 64], dtype=np.int32)
    inp, g = _score_case(m, npools, q_pos)
    plane = np.ascontiguousarray(inp["pool_k"].reshape(npools, 128).T)  # [128][npools]
    sc = torch.empty(m, npools, dtype=torch.float16, device="cuda")
    hk.indexer_score_legacy(dev_f16(inp["q_idx"]), dev_f16(plane), dev_f16(inp["w"]), dev(q_pos), sc, m, npools, npools)
    torch.cuda.synchronize()
    leg = bits(sc)
    assert np.array_equal(leg == NEG_INF, g == NEG_INF)
    fin = g != NEG_INF
    assert np.max(np.abs(synth.f16_bits_to_f32(leg)[fin] - synth.f16_bits_to_f32(g)[fin])) <= 4e-3


def _topk_gpu(scores_bits, s_stride, R, T, k, k_pad, fn=None, offset=0):
    buf = torch.zeros(scores_bits.size + offset, dtype=torch.float16, device="cuda")
    buf[offset:] = dev_f16(scores_bits.reshape(-1))
    idx = torch.full((R, k_pad), -7, dtype=torch.int32, device="cuda")
    (fn or hk.dsa_topk)(buf[offset:], s_stride, idx, R, T, k, k_pad)
    torch.cuda.synchronize()
    return idx.cpu().numpy()


@pytest.mark.parametrize("R,T,k,k_pad,stride_pad,offset", [
    (4, 1000, 512, 512, 0, 0), (3, 513, 512, 512, 7, 0), (2, 511, 512, 512, 1, 0), (2, 65536, 512, 512, 0, 0),
    (1, 8, 512, 512, 0, 0), (5, 20000, 512, 520, 0, 3), (2, 4096, 1, 8, 0, 0), (2, 3000, 0, 16, 0, 0),
    (16, 16384, 512, 512, 0, 0), (16, 16392, 512, 512, 0, 0), (17, 16392, 512, 512, 0, 0), (40, 30000, 512, 512, 8, 0)])
def test_topk_bit_exact_vs_oracle_and_reference(R, T, k, k_pad, stride_pad, offset):
    r = synth.rng(R * 7 + T)
    s_stride = T + stride_pad
    sc = r.standard_normal((R, s_stride), dtype=np.float32)
    sc = np.round(sc * 8) / 8 if T > 600 else sc           # coarse values: many exact ties at the threshold
    sc[:, T // 2:] = np.where(r.random((R, s_stride - T // 2)) < 0.3, -np.inf, sc[:, T // 2:])
    if R > 1:
        sc[1, : max(1, T - 5)] = -np.inf                       # a row with fewer than k finite entries
    scb = synth.f32_to_f16_bits(sc)
    want = orc.dsa_topk(scb, s_stride, R, T, k, k_pad)
    got = _topk_gpu(scb, s_stride, R, T, k, k_pad, offset=offset)
    assert np.array_equal(got, want)
    if ref.available() and k > 0:
        refi = _topk_gpu(scb, s_stride, R, T, k, k_pad, fn=lambda *a: ref.dsa_topk(*a, t_seq=T), offset=offset)
        assert np.array_equal(refi, want), "oracle pinned to the reference's top-k (set, order, padding)"


def test_topk_selects_the_true_top_k():
    """independent of the oracle: the selection is a true top-k, above-threshold entries come out in
    ascending index order followed by the threshold ties in ascending index order"""
    R, T, k = 3, 5000, 512
    sc = synth.rng(77).standard_normal((R, T), dtype=np.float32)
    scb = synth.f32_to_f16_bits(sc)
    got = _topk_gpu(scb, T, R, T, k, k)
    vals = synth.f16_bits_to_f32(scb)
    for r_ in range(R):
        sel = got[r_]
        kth = np.sort(vals[r_])[-k]
        assert len(set(sel.tolist())) == k and vals[r_][sel].min() == kth
        above = sel[vals[r_][sel] > kth]
        ties = sel[vals[r_][sel] == kth]
        assert (np.diff(above) > 0).all() and (np.diff(ties) > 0).all()
        assert np.array_equal(sel, np.concatenate([above, ties]))
        assert len(above) == (vals[r_] > kth).sum()
        # ties are the FIRST ones by index
        assert np.array_equal(ties, np.nonzero(vals[r_] == kth)[0][: len(ties)])


@pytest.mark.parametrize("per_row", [True, False])
def test_pool_expand_exact(per_row):
    m = 4
    r = np.random.RandomState(7)
    pidx = np.where(np.arange(m * 512) % 7 == 0, -1, r.randint(0, 30, m * 512)).astype(np.int32).reshape(m, 512)
    q_pos = np.array([255, 100, 2, 119], dtype=np.int32)
    raw = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
    if per_row:
        hk.pool_expand_row(dev(pidx), dev(q_pos), raw, m)
        want = orc.pool_expand(pidx, q_pos, m)
    else:
        hk.pool_expand(dev(pidx), dev(q_pos), raw, m, 100)
        want = orc.pool_expand(pidx, None, m, cur_pos=100)
    torch.cuda.synchronize()
    assert np.array_equal(raw.cpu().numpy(), want)
    if ref.available():
        raw2 = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
        if per_row:
            ref.pool_expand_row(dev(pidx), dev(q_pos), raw2, m)
        else:
            ref.pool_expand(dev(pidx), dev(q_pos), raw2, m, 100)
        torch.cuda.synchronize()
        assert np.array_equal(raw2.cpu().numpy(), want)


@pytest.mark.parametrize("G,P,k", [(1, 3000, 512), (2, 3000, 512), (3, 1400, 512), (8, 9000, 512), (4, 1000, 200), (2, 300, 512)])
def test_selection_over_rank_slices_equals_whole_row_selection(G, P, k):
    """hk_dsa_select_splitkv with the ranks' regions driven in turn by one process (all publications first, then all
    selections: no kernel ever waits for one that has not been launched): the selected pools equal hk_dsa_topk over the
    whole row, and the expanded rows of the ranks' slices together equal hk_pool_expand of that selection."""
    from helios_glm53flash_b200 import splitkv
    m = 2
    r = synth.rng(G * 1000 + P)
    sc = np.round(r.standard_normal((m, P), dtype=np.float32) * 4) / 4            # coarse: many exact ties
    sc[:, P // 3:] = np.where(r.random((m, P - P // 3)) < 0.2, -np.inf, sc[:, P // 3:])
    n_tokens = 4 * P + 2
    q_pos = np.array([n_tokens - 1, 4 * (P // 2) + 1], dtype=np.int32)
    for row in range(m):
        sc[row, (q_pos[row] + 1) // 4:] = -np.inf                                   # pools not yet complete for the row
    scb = synth.f32_to_f16_bits(sc)
    want = _topk_gpu(scb, P, m, P, k, 512)
    raw_want = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
    hk.pool_expand_row(dev(want), dev(q_pos), raw_want, m)
    raw_want = raw_want.cpu().numpy()

    nbytes = hk.dsa_select_region_bytes(m, G)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(G)]
    bases = torch.tensor([x.data_ptr() for x in regions], dtype=torch.int64, device="cuda")
    ctr = torch.zeros(1, dtype=torch.int32, device="cuda")
    qp = dev(q_pos)
    for step in range(3):                                                          # both candidate sets get used
        state = []
        for g in range(G):
            (p0, p1), (r0, r1) = splitkv.shard_pools(n_tokens, g, G)
            stride = max(8, (p1 - p0 + 7) // 8 * 8)
            loc = np.full((m, stride), 0x7c00, dtype=np.uint16)                    # +inf beyond the slice: must not be read
            loc[:, :p1 - p0] = scb[:, p0:p1]
            st = dict(sc=dev_f16(loc), lidx=torch.empty(m, 512, dtype=torch.int32, device="cuda"),
                      sel=torch.full((m, 512), -9, dtype=torch.int32, device="cuda"),
                      raw=torch.full((m, 2052), -9, dtype=torch.int32, device="cuda"), p=(p0, p1), r=(r0, r1), stride=stride)
            state.append(st)
            hk.dsa_select_splitkv(st["sc"], stride, p1 - p0, p0, st["lidx"], bases, regions[g].data_ptr(), G, g, m, k, qp, r0,
                                  r1 - r0, st["sel"], st["raw"], ctr, phases=1)
        for g, st in enumerate(state):
            hk.dsa_select_splitkv(st["sc"], st["stride"], st["p"][1] - st["p"][0], st["p"][0], st["lidx"], bases,
                                  regions[g].data_ptr(), G, g, m, k, qp, st["r"][0], st["r"][1] - st["r"][0], st["sel"],
                                  st["raw"], ctr, phases=2)
        torch.cuda.synchronize()
        assert hk.read_device_status(reset=True) == 0
        merged = np.full((m, 2052), -1, dtype=np.int64)
        for g, st in enumerate(state):
            assert np.array_equal(st["sel"].cpu().numpy(), want), (step, g)
            raw = st["raw"].cpu().numpy().astype(np.int64)
            assert ((raw == -1) | ((raw >= 0) & (raw < st["r"][1] - st["r"][0]))).all()
            here = raw >= 0
            assert (merged[here] == -1).all()                                      # every row belongs to exactly one rank
            merged[here] = raw[here] + st["r"][0]
        assert np.array_equal(merged, raw_want), step
        ctr += 1                                                                   # what the partial exchange of the step does


@pytest.mark.parametrize("R,T,k", [(2, 65536, 512), (1, 20000, 512), (3, 5000, 512), (40, 700, 512), (2, 300, 512), (1, 4096, 77)])
def test_topk_with_expansion_equals_topk_then_expand(R, T, k):
    r = synth.rng(R + T)
    sc = np.round(r.standard_normal((R, T), dtype=np.float32) * 4) / 4
    sc[:, T // 2:] = np.where(r.random((R, T - T // 2)) < 0.3, -np.inf, sc[:, T // 2:])
    q_pos = np.array([4 * T - 1 - 5 * i for i in range(R)], dtype=np.int32)
    scores = dev_f16(synth.f32_to_f16_bits(sc))
    idx0 = torch.full((R, 512), -7, dtype=torch.int32, device="cuda")
    raw0 = torch.full((R, 2052), -7, dtype=torch.int32, device="cuda")
    hk.dsa_topk(scores, T, idx0, R, T, k, 512)
    hk.pool_expand_row(idx0, dev(q_pos), raw0, R)
    idx1, raw1 = torch.full_like(idx0, -9), torch.full_like(raw0, -9)
    hk.dsa_topk_expand(scores, T, idx1, raw1, dev(q_pos), R, T, k)
    torch.cuda.synchronize()
    assert torch.equal(idx0, idx1) and torch.equal(raw0, raw1)


@pytest.mark.parametrize("m,npools", [(1, 65536), (1, 5000), (3, 600), (8, 20000), (20, 3000), (40, 2500)])
def test_indexer_select_equals_the_three_call_chain_also_from_a_graph(m, npools):
    q_pos = np.array([npools * 4 - 1 - 9 * r for r in range(m)], dtype=np.int32)
    inp, _ = _score_case(m, npools, q_pos, False, seed=5 + m)
    qi, pk, w, qp = dev_f16(inp["q_idx"]), dev_f16(inp["pool_k"]), dev_f16(inp["w"]), dev(q_pos)
    sc0 = torch.empty(m, npools, dtype=torch.float16, device="cuda")
    idx0 = torch.empty(m, 512, dtype=torch.int32, device="cuda")
    raw0 = torch.empty(m, 2052, dtype=torch.int32, device="cuda")
    hk.indexer_score(qi, pk, w, qp, sc0, m, npools)
    hk.dsa_topk(sc0, npools, idx0, m, npools, min(512, npools), 512)
    hk.pool_expand_row(idx0, qp, raw0, m)
    sc1, idx1, raw1 = torch.empty_like(sc0), torch.full_like(idx0, -9), torch.full_like(raw0, -9)
    run = lambda: hk.indexer_select(qi, pk, w, qp, sc1, idx1, raw1, m, npools, k=min(512, npools))
    run()
    torch.cuda.synchronize()
    assert torch.equal(idx0, idx1) and torch.equal(raw0, raw1)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
    for rep in range(3):
        # other keys every replay: the selection kernel must see the scores of THIS replay
        pk.copy_(torch.roll(pk, 1 + rep, 0))
        idx1.fill_(-9)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        hk.indexer_score(qi, pk, w, qp, sc0, m, npools)
        hk.dsa_topk(sc0, npools, idx0, m, npools, min(512, npools), 512)
        hk.pool_expand_row(idx0, qp, raw0, m)
        torch.cuda.synchronize()
        assert torch.equal(idx0, idx1) and torch.equal(raw0, raw1), rep
    assert hk.read_device_status() == 0
