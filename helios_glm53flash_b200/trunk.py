"""The attention hot path of the whole hybrid trunk - KDA layers and MLA layers chained the way the engine's
layer loop calls them (Runner::run_chunk -> layer_step -> kda_layer / mla_layer, src/engine/runner.cpp:976-1061,
:389-511, :514-695 of the reference) - on synthetic projection outputs.

What the trunk owns per layer is exactly what the engine's Cache owns (src/engine/cache.hpp:24-39): for a KDA
layer the conv window [3*H*128][4] bf16 and the recurrent state [H][128][128] f32; for an MLA layer the latent
cache [cap][512] f16, the raw k|gate ring and the pooled-key plane [cap/4][128] f16.  Everything between the
attention kernels of the real model (EXL3 projections, routing, FFN) is out of scope: its outputs are replaced
by one set of seeded synthetic tensors per layer KIND that every layer of that kind consumes, so layers differ
by their state, not by their inputs.

Call order per chunk of n rows at position pos:
  KDA layer   cast + short conv (fp32 projection rows -> bf16 q|k|v)     hk_kda_cast_conv
              gated chunked prefill (gate preparation inside)            hk_kda_chunked_prefill_gated
              gated RMS norm                                              hk_gated_rms_norm
  (n == 1)    conv + recurrence in one launch, then the norm             hk_kda_decode_step
  MLA layer   RMS norm + append to the latent cache                      hk_mla_cache_append
              indexer key layer norm, ring write + pooling               hk_layernorm_f16, hk_kpool_write
              absorbed query projection                                  hk_q_latent
              per block of 1,024 rows: scores, top-512, expansion        hk_indexer_score, hk_dsa_topk, hk_pool_expand
              sparse attention over the selected latents                 hk_mla_sparse
              absorbed output projection                                 hk_o_absorb
`fused=False` runs the KDA layer as the reference's own call sequence instead (transpose+cast, gate, conv,
recurrence launcher), the form the unchanged engine would call.

There is no CPU path: the module drives libhelios_b200 only.
"""
from types import SimpleNamespace

import numpy as np

from . import synth

RING_EXTRA = 4          # ring rows = max_chunk + 4 (src/engine/cache.cpp:10-14)
IDX_BLOCK = 1024        # rows per indexer / top-k block (src/engine/runner.cpp:118, :615-627)
KIDX = 512 * 4 + 4      # selected pools x 4 tokens + 4 tail tokens


class TrunkAttention:
    """n_kda KDA layers and n_mla MLA layers of one sequence (or `batch` sequences for the KDA side; the MLA side
    of the reference is single-sequence, so sequences take turns through it, each with its own planes)."""

    def __init__(self, n_kda=34, n_mla=11, heads=32, batch=1, max_ctx=262144, max_chunk=4096, seed=0, fused=True,
                 keep_outputs=False):
        import torch
        import helios_glm53flash_b200 as hk
        self.torch, self.hk = torch, hk
        self.n_kda, self.n_mla, self.H, self.B = n_kda, n_mla, heads, batch
        self.cap, self.max_chunk, self.fused, self.keep = max_ctx, max_chunk, fused, keep_outputs
        self.D, self.dim = 128, 3 * heads * 128
        t, dev = torch, "cuda"
        r = synth.rng(seed + 900)
        H, D, dim, n, B = heads, 128, self.dim, max_chunk, batch

        def f32(shape, scale=1.0):
            return t.from_numpy((scale * r.standard_normal(shape, dtype=np.float32)).astype(np.float32)).to(dev)

        def f16(shape, scale=1.0):
            return f32(shape, scale).half()

        # ---- synthetic projection outputs of one chunk (shared by all layers of a kind) ----
        raw = synth.kda_raw_gates(n, H, D, seed=seed)
        self.kda_in = {
            "x32": f32((B, n, dim)), "f": t.from_numpy(np.broadcast_to(raw["f"], (B, n, H, D)).copy()).to(dev),
            "b": t.from_numpy(np.broadcast_to(raw["b"], (B, n, H)).copy()).to(dev),
            "dt_bias": t.from_numpy(raw["dt_bias"]).to(dev), "a_log": t.from_numpy(raw["a_log"]).to(dev),
            "lower_bound": raw["lower_bound"], "gate_out": f32((B * n * H, D)),
            "conv_w": f32((dim, 4), 0.1).to(t.bfloat16), "norm_w": t.ones(D, dtype=t.bfloat16, device=dev)}
        self.mla_in = {
            "kv_pre": f32((n, 512)), "ln_w": f16((512,), 0.05) + 1.0, "idx_k": f16((n, 128)), "idx_g": f16((n, 128)),
            "knorm_w": f16((128,), 0.05) + 1.0, "knorm_b": f16((128,), 0.05), "ape": f32((4, 128), 0.1),
            "q_nope": f16((n, 64, 256), 0.5), "q_idx": f16((n, 32, 128)), "w": f16((n, 32)),
            "kv_b": f16((64 * 512, 512), 0.04)}
        # ---- per-layer state: the engine's Cache planes ----
        self.conv_state = [t.zeros(B, dim, 4, dtype=t.bfloat16, device=dev) for _ in range(n_kda)]
        self.rec_state = [t.zeros(B, 1, H, D, D, dtype=t.float32, device=dev) for _ in range(n_kda)]
        self.ckv = [[t.zeros(max_ctx, 512, dtype=t.float16, device=dev) for _ in range(n_mla)] for _ in range(B)]
        self.pool = [[t.zeros(max_ctx // 4, 128, dtype=t.float16, device=dev) for _ in range(n_mla)] for _ in range(B)]
        self.ring_rows = max_chunk + RING_EXTRA
        self.ring = [[t.zeros(self.ring_rows, 256, dtype=t.float16, device=dev) for _ in range(n_mla)] for _ in range(B)]
        # ---- scratch shared by all layers (the engine's per-chunk work buffers) ----
        self.qkv = t.empty(B, n, dim, dtype=t.bfloat16, device=dev)
        self.mixed = None if fused else t.empty(B, dim, n, dtype=t.bfloat16, device=dev)
        self.gate = None if fused else t.empty(B, n, H, D, dtype=t.float32, device=dev)
        self.beta = None if fused else t.empty(B, n, H, dtype=t.bfloat16, device=dev)
        self.rec_out = t.empty(B, n, H, D, dtype=t.bfloat16, device=dev)
        self.kda_y = t.empty(B * n * H, D, dtype=t.float16, device=dev)
        self.kda_ws = t.empty(max(256, hk.kda_chunked_workspace_bytes(B, n, H)), dtype=t.uint8, device=dev)
        self.idx_kn = t.empty(n, 128, dtype=t.float16, device=dev)
        self.q_lat = t.empty(n, 64, 512, dtype=t.float16, device=dev)
        self.qpos = t.empty(n, dtype=t.int32, device=dev)
        self.scores = t.empty(min(n, IDX_BLOCK), max_ctx // 4, dtype=t.float16, device=dev)
        self.topk = t.empty(n, 512, dtype=t.int32, device=dev)
        self.raw_idx = t.empty(n, KIDX, dtype=t.int32, device=dev)
        self.lat_out = t.empty(n, 64, 512, dtype=t.float16, device=dev)
        self.o_abs = t.empty(n, 64, 256, dtype=t.float16, device=dev)
        self.sparse_ws = t.empty(256, dtype=t.uint8, device=dev)          # grown on demand (split partials of few-row calls)
        self.x16 = t.empty(B, dim, dtype=t.bfloat16, device=dev)          # a decoded token's pre-conv q|k|v
        self.kept = {}
        self.stage_ms = {}
        self._events = []
        self._dec = None                                                  # per-sequence decode buffers and streams (batch > 1)

    # ------------------------------------------------------------------------------------------
    def _mark(self, name):
        """CUDA-event stage marks (device time per stage, summed over layers, read by stage_shares)"""
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append((name, ev))

    def stage_shares(self):
        self.torch.cuda.synchronize()
        tot = {}
        for (n0, e0), (n1, e1) in zip(self._events[:-1], self._events[1:]):
            if n1 != "begin":
                tot[n1] = tot.get(n1, 0.0) + e0.elapsed_time(e1)
        self._events = []
        return tot

    def kda_layer(self, L, n, timed=False):
        hk, ki, B, H, D, dim = self.hk, self.kda_in, self.B, self.H, self.D, self.dim
        x32, f, b = ki["x32"][:, :n], ki["f"][:, :n], ki["b"][:, :n]
        if n != self.max_chunk:
            x32, f, b = x32.contiguous(), f.contiguous(), b.contiguous()
        qkv, rec = self.qkv.view(-1)[:B * n * dim].view(B, n, dim), self.rec_out.view(-1)[:B * n * H * D].view(B, n, H, D)
        if n == 1 and self.fused:
            # a decoded token: the whole layer (cast, gates, conv, recurrence, gated norm) is one launch
            y = self.kda_y[:B * H]
            hk.kda_decode_layer(x32.reshape(B, dim), self.conv_state[L], ki["conv_w"], None, f.reshape(B, H, D), b.reshape(B, H),
                                ki["dt_bias"], ki["a_log"], ki["lower_bound"], self.rec_state[L], rec, ki["norm_w"],
                                ki["gate_out"][:B * H], y, B, H, epsilon=1e-6, gate_act=1)
            if self.keep:
                self.kept.setdefault(("kda", L), []).append((rec.clone(), y.clone()))
            return
        elif self.fused:
            hk.kda_cast_conv(x32, self.conv_state[L], None, ki["conv_w"], None, qkv, B, dim, n, True)
            if timed:
                self._mark("kda_cast_conv")
            hk.kda_chunked_prefill_gated(qkv, f, b, ki["dt_bias"], ki["a_log"], ki["lower_bound"], self.rec_state[L], rec,
                                         B, n, H, workspace=self.kda_ws) if n >= 64 else self._short(qkv, f, b, L, rec, n)
        else:
            mixed = self.mixed.view(-1)[:B * dim * n].view(B, dim, n)
            gate = self.gate.view(-1)[:B * n * H * D].view(B, n, H, D)
            beta = self.beta.view(-1)[:B * n * H].view(B, n, H)
            for s in range(B):
                hk.kda_transpose_cast(mixed[s], x32[s], n, dim)
                hk.kda_gate(b[s], f[s], ki["dt_bias"], ki["a_log"], ki["lower_bound"], beta[s], gate[s], n, H, D)
            hk.cuda_causal_conv1d_update(mixed, self.conv_state[L], None, ki["conv_w"], None, qkv, B, dim, n, 4, 4, True, False)
            if timed:
                self._mark("kda_cast_conv")
            hk.cuda_recurrent_gated_delta_rule(qkv, gate, beta, self.rec_state[L], rec, B, n, H, H, D, D, 1, None, True, False,
                                               workspace=self.kda_ws)
        if timed:
            self._mark("kda_recurrence")
        y = self.kda_y[:B * n * H]
        hk.gated_rms_norm(rec, ki["norm_w"], y, ki["gate_out"][:B * n * H], B * n * H, D, 1e-6, gate_act=1)
        if timed:
            self._mark("kda_gated_norm")
        if self.keep:
            self.kept.setdefault(("kda", L), []).append((rec.clone(), y.clone()))

    def _decode_gate(self, f, b):
        """gate preparation of a single decoded token (glue::kda_gate), for the one-launch decode step"""
        t, ki, B, H, D = self.torch, self.kda_in, self.B, self.H, self.D
        if not hasattr(self, "_dg"):
            self._dg = (t.empty(B, H, D, dtype=t.float32, device="cuda"), t.empty(B, H, dtype=t.bfloat16, device="cuda"))
        g, beta = self._dg
        self.hk.kda_gate(b.reshape(B, H), f.reshape(B, H, D), ki["dt_bias"], ki["a_log"], ki["lower_bound"], beta, g, B, H, D)
        return g, beta

    def _short(self, qkv, f, b, L, rec, n):
        """rows below one chunk (decode through the unfused call sequence): gate, then the recurrence launcher"""
        t, ki, B, H, D = self.torch, self.kda_in, self.B, self.H, self.D
        g = t.empty(B, n, H, D, dtype=t.float32, device="cuda")
        beta = t.empty(B, n, H, dtype=t.bfloat16, device="cuda")
        for s in range(B):
            self.hk.kda_gate(b[s], f[s], ki["dt_bias"], ki["a_log"], ki["lower_bound"], beta[s], g[s], n, H, D)
        self.hk.cuda_recurrent_gated_delta_rule(qkv, g, beta, self.rec_state[L], rec, B, n, H, H, D, D, 1, None, True, False)

    def _decode_bufs(self):
        """one set of single-row work buffers and one stream per sequence, so that the sequences' MLA layers of a decode
        step can run side by side (their caches are separate; the shared work buffers of a chunk are not)"""
        if self._dec is None:
            t, hk = self.torch, self.hk
            ns = hk.mla_auto_splits(1, KIDX)
            self._dec = [SimpleNamespace(
                idx_kn=t.empty(1, 128, dtype=t.float16, device="cuda"), q_lat=t.empty(1, 64, 512, dtype=t.float16, device="cuda"),
                qpos=t.empty(1, dtype=t.int32, device="cuda"), scores=t.empty(1, self.scores.shape[1], dtype=t.float16, device="cuda"),
                topk=t.empty(1, 512, dtype=t.int32, device="cuda"), raw_idx=t.empty(1, KIDX, dtype=t.int32, device="cuda"),
                lat_out=t.empty(1, 64, 512, dtype=t.float16, device="cuda"), o_abs=t.empty(1, 64, 256, dtype=t.float16, device="cuda"),
                sparse_ws=t.empty(max(256, hk.mla_partial_bytes(ns, 64)), dtype=t.uint8, device="cuda"),
                stream=t.cuda.Stream()) for _ in range(self.B)]
        return self._dec

    def mla_layer(self, L, n, pos, seq=0, timed=False, bufs=None):
        hk, mi, t = self.hk, self.mla_in, self.torch
        ckv, pool, ring = self.ckv[seq][L], self.pool[seq][L], self.ring[seq][L]
        wb = self if bufs is None else bufs                    # work buffers: the chunk's shared ones, or this sequence's own
        if n == 1 and self.fused:
            # a decoded token: append, key layer norm, pooled-key write and the position in one launch
            hk.mla_decode_prologue(mi["kv_pre"][:1], mi["ln_w"], ckv, 1e-6, mi["idx_k"][:1], mi["knorm_w"], mi["knorm_b"],
                                   wb.idx_kn[:1], 1e-5, mi["idx_g"][:1], ring, self.ring_rows, pool, mi["ape"], pos,
                                   q_pos_out=wb.qpos[:1])
        else:
            hk.mla_cache_append(mi["kv_pre"][:n], mi["ln_w"], ckv, pos, n, 1e-6)
            hk.layernorm_f16(mi["idx_k"][:n], mi["knorm_w"], mi["knorm_b"], wb.idx_kn[:n], n, 128, 1e-5)
            hk.kpool_write(wb.idx_kn[:n], mi["idx_g"][:n], ring, self.ring_rows, pool, mi["ape"], pos, n)
            t.arange(pos, pos + n, dtype=t.int32, device="cuda", out=wb.qpos[:n])
        if timed:
            self._mark("mla_append_kpool")
        hk.q_latent(mi["q_nope"][:n], mi["kv_b"], wb.q_lat[:n], n)
        if timed:
            self._mark("mla_q_latent")
        npools = (pos + n) // 4
        ktop = min(512, npools)
        if n <= 8 and self.fused and npools > 0:
            # decode rows: scores, top-k and expansion as two launches
            sc = wb.scores.view(-1)[:n * npools].view(n, npools)
            hk.indexer_select(mi["q_idx"][:n], pool, mi["w"][:n], wb.qpos[:n], sc, wb.topk[:n], wb.raw_idx[:n], n, npools, k=ktop)
            blocks = ()
        else:
            blocks = range(0, n, IDX_BLOCK)
        for off in blocks:
            rows = min(IDX_BLOCK, n - off)
            if npools > 0:
                sc = wb.scores.view(-1)[:rows * npools].view(rows, npools)
                hk.indexer_score(mi["q_idx"][off:off + rows], pool, mi["w"][off:off + rows], wb.qpos[off:off + rows], sc, rows, npools)
                if timed:
                    self._mark("mla_indexer_score")
                hk.dsa_topk(sc, npools, wb.topk[off:off + rows], rows, npools, ktop, 512)
            else:
                wb.topk[off:off + rows].fill_(-1)
            if timed:
                self._mark("mla_topk")
            hk.pool_expand_row(wb.topk[off:off + rows], wb.qpos[off:off + rows], wb.raw_idx[off:off + rows], rows)
        if timed:
            self._mark("mla_expand")
        ns = hk.mla_auto_splits(n, KIDX)
        need = hk.mla_partial_bytes(ns, n * 64) if ns > 1 else 0
        if need > wb.sparse_ws.numel():
            wb.sparse_ws = t.empty(need, dtype=t.uint8, device="cuda")
        hk.mla_sparse_decode(wb.q_lat[:n], ckv, wb.raw_idx[:n], KIDX, wb.lat_out[:n], n, n_split=ns, workspace=wb.sparse_ws)
        if timed:
            self._mark("mla_sparse_attention")
        hk.o_absorb(wb.lat_out[:n], mi["kv_b"], wb.o_abs[:n], n)
        if timed:
            self._mark("mla_o_absorb")
        if self.keep:
            self.kept.setdefault(("mla", L, seq), []).append((pos, n, wb.topk[:n].clone(), wb.raw_idx[:n].clone(),
                                                              wb.lat_out[:n].clone(), wb.o_abs[:n].clone()))

    def run_chunk(self, pos, n, timed=False):
        """all layers over rows pos .. pos + n - 1 (prefill chunk, or a decode step with n = 1).  The model interleaves
        the two kinds (three KDA layers, then one MLA layer); with synthetic inputs the order inside a chunk does not
        change any result, so the layers run kind by kind."""
        if timed:
            self._mark("begin")
        for L in range(self.n_kda):
            self.kda_layer(L, n, timed)
        if n == 1 and self.B > 1 and self.fused and not timed:
            # a decode step of several sequences: their MLA layers touch separate caches, so every sequence gets a stream
            # and single-row work buffers of its own and the chains run side by side (also inside a captured graph)
            t = self.torch
            cur = t.cuda.current_stream()
            for seq, bufs in enumerate(self._decode_bufs()):
                bufs.stream.wait_stream(cur)
                with t.cuda.stream(bufs.stream):
                    for L in range(self.n_mla):
                        self.mla_layer(L, n, pos, seq, False, bufs)
            for bufs in self._dec:
                cur.wait_stream(bufs.stream)
            return
        for seq in range(self.B):
            for L in range(self.n_mla):
                self.mla_layer(L, n, pos, seq, timed)

    def prefill(self, n_tokens, chunk=None, timed=False):
        chunk = chunk or self.max_chunk
        pos = 0
        while pos < n_tokens:
            n = min(chunk, n_tokens - pos)
            self.run_chunk(pos, n, timed)
            pos += n
        return pos
