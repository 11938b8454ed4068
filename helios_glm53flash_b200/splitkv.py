"""Long-context MLA decode split over the GPUs of one node (split-KV), one process per GPU.

Rank g owns a contiguous slice of the latent cache.  Two forms of the exchange exist.  The default
("all") lets every rank read every rank's whole partial set (one exchange hop; the loads of all sets are
in flight together).  The other ("heads", needs 64 % world == 0) is ``hk_mla_splitkv_heads_step``: every
rank merges its local splits into one partial set in its exchange region and signals; rank g then
combines ONLY heads [g * 64 / world, (g + 1) * 64 / world) from all ranks' partial sets and stores the
fp16 rows into every rank's region; a last kernel waits for all slices and copies them to the caller's
tensor.  Its bytes over NVLink per rank and step are independent of the number of ranks, but it needs two
exchange hops; measured on 2 and 4 GPUs it is the slower one (78 / 275 us against 64 / 242 us per step
at batch 1 / 8 on 2 GPUs, 69 / 184 against 47 / 155 on 4).  A decode step of the "all" form is, on every rank:
  1. ``hk_mla_dense_partial`` over the local slice -> un-normalised (m, l, acc) partial in a buffer that
     every peer has mapped (CUDA inter-process handle opened by each peer on its own device; NVLink),
  2. ``hk_peer_signal``: store the step's epoch into this rank's slot of every rank's flag array,
  3. ``hk_lse_combine_peers``: bounded wait until all slots of the local flag array show the epoch,
     then read the G partial sets through their peer pointers (plain loads over NVLink) and write the
     normalised output.  Every rank ends up with the full [m, 64, 512] result.
There is no collective library call on the data path and nothing but plain peer loads and stores; torch.distributed is used once,
at set-up, to exchange the IPC handles.  Waits are bounded: a rank that never signals makes the
others' combine give up after ``max_wait_ms`` with HK_ERR_TIMEOUT in the device status word.

The SPARSE step of one sequence (``SplitKVDecoder(sparse=True).step_sparse``) splits the pooled indexer keys and the
cache rows by pools (``shard_pools``): every rank scores its own pools, ``hk_dsa_select_splitkv`` exchanges each rank's
512 best candidates and selects from them exactly what the one-GPU top-512 selects, ``hk_mla_splitkv_sparse_step``
attends the selected rows of the local slice and runs the exchange above.  Measured at 262,144 tokens on 2 GPUs:
59 us per step against 31 us for the one-GPU chain: the step is latency-bound on one GPU already, so this form is
for cache capacity, not for speed.
"""
import numpy as np

from . import synth

PARTIAL_FLOATS_PER_ROW = 2 + 512      # m, l, acc[512] per (row, head)


def shard_tokens(n_tokens, rank, world):
    """[begin, end) of the cache rows owned by `rank`; slices differ by at most one row"""
    return synth.shard_range(n_tokens, rank, world)


def shard_pools(n_tokens, rank, world):
    """sparse split-KV: [first pool, end pool) and [first row, end row) of `rank`.  The COMPLETE pools (4 tokens each)
    are split evenly; a rank's rows are those of its pools, and the last rank also owns the up to 3 tokens of the
    incomplete pool at the end (they are only ever reached through the 4-token tail of the selection)."""
    p0, p1 = synth.shard_range(n_tokens // 4, rank, world)
    return (p0, p1), (4 * p0, n_tokens if rank == world - 1 else 4 * p1)


def region_layout(rows, world, cand_bytes=0):
    """byte offsets inside one rank's exchange region: flags | (m | l | acc) x 2.  The partial sets are
    double buffered by step parity: a rank may already write step s+1 while a slower peer still reads
    step s; it cannot reach step s+2 before that peer has signalled s+1, i.e. has finished reading s."""
    assert world * 4 <= 256
    pad = ((rows * 4 + 255) // 256) * 256
    lay = {"flags": 0}
    off = 256
    for par in (0, 1):
        lay["m%d" % par] = off
        lay["l%d" % par] = off + pad
        lay["acc%d" % par] = off + 2 * pad
        off += 2 * pad + rows * 512 * 4
    lay["cand"] = off                     # candidate area of the sparse selection (hk_dsa_select_splitkv), if any
    lay["total"] = off + cand_bytes
    return lay


class SplitKVDecoder:
    """Owns the peer-mapped exchange region of this rank and the pointer tables of all ranks."""

    def __init__(self, m, n_heads=64, group=None, max_wait_ms=1000, form=None, sparse=False):
        import torch
        import torch.distributed as dist
        import helios_glm53flash_b200 as hk
        self.torch, self.dist, self.hk = torch, dist, hk
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.m, self.n_heads, self.rows = m, n_heads, m * n_heads
        self.max_wait_ms = max_wait_ms
        self.form = form or "all"
        if self.form == "heads" and not (n_heads == 64 and 64 % self.world == 0):
            raise ValueError("the heads form needs 64 heads and a rank count that divides 64")
        self.sparse = bool(sparse)
        if self.sparse and self.form != "all":
            raise ValueError("the sparse step uses the 'all' form of the exchange")
        self.lay = region_layout(self.rows, self.world,
                                 ((hk.dsa_select_region_bytes(m, self.world) + 255) // 256) * 256 if sparse else 0)
        if self.form == "heads":
            self.lay = {"total": hk.load_library().hk_splitkv_region_bytes(m, n_heads)}
        # The exchange region is library-owned device memory with an inter-process handle; every peer
        # opens the handle with ITS OWN device current, which is what makes the mapping usable by that
        # device's kernels (set-up only: torch.distributed carries the 64-byte handles).
        self.local, handle = hk.peer_region_alloc(self.lay["total"])
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (handle, torch.cuda.current_device()), group=group)
        self.peers = []
        for r, (h, dev_index) in enumerate(gathered):
            if r == self.rank:
                self.peers.append(self.local)
            else:
                hk.enable_peer_access(dev_index)
                self.peers.append(hk.peer_region_open(h, self.lay["total"]))
        bases = [p.data_ptr() for p in self.peers]
        self.step_ctr = torch.zeros(1, dtype=torch.int32, device="cuda")   # "all" form: step number, advanced on the device
        self.epoch = 0
        self.workspace = None
        if self.form == "heads":
            self.region_ptrs = torch.tensor(bases, dtype=torch.int64, device="cuda")
            torch.cuda.synchronize()
            dist.barrier(group=group)
            return

        def table(key):
            return torch.tensor([b + self.lay[key] for b in bases], dtype=torch.int64, device="cuda")

        self.flag_ptrs = table("flags")
        # pointer tables of both exchange sets, [set][rank]
        self.m_ptrs, self.l_ptrs, self.acc_ptrs = [torch.cat([table(k + str(par)) for par in (0, 1)]) for k in ("m", "l", "acc")]
        self._views()
        if self.sparse:
            self.cand_ptrs = table("cand")
            self.local_idx = torch.empty(m, 512, dtype=torch.int32, device="cuda")
            self.sel_pools = torch.full((m, 512), -1, dtype=torch.int32, device="cuda")
            self.raw_local = torch.full((m, 2052), -1, dtype=torch.int32, device="cuda")
            self.qpos_local = torch.empty(m, dtype=torch.int32, device="cuda")
            self.scores = None
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _views(self):
        t, lay, rows = self.torch, self.lay, self.rows
        self.flags = self.local.as_tensor(lay["flags"], 4 * self.world, t.int32)
        self.part_m = [self.local.as_tensor(lay["m%d" % par], rows * 4, t.float32) for par in (0, 1)]
        self.part_l = [self.local.as_tensor(lay["l%d" % par], rows * 4, t.float32) for par in (0, 1)]
        self.part_acc = [self.local.as_tensor(lay["acc%d" % par], rows * 2048, t.float32) for par in (0, 1)]

    def close(self):
        """unmap the peers' regions, then (after a barrier: nobody still has it open) free the own one"""
        self.torch.cuda.synchronize()
        for r, p in enumerate(self.peers):
            if r != self.rank and p is not None:
                self.hk.peer_region_close(p)
        self.peers = []
        self.dist.barrier(group=self.group)
        if self.local is not None:
            self.hk.peer_region_free(self.local)
            self.local = None

    def step(self, q_lat, ckv_shard, n_local_keys, out, scale, signal=True, kv_base=None):
        """one decode step; q_lat [m, 64, 512] f16 (same on every rank), ckv_shard = this rank's rows,
        out [m, 64, 512] f16.  Every query row attends n_local_keys rows of ckv_shard starting at row
        kv_base[row] (device int64 [m]; default 0: one sequence).  signal=False withholds this rank's flag
        (failure-injection in tests)."""
        import helios_glm53flash_b200 as hk
        t = self.torch
        self.epoch += 1
        if getattr(self, "_n_keys", None) != int(n_local_keys):
            self._n_keys = int(n_local_keys)
            self._zero_base = t.zeros(self.m, dtype=t.int64, device="cuda")
            self._lens = t.full((self.m,), self._n_keys, dtype=t.int32, device="cuda")
            self._n_split = hk.mla_auto_splits(self.m, max(1, self._n_keys))
            nbytes = hk.mla_partial_bytes(self._n_split, self.rows)
            self.workspace = t.empty(max(256, nbytes), dtype=t.uint8, device="cuda")
        if self.form == "heads":
            base = self._zero_base if kv_base is None else kv_base
            hk._call("hk_mla_splitkv_heads_step", hk._ptr(q_lat), hk._ptr(ckv_shard), hk._ptr(base), hk._ptr(self._lens),
                     self.m, self.n_heads, float(scale), self._n_split, self._n_keys, hk._ptr(self.workspace),
                     self.workspace.numel(), hk._ptr(self.region_ptrs), self.world, self.rank,
                     hk._c.c_void_p(self.local.data_ptr()), hk._ptr(out), int(self.max_wait_ms), int(bool(signal)),
                     hk._stream(None))
            return
        hk.mla_splitkv_step(q_lat, ckv_shard, self._zero_base if kv_base is None else kv_base, self._lens,
                            (self.part_m[0], self.part_l[0], self.part_acc[0]),
                            (self.part_m[1], self.part_l[1], self.part_acc[1]), self.m, self.n_heads, scale,
                            self._n_split, self._n_keys, self.workspace, self.flag_ptrs, self.m_ptrs, self.l_ptrs,
                            self.acc_ptrs, self.world, self.rank, self.step_ctr, self.flags, out,
                            max_wait_ms=self.max_wait_ms, signal=signal)


    def step_sparse(self, q_lat, q_idx, w, q_pos, pool_shard, pool_range, ckv_shard, row_range, out, scale, signal=True,
                    signal_candidates=True):
        """one SPARSE decode step of one sequence: q_lat [m, 64, 512] f16, q_idx [m, 32, 128] / w [m, 32] of the
        indexer, q_pos device int32 [m] (global positions); pool_shard [p1 - p0, 128] = this rank's pooled keys,
        pool_range = (p0, p1), ckv_shard = this rank's cache rows, row_range = (r0, r1) (see shard_pools).  Scores of
        the local pools -> selection across ranks (self.sel_pools holds the GLOBAL selection afterwards) -> attention
        over the selected rows of the local slice -> exchange and combine.  Every rank gets the full result."""
        import helios_glm53flash_b200 as hk
        t = self.torch
        (p0, p1), (r0, r1) = pool_range, row_range
        npl = p1 - p0
        self.epoch += 1
        stride = max(8, ((npl + 7) // 8) * 8)
        if self.scores is None or self.scores.shape[1] < stride:
            self.scores = t.empty(self.m, stride, dtype=t.float16, device="cuda")
        if self.workspace is None or getattr(self, "_n_keys", None) != -2052:
            self._n_keys = -2052
            self._n_split = hk.mla_auto_splits(self.m, 2052)
            self.workspace = t.empty(max(256, hk.mla_partial_bytes(self._n_split, self.rows)), dtype=t.uint8, device="cuda")
        if npl > 0:
            t.sub(q_pos, r0, out=self.qpos_local)
            hk.indexer_score(q_idx, pool_shard, w, self.qpos_local, self.scores, self.m, npl, score_stride=self.scores.shape[1])
        hk.dsa_select_splitkv(self.scores, self.scores.shape[1], npl, p0, self.local_idx, self.cand_ptrs,
                              self.local.data_ptr() + self.lay["cand"], self.world, self.rank, self.m, 512, q_pos, r0,
                              r1 - r0, self.sel_pools, self.raw_local, self.step_ctr, max_wait_ms=self.max_wait_ms,
                              signal=signal_candidates)
        hk.mla_splitkv_sparse_step(q_lat, ckv_shard, r1 - r0, self.raw_local, 2052,
                                   (self.part_m[0], self.part_l[0], self.part_acc[0]),
                                   (self.part_m[1], self.part_l[1], self.part_acc[1]), self.m, self.n_heads, scale,
                                   self._n_split, self.workspace, self.flag_ptrs, self.m_ptrs, self.l_ptrs, self.acc_ptrs,
                                   self.world, self.rank, self.step_ctr, self.flags, out, max_wait_ms=self.max_wait_ms,
                                   signal=signal)

    def resync(self):
        """After a step timed out (device status HK_ERR_TIMEOUT) the ranks are no longer in lock step and a slow peer
        may still read an exchange set: every rank calls this before stepping again.  Host barrier, flags and step
        counters back to zero, host barrier."""
        self.torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        if self.form == "heads":
            self.hk._call("hk_splitkv_region_reset", self.hk._c.c_void_p(self.local.data_ptr()), self.m, self.n_heads,
                          self.hk._stream(None))
        else:
            self.flags.zero_()
            self.step_ctr.zero_()
            if self.sparse:
                self.local.as_tensor(self.lay["cand"], 256, self.torch.int32).zero_()
        self.epoch = 0
        self.hk.read_device_status(reset=True)
        self.torch.cuda.synchronize()
        self.dist.barrier(group=self.group)


def merge_partials_numpy(parts):
    """host restatement of the combine, for the CPU multi-process test: parts = list of (m, l, acc)"""
    m = np.stack([p[0] for p in parts]).astype(np.float64)
    l_ = np.stack([p[1] for p in parts]).astype(np.float64)
    acc = np.stack([p[2] for p in parts]).astype(np.float64)
    gm = m.max(axis=0)
    w = np.where(np.isinf(m), 0.0, np.exp(m - np.where(np.isinf(gm), 0.0, gm)))
    gl = (w * l_).sum(axis=0)
    o = (w[..., None] * acc).sum(axis=0)
    return np.where(gl[:, None] > 0, o / np.maximum(gl[:, None], 1e-300), 0.0)
