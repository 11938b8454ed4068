// Absorbed MLA flash attention over the 512-wide fp16 latent cache on the 5th-generation tensor
// cores: dense causal ranges and gathered (sparse) rows, decode and prefill rows, final output or
// split-KV partials.  One kernel serves helios::attn::mla_sparse_decode and
// helios::attn::mla_dense_prefill (reference: src/cuda/attn/attn.cu:394-699, scalar kernels, one
// block per (row, head) or head pair).
//
// Work item = (query row, key split) -> one CTA; all 64 heads of the row share every latent row that
// is staged, so the cache is read once per row (the reference re-reads it per head pair).
// Per tile of 48 keys (48 KB, three tiles in flight, invalid slots zero-filled):
//   S  [64 heads x 48 keys]  = Q  K^T   tcgen05 M64  N48 K512: Q and the tile both K-major
//   softmax: heads are TMEM lanes, keys are columns -> max / exp2 / sum run inside one thread; the
//            running reference max only moves when a tile exceeds it by 2^8 (lazy rescale of O)
//   O^T[512 ch x 64 heads] += V^T P^T   4 x tcgen05 M128 N64 K48: the SAME tile read MN-major as A
//            (the latent row is both key and value), P written K-major by the head threads
// The key tile sits in the 128-byte-swizzle layout: 8 blocks of 64 channels, each block = 48 key rows
// of 128 bytes with 16-byte chunk c of row r stored at c ^ (r % 8).  Read K-major (rows = keys) it is
// the B operand of Q K^T; the same bytes read MN-major (64 contiguous channels per key) are the A
// operand V^T.  Whole tiles of a dense range arrive with ONE TMA tensor copy each (3-D box
// {64 channels, 48 keys, 8 blocks} over the cache viewed as [row][block][64], 128-byte swizzle);
// gathered rows arrive as gather4 tensor copies (four cache rows x one 64-channel block each, 96 per tile; a separate
// instantiation of the kernel); ragged tails, and everything when the copy engine is not available, go through
// register-staged vector loads into the same layout.
//
// Warp roles (416 threads): warps 0-3 softmax + epilogue (one per TMEM lane quarter), warp 4 issues
// S = Q K^T, warp 12 issues O^T += V^T P^T (each as a converged warp with an elected lane, tc05.cuh),
// warps 5-11 stage the key tiles (the instantiation for gathered rows has 512 threads: warps 13-15 issue copies
// too).  S and P are double buffered, so QK^T of tile i+1 runs on the tensor
// pipe while tile i is in the softmax, and the copies of the next tiles are in flight during both.  The
// copies of the first three dense tiles leave at kernel entry; all warps stage the queries.  All
// hand-offs are mbarriers with bounded waits, executed by every lane of the waiting warp.
// HBM-bound by design: 1 KB per key for 128 K flops (128 flop/B), accumulators never leave TMEM.
#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime at first use)
#include <cuda_pipeline_primitives.h>

#include "mla_args.cuh"
#include <cstring>

#include "tc05.cuh"

namespace hk {

constexpr int FT_KEYS = 48;                       // keys per tile
constexpr int FT_NBUF = 3;                        // key tiles in flight
constexpr int FT_HEADS = 64;
constexpr int FT_THREADS = 416;                   // 4 softmax warps, QK^T issue warp, 7 loader warps, V^T P^T issue warp
constexpr int FT_LOAD_WARPS = 7;                  // warps 5-11
constexpr int FT_LOADERS = FT_LOAD_WARPS * 32;
constexpr int FT_ITEMS = (2 * FT_KEYS + FT_LOAD_WARPS - 1) / FT_LOAD_WARPS;   // half-rows per loader warp and tile
constexpr uint32_t FT_BLK = FT_KEYS * 128;        // one block of 64 channels: one 128-byte row per key
constexpr uint32_t FT_TILE = 8 * FT_BLK;          // 49152
constexpr uint32_t FQ_LBO = 128, FQ_SBO = 64 * 128;  // Q operand [64 heads][512] K-major
constexpr uint32_t FP_LBO = 128, FP_SBO = (FT_KEYS / 8) * 128;   // P operand [64 heads][keys] K-major
constexpr uint32_t FP_BYTES = FT_HEADS * FT_KEYS * 2;
constexpr uint32_t FS_Q = 0;                      // 65536
constexpr uint32_t FS_K = 65536;                  // FT_NBUF tiles, 1 KB aligned
constexpr uint32_t FS_P = FS_K + FT_NBUF * FT_TILE; // 2 x FP_BYTES
constexpr uint32_t FS_MISC = FS_P + 2 * FP_BYTES;  // alpha[2][64], m[64], l[64], masks, flags
constexpr uint32_t FS_SMEM = FS_MISC + 1536 + 1024;   // + slack to align the base to 1 KB (swizzle atoms)
#ifndef HK_FT_PF_AHEAD
#define HK_FT_PF_AHEAD 5
#endif
constexpr int FT_PF_AHEAD = HK_FT_PF_AHEAD;         // tiles between the L2 look-ahead prefetch and the tile being staged
constexpr int FT_POLL_NS = 40;                    // poll back-off of the waiting warps
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;         // log2 units: P stays below 2^8, fine for fp16

// Optional timeline instrumentation (diagnostic build, -DHK_DIAG): CTA (0,0) stamps clock64 at the
// hand-off points of its first 64 tiles; hk_debug_flash_trace copies the stamps to the host.
#ifdef HK_DIAG
__device__ long long hk_flash_trace[64 * 16];
__device__ unsigned long long hk_flash_cta[2 * 4096];   // per CTA: globaltimer at start and end
__device__ __forceinline__ unsigned long long ft_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FT_CTA_STAMP(which)                                                                       \
  do {                                                                                             \
    const unsigned cta = blockIdx.y * gridDim.x + blockIdx.x;                                      \
    if (threadIdx.x == 0 && cta < 4096) hk_flash_cta[2 * cta + (which)] = ft_globaltimer();        \
  } while (0)
#define FT_TRACE(slot, tile)                                                         \
  do {                                                                               \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (tile) < 64) hk_flash_trace[(tile) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define FT_TRACE(slot, tile) do { } while (0)
#define FT_CTA_STAMP(which) do { } while (0)
#endif

__device__ __forceinline__ void softmax_group_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void tma_load_tile(void* smem_dst, const CUtensorMap* tmap, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          tc::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(0), "r"(row), "r"(0), "r"(tc::smem_u32(bar))
      : "memory");
}

// Four gathered cache rows x one 64-channel block (4 x 128 B) in one tensor copy: the 2-D map covers the cache as
// [row][512 channels] with a box of {64 channels, 1 row}; the instruction names four row coordinates, the copy engine
// lays the four 128-byte pieces down one after the other and applies the 128-byte swizzle by destination address, i.e.
// exactly key slots k .. k+3 of a block of the tile layout.  A negative row is outside the tensor: zero fill.
__device__ __forceinline__ void tma_gather4_rows(void* smem_dst, const CUtensorMap* tmap, int channel, int r0, int r1, int r2,
                                                 int r3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(
          tc::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(channel), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(tc::smem_u32(bar))
      : "memory");
}

// The gather instantiation runs three more loader warps (warps 13-15): a warp gets one copy out per about 90 cycles
// whichever lanes issue them, so the 96 copies of a tile are spread over 10 warps x 10 lanes.
constexpr int FT_G4_THREADS = 512;
constexpr int FT_G4_WARPS = FT_LOAD_WARPS + 3;
constexpr int FT_G4_LANES = 10;
static_assert(FT_KEYS % 4 == 0 && FT_G4_WARPS * FT_G4_LANES >= (FT_KEYS / 4) * 8, "one gather4 per (key quad, block)");

// G4: gathered rows through the copy engine (use_tma == 2).  A separate instantiation: with both loaders in one
// kernel the dense paths lost 3-14 % (256-row dense prefill 1.55 -> 1.77 ms) to the register allocation of the whole.
template <bool G4>
__global__ __launch_bounds__(G4 ? FT_G4_THREADS : FT_THREADS, 1) void mla_flash_tc_kernel(MlaArgs a, int* __restrict__ status,
                                                                     const __grid_constant__ CUtensorMap tmap,
                                                                     int use_tma) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + FS_Q;
  float* s_alpha = reinterpret_cast<float*>(smem + FS_MISC);       // [2][64]
  float* s_m = s_alpha + 128;
  float* s_l = s_m + 64;
  unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(s_l + 64);  // [FT_NBUF]
  int* s_flag = reinterpret_cast<int*>(s_mask + 4);                // [2]
  // per key tile buffer: k_full (tile landed), t_done (its V^T P^T finished); per S / P buffer (two):
  // s_full, s_free, p_full
  __shared__ uint64_t k_full[FT_NBUF], t_done[FT_NBUF], s_full[2], s_free[2], p_full[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // provably warp-uniform flag: the branch into the tensor-core issue role stays converged for the compiler
  const int warp_u = tc::warp_index_uniform();
  const bool mma_warp = warp_u == 4 || warp_u == 12;   // 4 issues S = Q K^T, 12 issues O^T += V^T P^T
  const int sp = blockIdx.x, r = blockIdx.y;
  // a kernel launched as this grid's programmatic dependent (the LSE combine) may be placed from now on; it waits
  // for this grid's completion itself before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  FT_CTA_STAMP(0);
  if (tid == 0) FT_TRACE(13, 0);                      // kernel entry
  const bool sparse = a.raw_idx != nullptr;
  int n;
  int64_t base = 0;
  if (sparse) n = a.kidx;
  else {
    n = a.kv_len ? a.kv_len[r] : a.pos_start + r + 1;
    base = a.kv_base ? a.kv_base[r] : 0;
    if (a.ckv_rows > 0) n = (int)max((int64_t)0, min((int64_t)n, a.ckv_rows - base));   // never past the end of the cache
  }
  // gathered row numbers beyond the cache are holes
  auto in_cache = [&](int tk) -> int { return (a.ckv_rows > 0 && (int64_t)tk >= a.ckv_rows) ? -1 : tk; };
  // split boundaries on tile granularity
  const int tiles_total = (n + FT_KEYS - 1) / FT_KEYS;
  const int tiles_per = (tiles_total + a.n_split - 1) / a.n_split;
  const int k0 = min(n, sp * tiles_per * FT_KEYS), k1 = min(n, (sp + 1) * tiles_per * FT_KEYS);
  const int n_tiles = (k1 - k0 + FT_KEYS - 1) / FT_KEYS;
  // a tile goes through TMA when it is a whole tile of a dense range
  auto tile_is_tma = [&](int t) { return use_tma == 1 && !sparse && (k0 + (t + 1) * FT_KEYS <= k1); };

  if (tid == 0) {
#pragma unroll
    for (int b = 0; b < FT_NBUF; b++) {
      tc::mbar_init(&k_full[b], G4 ? FT_G4_WARPS * 32 : FT_LOADERS);
      tc::mbar_init(&t_done[b], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; b++) {
      tc::mbar_init(&s_full[b], 1);
      tc::mbar_init(&s_free[b], 128);
      tc::mbar_init(&p_full[b], 128);
      s_flag[b] = 0;
    }
    tc::mbar_fence_init();
    abort_flag = 0;
    // The copies of the first FT_NBUF dense tiles leave at once, from the thread that has just initialised their
    // barriers: they fly while the queries are staged below (measured before: 6 us from kernel entry to the first
    // tile copy at batch 8, the queries being loaded first in five dependent batches by the loader warps alone).
    // The byte count is raised without an arrival; the loader thread that owns the copies arrives like the others.
    for (int t = 0; t < FT_NBUF && t < n_tiles; t++) {
      if (tile_is_tma(t)) {
        tc::mbar_expect_tx(&k_full[t], FT_KEYS * LATENT * 2);
        tma_load_tile(smem + FS_K + t * FT_TILE, &tmap, (int)(base + k0 + t * FT_KEYS), &k_full[t]);
      }
    }
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);
  if (n_tiles > 0) {
    // Q [64 heads][512] -> K-major operand tile, staged by ALL warps with every load of a thread in flight at
    // once.  item = (head group, chunk quad); lanes = 8 heads x 4 chunks -> one 128-byte core matrix per octet
    constexpr int NW = (G4 ? FT_G4_THREADS : FT_THREADS) / 32, QI = (128 + NW - 1) / NW;
    const __half* q = a.q_lat + (size_t)r * FT_HEADS * LATENT;
    uint4 qs[QI];
#pragma unroll
    for (int u = 0; u < QI; u++) {
      const int it = warp + u * NW;
      if (it < 128) {
        const int hg = it >> 4, ch = (it & 15) * 4 + (lane >> 3), h = hg * 8 + (lane & 7);
        qs[u] = *reinterpret_cast<const uint4*>(q + (size_t)h * LATENT + ch * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < QI; u++) {
      const int it = warp + u * NW;
      if (it < 128) {
        const int hg = it >> 4, ch = (it & 15) * 4 + (lane >> 3);
        *reinterpret_cast<uint4*>(sQ + hg * FQ_SBO + ch * FQ_LBO + (lane & 7) * 16) = qs[u];
      }
    }
    tc::fence_async_smem();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;   // S: 2 x 64 columns; O^T: 4 x 64 columns
  bool ok = true;

  if (!mma_warp && warp >= 5) {   // warps 5-11 (and 13-15 of the gather instantiation)
    // =========================== loaders: the key tiles ===========================
    // Register-staged copies: every loader warp first issues all of its 16-byte loads of the NEXT
    // tile (they fly while the tensor pipe still owns the buffer), then waits for the buffer, then
    // stores.  Plain vector loads: the per-thread cp.async path sustains far fewer bytes in flight.
    const int lw = (G4 && warp >= 12) ? warp - 6 : warp - 5;
    uint4 stage[FT_ITEMS];
    // L2 prefetch of the tiles ahead keeps HBM busy while this CTA computes: the register-staged
    // loads below then hit L2.  Dense: one contiguous range per tile; sparse: one 1 KB row per lane.
    // Gathered rows: the look-ahead costs one bulk prefetch per row, and the unit that takes them serialises the 32
    // lanes of a warp (measured: about 4,000 cycles per 48-row tile in the warp that issues them).  That is worth it
    // when a CTA has only a few tiles and its rows come from HBM (decode: about two tiles per CTA); in long gathered
    // runs (prefill rows: 43 tiles per CTA, rows shared by many queries and mostly in L2) it was the largest part of
    // the tile period, so it is only done for short runs.
    const bool pf_rows = n_tiles <= 8 && !G4;
    auto prefetch_tile = [&](int t) {
      if (lw != 0 || t >= n_tiles) return;
      const int q0 = k0 + t * FT_KEYS;
      if (!sparse) {
        const int cnt = min(FT_KEYS, k1 - q0);
        if (lane == 0 && cnt > 0) tc::prefetch_l2(a.ckv + (size_t)(base + q0) * LATENT, (uint32_t)cnt * LATENT * 2);
      } else if (pf_rows) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int pp = q0 + half * 32 + lane;
          if (half * 32 + lane < FT_KEYS && pp < k1) {
            const int tk = in_cache(a.raw_idx[(size_t)r * a.kidx + pp]);
            if (tk >= 0) tc::prefetch_l2(a.ckv + (size_t)tk * LATENT, LATENT * 2);
          }
        }
      }
    };
#pragma unroll 1
    for (int t = FT_NBUF - 1; t < FT_PF_AHEAD; t++) prefetch_tile(t);   // (nothing for gathered rows through the copy engine)
    // Gathered rows through the copy engine: the row numbers a lane needs are fetched TWO tiles ahead with volatile
    // loads, so that they are issued where they stand and not moved down to their first use (the row list of a query
    // is read once, from HBM); range checks that need the value (in_cache) are applied when it is used.
    auto ld_idx = [&](int p) -> int {
      int v;
      asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(a.raw_idx + (size_t)r * a.kidx + p));
      return v;
    };
    auto item_index = [&](int tile_i, int j) -> int {      // row number of item j of this warp, -1 = hole
      const int it = lw + j * FT_LOAD_WARPS;
      const int p = k0 + tile_i * FT_KEYS + (it >> 1);
      return (sparse && tile_i < n_tiles && j < FT_ITEMS && it < 2 * FT_KEYS && p < k1) ? a.raw_idx[(size_t)r * a.kidx + p] : -1;
    };
    auto mask_index = [&](int tile_i, int half) -> int {   // warp 0: row number of key half*32 + lane
      const int p = k0 + tile_i * FT_KEYS + half * 32 + lane;
      return (sparse && lw == 0 && tile_i < n_tiles && half * 32 + lane < FT_KEYS && p < k1) ? (G4 ? ld_idx(p) : a.raw_idx[(size_t)r * a.kidx + p]) : -1;
    };
    if (G4) {
      // ---- gathered rows through the copy engine: 96 gather4 copies per tile, one per (key quad, 64-channel block),
      // issued by 14 lanes of each loader warp.  Nothing passes through registers or the load/store unit, whose
      // outstanding-request capacity held the register-staged path to about 13 B per cycle and SM. ----
      const int u = lw * FT_G4_LANES + lane;
      const bool issuer = lane < FT_G4_LANES && u < (FT_KEYS / 4) * 8;
      const int kq = u >> 3, blk = u & 7;
      auto quad_index = [&](int tile_i, int e) -> int {
        const int p = k0 + tile_i * FT_KEYS + kq * 4 + e;
        return (issuer && tile_i < n_tiles && p < k1) ? ld_idx(p) : -1;
      };
      int qa[4], qb[4];
#pragma unroll
      for (int e = 0; e < 4; e++) { qa[e] = quad_index(0, e); qb[e] = quad_index(1, e); }
      int mk0_n1 = mask_index(0, 0), mk1_n1 = mask_index(0, 1), mk0_n2 = mask_index(1, 0), mk1_n2 = mask_index(1, 1);
      for (int tile = 0; tile < n_tiles; tile++) {
        const int buf = tile % FT_NBUF;
        const int p0 = k0 + tile * FT_KEYS;
        int rows4[4];
#pragma unroll
        for (int e = 0; e < 4; e++) { rows4[e] = in_cache(qa[e]); qa[e] = qb[e]; qb[e] = quad_index(tile + 2, e); }
        const int mk0 = in_cache(mk0_n1), mk1 = in_cache(mk1_n1);
        mk0_n1 = mk0_n2; mk1_n1 = mk1_n2;
        mk0_n2 = mask_index(tile + 2, 0);
        mk1_n2 = mask_index(tile + 2, 1);
        unsigned long long mk = 0;
        if (lw == 0) {
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int p = p0 + half * 32 + lane;
            const bool v = half * 32 + lane < FT_KEYS && p < k1 && (half ? mk1 : mk0) >= 0;
            mk |= (unsigned long long)__ballot_sync(0xffffffffu, v) << (32 * half);
          }
        }
        if (tile >= FT_NBUF) ok = tc::mbar_wait<FT_POLL_NS>(&t_done[buf], ((tile - FT_NBUF) / FT_NBUF) & 1, &abort_flag, 5) && ok;
        if (tid == 160) FT_TRACE(0, tile);
        if (lw == 0 && lane == 0) s_mask[buf] = mk;
        if (issuer && ok) {
          tc::mbar_arrive_expect_tx(&k_full[buf], 4 * 128);
          tma_gather4_rows(smem + FS_K + buf * FT_TILE + blk * FT_BLK + kq * 4 * 128, &tmap, blk * 64,
                           rows4[0] < 0 ? -1 : rows4[0], rows4[1] < 0 ? -1 : rows4[1], rows4[2] < 0 ? -1 : rows4[2],
                           rows4[3] < 0 ? -1 : rows4[3], &k_full[buf]);
        } else {
          tc::mbar_arrive(&k_full[buf]);
        }
        if (tid == 160) FT_TRACE(1, tile);
      }
    } else {
    // (register-staged path: gathered rows only without the copy engine; row numbers one tile ahead, plain loads)
    int idx_next = item_index(0, lane), mk0_next = mask_index(0, 0), mk1_next = mask_index(0, 1);
    for (int tile = 0; tile < n_tiles; tile++) {
      const int buf = tile % FT_NBUF;
      const int p0 = k0 + tile * FT_KEYS;
      const bool via_tma = tile_is_tma(tile);
      prefetch_tile(tile + FT_PF_AHEAD);
      if (tid == 160 && tile >= 2) FT_TRACE(13, tile);   // look-ahead prefetch issued
      const int idx_cur = idx_next, mk0 = in_cache(mk0_next), mk1 = in_cache(mk1_next);
      idx_next = item_index(tile + 1, lane);
      mk0_next = mask_index(tile + 1, 0);
      mk1_next = mask_index(tile + 1, 1);
      // item = (key, half row): lane copies chunk half*32 + lane of that key's 1 KB latent row
      // (a tile that arrives as a tensor copy skips all of this: the loader warps' instructions compete with the
      // softmax warps for issue slots, and the kernel executes about 4 K warp instructions per tile as it is)
      if (!via_tma) {
#pragma unroll
        for (int j = 0; j < FT_ITEMS; j++) {
          const int it = lw + j * FT_LOAD_WARPS;
          stage[j] = make_uint4(0, 0, 0, 0);
          const int row_j = sparse ? in_cache(__shfl_sync(0xffffffffu, idx_cur, j)) : -1;
          if (it < 2 * FT_KEYS) {
            const int p = p0 + (it >> 1);
            int64_t tok = -1;
            if (p < k1) tok = sparse ? (int64_t)row_j : base + p;
            if (tok >= 0) stage[j] = ld_stream16(a.ckv + (size_t)tok * LATENT + ((it & 1) * 32 + lane) * 8);
          }
        }
      }
      if (tid == 160 && tile >= 2) FT_TRACE(14, tile);   // this tile's row loads issued
      unsigned long long mk = 0;                       // validity of the key slots of this tile
      if (lw == 0) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int p = p0 + half * 32 + lane;
          bool v = half * 32 + lane < FT_KEYS && p < k1;
          if (v && sparse) v = (half ? mk1 : mk0) >= 0;
          mk |= (unsigned long long)__ballot_sync(0xffffffffu, v) << (32 * half);
        }
      }
      if (tid == 160 && tile >= 2) FT_TRACE(15, tile);   // validity mask built
      if (tile >= FT_NBUF) ok = tc::mbar_wait<FT_POLL_NS>(&t_done[buf], ((tile - FT_NBUF) / FT_NBUF) & 1, &abort_flag, 5) && ok;
      if (tid == 160) FT_TRACE(0, tile);               // buffer free, stores start
      uint8_t* dst0 = smem + FS_K + buf * FT_TILE;
      if (!via_tma) {
#pragma unroll
        for (int j = 0; j < FT_ITEMS; j++) {
          const int it = lw + j * FT_LOAD_WARPS;
          if (it < 2 * FT_KEYS) {
            const int key = it >> 1, ch = (it & 1) * 32 + lane;
            *reinterpret_cast<uint4*>(dst0 + tc::sw128_off(key, ch, FT_BLK)) = stage[j];
          }
        }
      }
      if (lw == 0 && lane == 0) s_mask[buf] = mk;
      if (via_tma && lw == 0 && lane == 0) {
        // one thread arms the barrier with the byte count and fires the tensor copy; the other loader
        // threads just arrive, the phase completes when the 64 KB have landed
        if (tile >= FT_NBUF) {
          tc::mbar_arrive_expect_tx(&k_full[buf], FT_KEYS * LATENT * 2);
          tma_load_tile(dst0, &tmap, (int)(base + p0), &k_full[buf]);
        } else {
          tc::mbar_arrive(&k_full[buf]);               // this tile's copy left at kernel entry
        }
      } else {
        tc::fence_async_smem();
        tc::mbar_arrive(&k_full[buf]);
      }
      if (tid == 160) FT_TRACE(1, tile);               // tile published
    }
    }
  } else if (mma_warp) {
    // =========================== tensor-core issue (whole warp, one elected lane) ===========================
    // Every lane runs the loop, polls the barriers and computes the (warp-uniform) descriptors; the elected
    // lane alone issues.  See tc05.cuh: issued from a single diverged thread each MMA costs ~47 cycles of
    // operand moves, from a converged warp the M64 N48 products go out every ~29 cycles.
    {
      const uint32_t leader = tc::elect_one();
      // EVERY lane polls (one shared-memory request per warp either way).  A leader-only wait would split the
      // warp into two groups that run this loop at different times while the compiler, which sees only
      // warp-uniform branch conditions here, keeps loop state in per-warp uniform registers.
      auto wait_u = [&](uint64_t* bar, uint32_t parity, int code) {
        const bool done = tc::mbar_wait<FT_POLL_NS>(bar, parity, &abort_flag, code);
        return __all_sync(0xffffffffu, done) != 0;
      };
      const uint32_t q_addr = tc::smem_u32(sQ);
      const uint32_t idesc_s = tc::make_idesc(64, FT_KEYS, tc::FMT_F16, tc::FMT_F16, false, false);
      const uint32_t idesc_o = tc::make_idesc(128, FT_HEADS, tc::FMT_F16, tc::FMT_F16, true, false);
      auto gemm2 = [&](int t) {                        // O^T += V^T P^T of tile t
        const int b = t & 1, kb = t % FT_NBUF;
        const uint32_t k_addr = tc::smem_u32(smem + FS_K + kb * FT_TILE);
        const uint32_t p_addr = tc::smem_u32(smem + FS_P + b * FP_BYTES);
        // V^T: M = 128 channels = two 64-channel blocks (leading offset), K = keys in 8-row atoms of 1 KB
        const uint64_t ad0 = tc::make_sdesc_sw128(k_addr, FT_BLK, 1024);
        const uint64_t bd0 = tc::make_sdesc(p_addr, FP_LBO, FP_SBO);
#pragma unroll
        for (int mt = 0; mt < 4; mt++)
#pragma unroll
          for (int kk = 0; kk < FT_KEYS / 16; kk++)
            tc::mma_f16_if(leader, tO + mt * 64, tc::sdesc_advance(ad0, mt * 2 * FT_BLK + kk * 2048),
                           tc::sdesc_advance(bd0, kk * 2 * FP_LBO), idesc_o, t > 0 || kk > 0);
        tc::mma_commit_if(leader, &t_done[kb]);
      };
      // The two products have issuing warps of their own: S = Q K^T of tile t + 1 goes out as soon as its keys
      // have landed and the S buffer is free, whatever the state of tile t's softmax; O^T += V^T P^T of tile t
      // follows its P.  (One warp issuing both spent ~700 cycles per tile between its two waits.)
      if (warp_u == 4) {
        for (int tile = 0; tile < n_tiles; tile++) {
          const int b = tile & 1, kb = tile % FT_NBUF;
          if (leader) FT_TRACE(12, tile);              // waits for this tile's keys start
          ok = wait_u(&k_full[kb], (tile / FT_NBUF) & 1, 1) && ok;
          if (leader) FT_TRACE(2, tile);               // keys seen landed by the issuing warp
          if (tile >= 2) ok = wait_u(&s_free[b], ((tile - 2) >> 1) & 1, 2) && ok;
          tc::fence_after_sync();
          if (leader) FT_TRACE(3, tile);               // operands ready, QK^T issue starts
          const uint32_t k_addr = tc::smem_u32(smem + FS_K + kb * FT_TILE);
          const uint64_t ad0 = tc::make_sdesc(q_addr, FQ_LBO, FQ_SBO);
          // keys as N in 1 KB atoms; 16 channels = 32 B inside the 128-byte row, 64 channels per block
          const uint64_t bd0 = tc::make_sdesc_sw128(k_addr, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < LATENT / 16; kk++)     // S = Q K^T
            tc::mma_f16_if(leader, tS + b * 64, tc::sdesc_advance(ad0, kk * 2 * FQ_LBO),
                           tc::sdesc_advance(bd0, (kk >> 2) * FT_BLK + (kk & 3) * 32), idesc_s, kk > 0);
          tc::mma_commit_if(leader, &s_full[b]);
          if (leader) FT_TRACE(4, tile);               // QK^T issued
        }
      } else {
        for (int tile = 0; tile < n_tiles; tile++) {
          ok = wait_u(&p_full[tile & 1], (tile >> 1) & 1, 3) && ok;
          tc::fence_after_sync();
          if (leader) FT_TRACE(5, tile);               // P ready
          gemm2(tile);
          if (leader) FT_TRACE(6, tile);               // V^T P^T issued
        }
      }
    }
  } else {
    // =========================== softmax warps ===========================
    // The S accumulator (M = 64) keeps head 16w + i in TMEM lane 32w + i, i < 16.  It is read with the
    // 16x256b shape so that all 32 lanes work: thread t owns heads hA = 16w + t/4 and hB = hA + 8 and,
    // of every 8 keys, keys 2(t%4) and 2(t%4)+1; the four threads of a quad share their row maxima by
    // shuffle and keep partial row sums that are added up once at the end.
    const float sc2 = a.scale * LOG2E;
    const int quad = lane & 3;
    const int hA = warp * 16 + (lane >> 2), hB = hA + 8;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    for (int tile = 0; tile < n_tiles; tile++) {
      const int b = tile & 1, kb = tile % FT_NBUF;
      ok = tc::mbar_wait<FT_POLL_NS>(&k_full[kb], (tile / FT_NBUF) & 1, &abort_flag, 6) && ok;   // makes the tile's mask visible
      ok = tc::mbar_wait<FT_POLL_NS>(&s_full[b], (tile >> 1) & 1, &abort_flag, 7) && ok;
      tc::fence_after_sync();
      if (tid == 0) FT_TRACE(7, tile);                 // S ready
      uint32_t sv[FT_KEYS / 2];
      static_assert(FT_KEYS == 48, "the S read below is 32 + 16 columns");
      tc::tmem_ld_16x256b_x4(tS + b * 64 + ((uint32_t)(warp * 32) << 16), sv);
      tc::tmem_ld_16x256b_x2(tS + b * 64 + 32 + ((uint32_t)(warp * 32) << 16), sv + 16);
      tc::tmem_ld_wait();
      tc::fence_before_sync();
      tc::mbar_arrive(&s_free[b]);
      const unsigned long long mask = s_mask[kb] >> (2 * quad);
      float tA = -INFINITY, tB = -INFINITY;
#pragma unroll
      for (int j = 0; j < FT_KEYS / 8; j++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const bool valid = (mask >> (8 * j + e)) & 1ull;
          const float vA = valid ? __uint_as_float(sv[4 * j + e]) * sc2 : -INFINITY;
          const float vB = valid ? __uint_as_float(sv[4 * j + 2 + e]) * sc2 : -INFINITY;
          sv[4 * j + e] = __float_as_uint(vA);
          sv[4 * j + 2 + e] = __float_as_uint(vB);
          tA = fmaxf(tA, vA);
          tB = fmaxf(tB, vB);
        }
      }
      tA = fmaxf(tA, __shfl_xor_sync(0xffffffffu, tA, 1)); tA = fmaxf(tA, __shfl_xor_sync(0xffffffffu, tA, 2));
      tB = fmaxf(tB, __shfl_xor_sync(0xffffffffu, tB, 1)); tB = fmaxf(tB, __shfl_xor_sync(0xffffffffu, tB, 2));
      float alA = 1.f, alB = 1.f;
      bool moved = false;
      if (tA > mA + RESCALE_THRESHOLD || (mA == -INFINITY && tA > -INFINITY)) {
        alA = (mA == -INFINITY) ? 0.f : exp2f(mA - tA);
        mA = tA; lA *= alA; moved = true;
      }
      if (tB > mB + RESCALE_THRESHOLD || (mB == -INFINITY && tB > -INFINITY)) {
        alB = (mB == -INFINITY) ? 0.f : exp2f(mB - tB);
        mB = tB; lB *= alB; moved = true;
      }
      if (quad == 0) {
        s_alpha[b * 64 + hA] = alA;
        s_alpha[b * 64 + hB] = alB;
        if (moved && tile > 0) s_flag[b] = tile + 1;   // stamped with the tile: never needs a reset
      }
      if (tid == 0) FT_TRACE(8, tile);                 // max done
      softmax_group_sync();
      if (tid == 0) FT_TRACE(9, tile);                 // group barrier passed
      const bool rescale = s_flag[b] == tile + 1;
      if (rescale) {
        // rare: a head's reference max moved.  O^T (columns = heads) is rescaled after the previous
        // tile's V^T P^T has completed and before this tile's is issued (it waits for p_full below).
        ok = tc::mbar_wait<FT_POLL_NS>(&t_done[(tile - 1) % FT_NBUF], ((tile - 1) / FT_NBUF) & 1, &abort_flag, 8) && ok;
        tc::fence_after_sync();
#pragma unroll 1
        for (int mt = 0; mt < 4; mt++) {
#pragma unroll 1
          for (int c0 = 0; c0 < FT_HEADS; c0 += 32) {
            uint32_t o[32];
            const uint32_t addr = tO + mt * 64 + c0 + ((uint32_t)(warp * 32) << 16);
            tc::tmem_ld32(addr, o);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * s_alpha[b * 64 + c0 + j]);
            tc::tmem_st32(addr, o);
          }
        }
        tc::tmem_st_wait();
      }
      // the P buffer of this parity was last read by the V^T P^T of tile-2
      if (tile >= 2) ok = tc::mbar_wait<FT_POLL_NS>(&t_done[(tile - 2) % FT_NBUF], ((tile - 2) / FT_NBUF) & 1, &abort_flag, 9) && ok;
      // P operand [64 heads][64 keys] K-major: chunk j of a head's row holds keys 8j..8j+7; this thread
      // writes its two keys (4 bytes) of every chunk, for both of its heads
      uint8_t* pA = smem + FS_P + b * FP_BYTES + (hA >> 3) * FP_SBO + (hA & 7) * 16 + quad * 4;
      uint8_t* pB = smem + FS_P + b * FP_BYTES + (hB >> 3) * FP_SBO + (hB & 7) * 16 + quad * 4;
      const bool liveA = mA != -INFINITY, liveB = mB != -INFINITY;
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int j = 0; j < FT_KEYS / 8; j++) {
        const float a0 = liveA ? exp2f(__uint_as_float(sv[4 * j]) - mA) : 0.f;
        const float a1 = liveA ? exp2f(__uint_as_float(sv[4 * j + 1]) - mA) : 0.f;
        const float b0 = liveB ? exp2f(__uint_as_float(sv[4 * j + 2]) - mB) : 0.f;
        const float b1 = liveB ? exp2f(__uint_as_float(sv[4 * j + 3]) - mB) : 0.f;
        sumA += a0 + a1;
        sumB += b0 + b1;
        __half2 ha = __floats2half2_rn(a0, a1), hb = __floats2half2_rn(b0, b1);
        *reinterpret_cast<uint32_t*>(pA + j * FP_LBO) = *reinterpret_cast<uint32_t*>(&ha);
        *reinterpret_cast<uint32_t*>(pB + j * FP_LBO) = *reinterpret_cast<uint32_t*>(&hb);
      }
      lA += sumA;
      lB += sumB;
      if (tid == 0) FT_TRACE(10, tile);                // P written
      tc::fence_async_smem();
      tc::fence_before_sync();
      tc::mbar_arrive(&p_full[b]);
      if (tid == 0) FT_TRACE(11, tile);                // P published
    }
    // per-head totals: add the partial row sums of the four threads of each quad
    lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (quad == 0) {
      s_m[hA] = mA; s_l[hA] = lA;
      s_m[hB] = mB; s_l[hB] = lB;
    }
    // ---- epilogue (softmax warps): wait for the last V^T P^T, then write the result ----
    if (tid == 0) FT_TRACE(14, 0);                    // softmax loop done
    if (n_tiles > 0) ok = tc::mbar_wait<FT_POLL_NS>(&t_done[(n_tiles - 1) % FT_NBUF], ((n_tiles - 1) / FT_NBUF) & 1, &abort_flag, 10) && ok;
    tc::fence_after_sync();
    softmax_group_sync();
    if (tid == 0) FT_TRACE(15, 0);                    // last V^T P^T complete, write-out starts
    const size_t rows = (size_t)a.m * FT_HEADS;
    const size_t rh0 = (size_t)r * FT_HEADS;
    if (ok && !abort_flag) {
#pragma unroll 1
      for (int mt = 0; mt < 4; mt++) {
        const int ch = mt * 128 + tid;   // TMEM lane = channel inside the M tile
#pragma unroll 1
        for (int c0 = 0; c0 < FT_HEADS; c0 += 32) {
          uint32_t o[32];
          if (n_tiles > 0) {
            tc::tmem_ld32(tO + mt * 64 + c0 + ((uint32_t)(warp * 32) << 16), o);
            tc::tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) o[j] = 0u;
          }
          if (a.out) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const float l = s_l[c0 + j];
              const float v = l > 0.f ? __uint_as_float(o[j]) / l : 0.f;
              a.out[(rh0 + c0 + j) * LATENT + ch] = __float2half_rn(v);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
              a.part_acc[((size_t)sp * rows + rh0 + c0 + j) * LATENT + ch] = s_l[c0 + j] > 0.f ? __uint_as_float(o[j]) : 0.f;
          }
        }
      }
      if (!a.out && tid < FT_HEADS) {
        const float mr = s_m[tid];
        a.part_m[(size_t)sp * rows + rh0 + tid] = (mr == -INFINITY || !(s_l[tid] > 0.f)) ? -INFINITY : mr / LOG2E;
        a.part_l[(size_t)sp * rows + rh0 + tid] = s_l[tid];
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0) FT_TRACE(13, 1);                      // all roles done
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
  FT_CTA_STAMP(1);
}

#ifdef HK_DIAG
}  // namespace hk
extern "C" __attribute__((visibility("default"))) int hk_debug_flash_trace(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, hk::hk_flash_trace, sizeof(long long) * 64 * 16) == cudaSuccess ? 0 : 3;
}
extern "C" __attribute__((visibility("default"))) int hk_debug_flash_cta(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, hk::hk_flash_cta, sizeof(unsigned long long) * 2 * 4096) == cudaSuccess ? 0 : 3;
}
namespace hk {
#endif

int mla_flash_tc_auto_splits(int m, int n_keys) {
  // at most one CTA per SM (a second wave would double the time), at least two 64-key tiles per
  // split, splits of equal tile counts
  const int sms = sm_count();
  const int tiles = (n_keys + FT_KEYS - 1) / FT_KEYS;
  int want = sms / (m > 0 ? m : 1);
  if (want > 256) want = 256;
  if (want < 1) want = 1;
  int tiles_per = (tiles + want - 1) / want;
  if (tiles_per < 2) tiles_per = 2;
  int n_split = (tiles + tiles_per - 1) / tiles_per;
  return n_split < 1 ? 1 : n_split;
}

int mla_flash_tc_launch(const MlaArgs& a, cudaStream_t s) {
  if (a.n_heads != FT_HEADS) return HK_ERR_UNSUPPORTED;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(mla_flash_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FS_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(mla_flash_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FS_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  // tensor map over the latent cache for the dense path: [row][block 8][64 x fp16]; the row extent is the cache's
  // row count when the caller gave it (the copy engine then zero-fills anything past the end), else an upper bound
  alignas(64) CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  int use_tma = 0;
  static const bool tma_disabled = getenv("HK_MLA_NO_TMA") != nullptr;   // debug switch: vector-load path only
  if (!tma_disabled) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
          qres == cudaDriverEntryPointSuccess)
        encode = (EncodeFn)fn;
      looked_up = true;
    }
    if (encode && a.raw_idx) {
      // gathered rows: 2-D map [row][512 channels], box {64 channels, 1 row} for the four-row gather copies
      const cuuint64_t dims[2] = {LATENT, a.ckv_rows > 0 ? (cuuint64_t)a.ckv_rows : (cuuint64_t)1 << 31};
      const cuuint64_t strides[1] = {LATENT * 2};
      const cuuint32_t box[2] = {64, 1};
      const cuuint32_t estr[2] = {1, 1};
      if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.ckv, dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
        use_tma = 2;
    } else if (encode) {
      const cuuint64_t dims[3] = {64, a.ckv_rows > 0 ? (cuuint64_t)a.ckv_rows : (cuuint64_t)1 << 31, 8};
      const cuuint64_t strides[2] = {LATENT * 2, 128};
      const cuuint32_t box[3] = {64, FT_KEYS, 8};
      const cuuint32_t estr[3] = {1, 1, 1};
      if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void*)a.ckv, dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
        use_tma = 1;
    }
  }
  dim3 grid(a.n_split, a.m);
  if (use_tma == 2)
    mla_flash_tc_kernel<true><<<grid, FT_G4_THREADS, FS_SMEM, s>>>(a, device_status_ptr(), tmap, use_tma);
  else
    mla_flash_tc_kernel<false><<<grid, FT_THREADS, FS_SMEM, s>>>(a, device_status_ptr(), tmap, use_tma);
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

}  // namespace hk
