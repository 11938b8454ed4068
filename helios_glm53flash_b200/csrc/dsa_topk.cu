// Exact top-k selection over fp16 score rows for the DSA indexer.
// Interface and output contract of helios::aux::dsa_topk (reference: src/cuda/aux/dsa_topk.cu:73-273,
// :668-732): on the order-preserving 16-bit key of the fp16 bit pattern (:21-24) find the k-th
// largest value v*; emit every entry above v* in ascending index order, then entries equal to v*
// in ascending index order until k are out; -inf (and anything below it) is never selected; if a
// row holds fewer than k selectable entries all of them are emitted; the rest of the k_pad-wide
// output row is -1.  Integer work: results are bit-exact by construction.
//
// One CTA of 1024 threads per row, three sweeps of the row (the reference makes four: two
// histogram sweeps and two compaction sweeps).  Sweep 1 histograms the top 11 key bits, sweep 2 the
// low 5 bits inside the crossing bucket, sweep 3 is a single ordered compaction that places the
// "above" entries and the tie entries at once (their final offsets are known after sweep 2).
#include <cooperative_groups.h>

#include "hk_common.cuh"

namespace hk {

constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr uint32_t KEY_NEG_INF = 0x03ffu;  // key of fp16 -inf (0xfc00)

__device__ __forceinline__ uint32_t topk_key(uint32_t u16) {
  return (u16 & 0x8000u) ? (~u16 & 0xffffu) : (u16 | 0x8000u);
}

// Exclusive block scan of one int per thread; returns the exclusive prefix, *total = block sum.
// `scratch` holds TK_WARPS + 1 ints.  Contains two barriers.
__device__ __forceinline__ int block_exscan(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int wv = scratch[lane];
    int wi = wv;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    scratch[lane] = wi - wv;
    if (lane == 31) scratch[TK_WARPS] = wi;
  }
  __syncthreads();
  *total = scratch[TK_WARPS];
  return scratch[warp] + incl - v;
}

// load 8 consecutive keys starting at element i8*8 (VEC: one 16-byte load), invalid ones as 0
template <bool VEC>
__device__ __forceinline__ void load8(const uint16_t* row, int i8, int T, uint32_t (&key)[8]) {
  const int base = i8 * 8;
  if (VEC && base + 8 <= T) {
    uint4 v = *reinterpret_cast<const uint4*>(row + base);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      key[2 * j] = topk_key(w[j] & 0xffffu);
      key[2 * j + 1] = topk_key(w[j] >> 16);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++) key[j] = (base + j < T) ? topk_key(row[base + j]) : 0u;
  }
}

// Where a selected index goes: the index row and, optionally, the expanded token row of the same slot
// (helios::attn::pool_expand_row folded in: slot i -> tokens 4 idx .. 4 idx + 3, each kept if <= cur, else -1; the
// caller appends the four tail tokens in slot k_pad).
struct TopkSink {
  int* idx;          // [k_pad] (global or shared)
  int4* raw;         // [k_pad + 1] or nullptr
  int cur;
  __device__ __forceinline__ void put(int slot, int v) const {
    idx[slot] = v;
    if (raw) {
      const int tk = v * POOL;
      raw[slot] = v < 0 ? make_int4(-1, -1, -1, -1)
                        : make_int4(tk <= cur ? tk : -1, tk + 1 <= cur ? tk + 1 : -1, tk + 2 <= cur ? tk + 2 : -1,
                                    tk + 3 <= cur ? tk + 3 : -1);
    }
  }
  __device__ __forceinline__ void put_tail(int k_pad) const {
    if (raw)
      raw[k_pad] = make_int4(cur - 3 >= 0 ? cur - 3 : -1, cur - 2 >= 0 ? cur - 2 : -1, cur - 1 >= 0 ? cur - 1 : -1,
                             cur >= 0 ? cur : -1);
  }
};

// One row by one CTA of TK_THREADS threads; `row` and the sink's index row may point to global or shared memory.
template <bool VEC>
__device__ __forceinline__ void topk_row(const uint16_t* row, const TopkSink row_o, int T, int k, int k_pad) {
  const int t = threadIdx.x;
  const int n_slots = (T + 7) >> 3;

  __shared__ int hist[2048];
  __shared__ int scan_ws[TK_WARPS + 1];
  __shared__ int sh_sel[3];  // crossing bucket, count above it, (sweep 2) low bits

  // ---- sweep 1: histogram of key >> 5 over selectable entries (bucket >= 32 <=> key > -inf) ----
  for (int i = t; i < 2048; i += TK_THREADS) hist[i] = 0;
  __syncthreads();
  for (int i8 = t; i8 < n_slots; i8 += TK_THREADS) {
    uint32_t key[8];
    load8<VEC>(row, i8, T, key);
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (key[j] > KEY_NEG_INF) atomicAdd(&hist[key[j] >> 5], 1);
  }
  __syncthreads();
  // thread t owns buckets 2047-2t and 2046-2t (descending); find where the running count crosses k
  int h_hi = hist[2047 - 2 * t], h_lo = hist[2046 - 2 * t];
  int total_sel;
  int excl = block_exscan(h_hi + h_lo, scan_ws, &total_sel);
  if (t == 0) sh_sel[0] = -1;
  __syncthreads();
  if (total_sel >= k && k > 0) {
    if (excl < k && excl + h_hi >= k) { sh_sel[0] = 2047 - 2 * t; sh_sel[1] = excl; }
    else if (excl + h_hi < k && excl + h_hi + h_lo >= k) { sh_sel[0] = 2046 - 2 * t; sh_sel[1] = excl + h_hi; }
  }
  __syncthreads();
  const int b1 = sh_sel[0];
  uint32_t thresh;
  int cnt_gt, n_eq_take;
  if (b1 < 0) {
    // fewer than k selectable entries (or k == 0): take them all, no ties
    thresh = KEY_NEG_INF;
    cnt_gt = k > 0 ? total_sel : 0;
    n_eq_take = 0;
    if (k == 0) thresh = 0xffffu;
  } else {
    const int above1 = sh_sel[1];
    // ---- sweep 2: low 5 bits inside bucket b1 ----
    if (t < 32) hist[t] = 0;
    __syncthreads();
    for (int i8 = t; i8 < n_slots; i8 += TK_THREADS) {
      uint32_t key[8];
      load8<VEC>(row, i8, T, key);
#pragma unroll
      for (int j = 0; j < 8; j++)
        if ((int)(key[j] >> 5) == b1) atomicAdd(&hist[key[j] & 31u], 1);
    }
    __syncthreads();
    if (t < 32) {
      // lane l owns low value 31-l (descending)
      const int hv = hist[31 - t];
      int incl = hv;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (t >= o) incl += n;
      }
      const int need = k - above1;
      if (incl - hv < need && incl >= need) { sh_sel[2] = 31 - t; sh_sel[1] = above1 + incl - hv; }
    }
    __syncthreads();
    thresh = ((uint32_t)b1 << 5) | (uint32_t)sh_sel[2];
    cnt_gt = sh_sel[1];
    n_eq_take = k - cnt_gt;
  }

  // ---- sweep 3: ordered compaction, 8 consecutive elements per thread per tile ----
  int base_gt = 0, base_eq = 0;
  const int n_tiles = (n_slots + TK_THREADS - 1) / TK_THREADS;
  for (int tile = 0; tile < n_tiles; tile++) {
    if (base_gt >= cnt_gt && base_eq >= n_eq_take) break;  // block-uniform
    const int i8 = tile * TK_THREADS + t;
    uint32_t m_gt = 0, m_eq = 0;
    if (i8 < n_slots) {
      uint32_t key[8];
      load8<VEC>(row, i8, T, key);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        if (key[j] > thresh && key[j] > KEY_NEG_INF) m_gt |= 1u << j;
        if (key[j] == thresh && n_eq_take > 0) m_eq |= 1u << j;
      }
    }
    const int packed = __popc(m_gt) | (__popc(m_eq) << 16);
    int tot;
    const int ex = block_exscan(packed, scan_ws, &tot);
    int o_gt = base_gt + (ex & 0xffff);
    int o_eq = base_eq + (ex >> 16);
    const int ibase = i8 * 8;
    while (m_gt) {
      const int j = __ffs((int)m_gt) - 1;
      m_gt &= m_gt - 1;
      row_o.put(o_gt++, ibase + j);
    }
    while (m_eq) {
      const int j = __ffs((int)m_eq) - 1;
      m_eq &= m_eq - 1;
      if (o_eq < n_eq_take) row_o.put(cnt_gt + o_eq, ibase + j);
      o_eq++;
    }
    base_gt += tot & 0xffff;
    base_eq += tot >> 16;
  }
  const int emitted = cnt_gt + min(base_eq, n_eq_take);
  for (int j = emitted + t; j < k_pad; j += TK_THREADS) row_o.put(j, -1);
  if (t == 0) row_o.put_tail(k_pad);
}

// raw != nullptr: the expanded token rows [R][4 k_pad + 4] are written as well, row r clipped at q_pos[r]
template <bool VEC>
__global__ __launch_bounds__(TK_THREADS) void dsa_topk_kernel(
    const uint16_t* scores, int* __restrict__ out, int T, int s_stride, int k,
    int k_pad, const int* __restrict__ t_ptr, int t_seq, int* __restrict__ raw, const int* __restrict__ q_pos) {
  // behind a kernel that allowed its dependents to start early (the scorer): wait for its scores
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (t_ptr) T = t_seq > 0 ? t_ptr[blockIdx.x / t_seq] : *t_ptr;
  TopkSink sink{out + (size_t)blockIdx.x * k_pad,
                raw ? reinterpret_cast<int4*>(raw + (size_t)blockIdx.x * (4 * k_pad + 4)) : nullptr,
                raw ? q_pos[blockIdx.x] : 0};
  topk_row<VEC>(scores + (size_t)blockIdx.x * s_stride, sink, T, k, k_pad);
}


// ------------------------------------------------------------------------------------------------
// Rows of at most 65,536 scores (the decode case is ONE such row): a thread-block cluster of 8 CTAs
// works on a row, CTA c on elements [8192 c, 8192 (c+1)), every thread on 8 consecutive elements that
// stay in registers, so the row is read from global memory once and no sweep is longer than 8 keys
// per thread.  The CTAs meet through distributed shared memory: the bucket histograms are summed
// slice-wise and the sums stored into every CTA, each CTA then finds the crossing bucket itself; the
// low-bit count sets are read by every CTA, which finds the threshold and, from the per-CTA counts, the
// offset of its own ordered output - four cluster barriers in all, no hand-back round trips.
// ------------------------------------------------------------------------------------------------
#ifdef HK_TOPK_TRACE
__device__ long long hk_topk_trace[16];
#define TK_TRACE(slot) do { if (threadIdx.x == 0 && blockIdx.x == 0) hk_topk_trace[slot] = clock64(); } while (0)
#else
#define TK_TRACE(slot) do { } while (0)
#endif
constexpr int TKC_CTAS = 8;
constexpr int TKC_MAX_T = TKC_CTAS * TK_THREADS * 8;      // 65536

template <bool VEC>
__global__ __cluster_dims__(TKC_CTAS, 1, 1) __launch_bounds__(TK_THREADS) void dsa_topk_cluster_kernel(
    const uint16_t* scores, int* __restrict__ out, int T, int s_stride, int k, int k_pad,
    int* __restrict__ raw, const int* __restrict__ q_pos) {
  namespace cg = cooperative_groups;
  asm volatile("griddepcontrol.wait;" ::: "memory");   // see dsa_topk_kernel
  cg::cluster_group cluster = cg::this_cluster();
  const int c = (int)cluster.block_rank();
  const int row_id = blockIdx.x / TKC_CTAS;
  const uint16_t* row = scores + (size_t)row_id * s_stride;
  const TopkSink row_o{out + (size_t)row_id * k_pad,
                       raw ? reinterpret_cast<int4*>(raw + (size_t)row_id * (4 * k_pad + 4)) : nullptr, raw ? q_pos[row_id] : 0};
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

  __shared__ int hist[2048];       // this CTA's bucket counts
  __shared__ int ghist[2048];      // bucket counts of the whole row (every CTA gets a copy)
  __shared__ int low[33];          // this CTA: counts of the low 5 bits inside the crossing bucket; [32] = keys above it
  __shared__ int scan_ws[TK_WARPS + 1];
  __shared__ int sh_sel[3];
  __shared__ int sh_off[6];        // threshold low bits, count above threshold, this CTA's bases, total ties

  TK_TRACE(0);
  uint32_t key[8];
  const int i8 = c * TK_THREADS + t;
  load8<VEC>(row, i8, T, key);     // beyond T: key 0, never selectable
  for (int i = t; i < 2048; i += TK_THREADS) hist[i] = 0;
  if (t < 33) low[t] = 0;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; j++)
    if (key[j] > KEY_NEG_INF) atomicAdd(&hist[key[j] >> 5], 1);
  cluster.sync();                  // (1) all local histograms complete
  TK_TRACE(1);
  // slice c of the buckets is summed over the eight CTAs by CTA c and stored into EVERY CTA's copy of
  // the row histogram (reading all eight histograms in all eight CTAs costs far more distributed traffic)
  if (t < 2048 / TKC_CTAS) {
    const int bin = c * (2048 / TKC_CTAS) + t;
    int sum = 0;
#pragma unroll
    for (int rk = 0; rk < TKC_CTAS; rk++) sum += cluster.map_shared_rank(hist, rk)[bin];
#pragma unroll
    for (int rk = 0; rk < TKC_CTAS; rk++) cluster.map_shared_rank(ghist, rk)[bin] = sum;
  }
  cluster.sync();                  // (2) every CTA holds the row histogram
  // thread t owns buckets 2047-2t and 2046-2t (descending) and finds where the running count crosses k
  const int h_hi = ghist[2047 - 2 * t], h_lo = ghist[2046 - 2 * t];
  int total_sel;
  const int excl = block_exscan(h_hi + h_lo, scan_ws, &total_sel);
  if (t == 0) { sh_sel[0] = -1; sh_sel[1] = 0; }
  __syncthreads();
  if (total_sel >= k && k > 0) {
    if (excl < k && excl + h_hi >= k) { sh_sel[0] = 2047 - 2 * t; sh_sel[1] = excl; }
    else if (excl + h_hi < k && excl + h_hi + h_lo >= k) { sh_sel[0] = 2046 - 2 * t; sh_sel[1] = excl + h_hi; }
  }
  __syncthreads();
  const int b1 = sh_sel[0], above1 = sh_sel[1];
  TK_TRACE(2);
  // local counts: low 5 bits inside bucket b1, and the keys in buckets above it.  Without a crossing bucket
  // (fewer than k selectable entries, or k == 0) every selectable key counts as "above".
  const int b_eff = b1 < 0 ? 31 : b1;
  int n_above = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int bk = (int)(key[j] >> 5);
    if (bk == b1) atomicAdd(&low[key[j] & 31u], 1);
    n_above += bk > b_eff;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) n_above += __shfl_xor_sync(0xffffffffu, n_above, o);
  if (lane == 0 && n_above) atomicAdd(&low[32], n_above);
  cluster.sync();                  // (3) all local low-bit counts complete
  TK_TRACE(3);
  if (warp == 0) {
    // lane l owns low value 31-l (descending); per CTA counts first, then the row's
    int mine[TKC_CTAS], above_c[TKC_CTAS], g = 0;
#pragma unroll
    for (int rk = 0; rk < TKC_CTAS; rk++) {
      const int* rl = cluster.map_shared_rank(low, rk);
      mine[rk] = rl[31 - lane];
      above_c[rk] = rl[32];
      g += mine[rk];
    }
    int lowbits = 0, cnt_gt_row = k > 0 ? total_sel : 0, need_eq = 0;
    if (b1 >= 0) {
      int incl = g;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      const int need = k - above1;
      const unsigned who = __ballot_sync(0xffffffffu, incl - g < need && incl >= need);
      const int src = __ffs((int)who) - 1;                  // lane of the crossing low value
      lowbits = 31 - src;
      cnt_gt_row = above1 + __shfl_sync(0xffffffffu, incl - g, src);
      need_eq = k - cnt_gt_row;
      // per CTA: keys above the threshold = above the bucket + low values above lowbits (lanes < src); ties = lane src
      int base_gt = 0, base_eq = 0, all_eq = 0;
#pragma unroll
      for (int rk = 0; rk < TKC_CTAS; rk++) {
        int hi = lane < src ? mine[rk] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) hi += __shfl_xor_sync(0xffffffffu, hi, o);
        const int eq = __shfl_sync(0xffffffffu, mine[rk], src);
        if (rk < c) { base_gt += above_c[rk] + hi; base_eq += eq; }
        all_eq += eq;
      }
      if (lane == 0) { sh_off[2] = base_gt; sh_off[3] = base_eq; sh_off[4] = all_eq; }
    } else {
      int base_gt = 0;
#pragma unroll
      for (int rk = 0; rk < TKC_CTAS; rk++)
        if (rk < c) base_gt += above_c[rk];
      if (lane == 0) { sh_off[2] = k > 0 ? base_gt : 0; sh_off[3] = 0; sh_off[4] = 0; }
    }
    if (lane == 0) { sh_off[0] = lowbits; sh_off[1] = cnt_gt_row; sh_off[5] = need_eq; }
  }
  __syncthreads();
  uint32_t thresh;
  const int cnt_gt = sh_off[1], n_eq_take = sh_off[5];
  if (b1 < 0) thresh = k == 0 ? 0xffffu : KEY_NEG_INF;
  else thresh = ((uint32_t)b1 << 5) | (uint32_t)sh_off[0];
  TK_TRACE(4);
  // ---- ordered compaction inside the CTA, offset by the counts of the CTAs before it ----
  uint32_t m_gt = 0, m_eq = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if (key[j] > thresh && key[j] > KEY_NEG_INF) m_gt |= 1u << j;
    if (key[j] == thresh && n_eq_take > 0) m_eq |= 1u << j;
  }
  int tot;
  const int ex = block_exscan(__popc(m_gt) | (__popc(m_eq) << 16), scan_ws, &tot);
  TK_TRACE(5);
  int o_gt = sh_off[2] + (ex & 0xffff);
  int o_eq = sh_off[3] + (ex >> 16);
  const int ibase = i8 * 8;
  while (m_gt) {
    const int j = __ffs((int)m_gt) - 1;
    m_gt &= m_gt - 1;
    row_o.put(o_gt++, ibase + j);
  }
  while (m_eq) {
    const int j = __ffs((int)m_eq) - 1;
    m_eq &= m_eq - 1;
    if (o_eq < n_eq_take) row_o.put(cnt_gt + o_eq, ibase + j);
    o_eq++;
  }
  if (c == 0) {
    const int emitted = cnt_gt + min(sh_off[4], n_eq_take);
    for (int j = emitted + t; j < k_pad; j += TK_THREADS) row_o.put(j, -1);
    if (t == 0) row_o.put_tail(k_pad);
  }
  TK_TRACE(6);
  cluster.sync();                  // (4) no CTA leaves while a peer may still read its shared memory
}

}  // namespace hk

#ifdef HK_TOPK_TRACE
extern "C" __attribute__((visibility("default"))) int hk_debug_topk_trace(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, hk::hk_topk_trace, sizeof(long long) * 16) == cudaSuccess ? 0 : 3;
}
#endif

namespace hk {
// common launcher; raw != nullptr adds the expansion, pdl launches the kernel as a programmatic dependent of the
// kernel before it in the stream (which must have released its dependents: the decode scorer does)
static int topk_launch(const void* scores, int s_stride, int* indices, int R, int T, int k, int k_pad, const int* t_ptr,
                       int t_seq, int* raw, const int* q_pos, bool pdl, cudaStream_t s) {
  const bool vec = (s_stride % 8 == 0) && aligned(scores, 16);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(TK_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const uint16_t* sc = (const uint16_t*)scores;
  cudaError_t e;
  if (T > 16384 && T <= TKC_MAX_T && R <= 16 && !t_ptr) {
    // a few long rows (decode): one 8-CTA cluster per row.  With many rows (prefill) the clusters queue for
    // eight free SMs of one GPC each and the one-CTA kernel below is 3 to 20 times faster (measured at
    // 64 to 4,096 rows); up to 16,384 scores one CTA is as fast as the cluster even for a single row.
    cfg.gridDim = dim3(R * TKC_CTAS);
    e = vec ? cudaLaunchKernelEx(&cfg, dsa_topk_cluster_kernel<true>, sc, indices, T, s_stride, k, k_pad, raw, q_pos)
            : cudaLaunchKernelEx(&cfg, dsa_topk_cluster_kernel<false>, sc, indices, T, s_stride, k, k_pad, raw, q_pos);
  } else {
    cfg.gridDim = dim3(R);
    e = vec ? cudaLaunchKernelEx(&cfg, dsa_topk_kernel<true>, sc, indices, T, s_stride, k, k_pad, t_ptr, t_seq, raw, q_pos)
            : cudaLaunchKernelEx(&cfg, dsa_topk_kernel<false>, sc, indices, T, s_stride, k, k_pad, t_ptr, t_seq, raw, q_pos);
  }
  return e == cudaSuccess && cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}
}  // namespace hk

HK_API int hk_dsa_topk(const void* scores, int s_stride, int* indices, int R, int T, int k,
                       int k_pad, const int* t_ptr, int t_seq, void* stream) {
  using namespace hk;
  HK_REQUIRE(scores && indices && R >= 0 && T >= 0 && k >= 0 && k <= k_pad && s_stride >= 0);
  HK_REQUIRE(k <= 32767);  // packed 16-bit counters in the compaction scan
  if (R == 0) return HK_OK;
  return topk_launch(scores, s_stride, indices, R, T, k, k_pad, t_ptr, t_seq, nullptr, nullptr, false, as_stream(stream));
}

HK_API int hk_dsa_topk_expand(const void* scores, int s_stride, int* indices, int* raw_idx, const int* q_pos, int R, int T,
                              int k, int after_scorer, void* stream) {
  using namespace hk;
  HK_REQUIRE(scores && indices && raw_idx && q_pos && R >= 0 && T >= 0 && k >= 0 && k <= 512 && s_stride >= 0);
  HK_REQUIRE(aligned(raw_idx, 16));
  if (R == 0) return HK_OK;
  return topk_launch(scores, s_stride, indices, R, T, k, 512, nullptr, 0, raw_idx, q_pos, after_scorer != 0, as_stream(stream));
}

#include "dsa_select_splitkv.cuh"
