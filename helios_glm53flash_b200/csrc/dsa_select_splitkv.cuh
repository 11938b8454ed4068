// Top-512 selection of the DSA indexer when the pooled keys of ONE sequence are split over the GPUs of a node
// (sparse split-KV decode).  Rank g scores only its own pools and takes a local top-k; the k candidates of every
// rank (score bits + global pool index, 3 KB per query row) are stored into every rank's exchange region; every
// rank then selects the k best of the G x k candidates and expands them to cache rows of its own slice.
//
// Why the result equals the one-GPU selection of helios::aux::dsa_topk (reference: src/cuda/aux/dsa_topk.cu:179-267,
// "above the k-th value in ascending index order, then ties in ascending index order"): an entry of rank g that the
// whole-row selection takes has fewer than k entries of rank g ahead of it (larger score, or equal score and smaller
// index: all of them are taken by the whole-row selection as well), so it is among rank g's local top-k.  The
// candidate row is laid out rank by rank and, inside a rank, in ascending pool index (the local result's two ascending
// runs are merged here), i.e. in ascending GLOBAL pool index: position order equals index order and the same
// selection routine run over the candidate row breaks ties exactly as it would over the whole row.
//
// Exchange-region part used here (offsets from `cand_base` of a rank's region; G ranks, m query rows, set = step & 1):
//   int   cflags[64]                 [0, G): candidate flags (slot r = last step rank r has published); [32]: ticket
//   int   idx[2][m][G][512]          global pool index or -1
//   u16   sc [2][m][G][512]          fp16 bits, 0xfc00 (-inf) where idx is -1
// Double buffering by step parity is safe for the same reason as for the partial sets: a rank reaches step e + 1 only
// after every peer has signalled its step-e partial, i.e. has finished reading the candidates of step e - 1.
#pragma once

namespace hk {

constexpr int SEL_K = 512;
constexpr int SEL_MAX_RANKS = 8;

__host__ __device__ inline size_t sel_idx_off(int m, int G, int set, int row, int src) {
  return 256 + ((((size_t)set * m + row) * G + src) * SEL_K) * 4;
}
__host__ __device__ inline size_t sel_sc_off(int m, int G, int set, int row, int src) {
  return 256 + (size_t)2 * m * G * SEL_K * 4 + ((((size_t)set * m + row) * G + src) * SEL_K) * 2;
}
inline size_t sel_region_bytes(int m, int G) { return 256 + (size_t)2 * m * G * SEL_K * 6; }

// grid = m, block = 512.  local_idx [m][512]: this rank's local selection (dsa_topk output: -1 padded).
__global__ __launch_bounds__(SEL_K) void sel_publish_kernel(const uint16_t* __restrict__ scores, int s_stride,
                                                           const int* __restrict__ local_idx, int pool_base,
                                                           char* const* __restrict__ cand_bases, int n_ranks, int my_rank,
                                                           int m, const int* __restrict__ step_ctr, int do_signal) {
  __shared__ int s_idx[SEL_K];
  __shared__ int s_oidx[SEL_K];
  __shared__ uint16_t s_osc[SEL_K];
  __shared__ int s_na;
  __shared__ int s_last;
  const int row = blockIdx.x, i = threadIdx.x;
  const int epoch = *step_ctr + 1, set = epoch & 1;
  const int li = local_idx[(size_t)row * SEL_K + i];
  const bool valid = li >= 0;
  s_idx[i] = li;
  s_oidx[i] = -1;
  s_osc[i] = 0xfc00u;
  if (i == 0) s_na = SEL_K;
  const int n_valid = __syncthreads_count(valid);          // valid entries are a prefix of the row
  // first run: entries above the local threshold (ascending); second run: ties (ascending).  The second run starts
  // at the first descent, if there is one.
  if (i > 0 && valid && li < s_idx[i - 1]) atomicMin(&s_na, i);
  __syncthreads();
  const int na = min(s_na, n_valid);
  if (valid) {
    int lo, hi;                                           // the other run
    if (i < na) { lo = na; hi = n_valid; } else { lo = 0; hi = na; }
    const int start = lo;
    while (lo < hi) {                                     // number of entries of the other run below li
      const int mid = (lo + hi) >> 1;
      if (s_idx[mid] < li) lo = mid + 1; else hi = mid;
    }
    const int r = (i < na ? i : i - na) + (lo - start);
    s_oidx[r] = li + pool_base;
    s_osc[r] = scores[(size_t)row * s_stride + li];
  }
  __syncthreads();
  for (int g = 0; g < n_ranks; g++) {
    char* base = cand_bases[g];
    reinterpret_cast<int*>(base + sel_idx_off(m, n_ranks, set, row, my_rank))[i] = s_oidx[i];
    if (i < SEL_K / 2)
      reinterpret_cast<uint32_t*>(base + sel_sc_off(m, n_ranks, set, row, my_rank))[i] =
          (uint32_t)s_osc[2 * i] | ((uint32_t)s_osc[2 * i + 1] << 16);
  }
  // the CTA that takes the last ticket publishes the step to every rank
  __threadfence_system();
  __syncthreads();
  int* my_flags = reinterpret_cast<int*>(cand_bases[my_rank]);
  if (i == 0) {
    const int tk = atomicAdd(my_flags + 32, 1);
    s_last = tk == m - 1;
    if (s_last) my_flags[32] = 0;
  }
  __syncthreads();
  if (s_last && do_signal && i < n_ranks) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int*>(cand_bases[i]) + my_rank), "r"(epoch)
                 : "memory");
  }
}

// grid = m, block = 1024.  Waits (bounded) for every rank's candidates of this step in the LOCAL region, selects,
// writes the selected GLOBAL pool indices (sel_pools [m][512], may be NULL) and the expanded cache rows relative to
// this rank's slice (raw_local [m][4*512 + 4]: row - row_base if inside [0, n_local_rows), else -1; the four tail
// positions q_pos - 3 .. q_pos are appended as helios::attn::pool_expand_row does).
__global__ __launch_bounds__(TK_THREADS) void sel_select_kernel(const char* __restrict__ cand_base, int n_ranks, int m, int k,
                                                               const int* __restrict__ q_pos, int row_base, int n_local_rows,
                                                               int* __restrict__ sel_pools, int* __restrict__ raw_local,
                                                               const int* __restrict__ step_ctr, long long max_wait_cycles,
                                                               int* __restrict__ status) {
  __shared__ __align__(16) uint16_t s_sc[SEL_MAX_RANKS * SEL_K];
  __shared__ int s_ci[SEL_MAX_RANKS * SEL_K];
  __shared__ int s_pos[SEL_K];
  __shared__ int s_ready;
  const int row = blockIdx.x, t = threadIdx.x;
  const int epoch = *step_ctr + 1, set = epoch & 1;
  const int n_cand = n_ranks * SEL_K;
  if (t == 0) {
    const int* flags = reinterpret_cast<const int*>(cand_base);
    int ok = 1;
    const long long t0 = clock64();
    for (int g = 0; g < n_ranks && ok; g++) {
      for (;;) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + g) : "memory");
        if (v >= epoch) break;
        if (clock64() - t0 > max_wait_cycles) { ok = 0; break; }
        __nanosleep(200);
      }
    }
    s_ready = ok;
    if (!ok && status) atomicExch(status, HK_ERR_TIMEOUT);
  }
  __syncthreads();
  if (!s_ready) return;
  // candidates were written by other GPUs: volatile loads into shared memory, selection from there
  const int* gi = reinterpret_cast<const int*>(cand_base + sel_idx_off(m, n_ranks, set, row, 0));
  const uint32_t* gs = reinterpret_cast<const uint32_t*>(cand_base + sel_sc_off(m, n_ranks, set, row, 0));
  for (int j = t; j < n_cand; j += TK_THREADS) s_ci[j] = __ldcv(gi + j);
  for (int j = t; j < n_cand / 2; j += TK_THREADS) reinterpret_cast<uint32_t*>(s_sc)[j] = __ldcv(gs + j);
  __syncthreads();
  topk_row<true>(s_sc, TopkSink{s_pos, nullptr, 0}, n_cand, k, SEL_K);
  __syncthreads();
  const int cur = q_pos[row];
  int4* out = reinterpret_cast<int4*>(raw_local + (size_t)row * (SEL_K * 4 + 4));
  auto local = [&](int tok) { const int r = tok - row_base; return (tok >= 0 && tok <= cur && r >= 0 && r < n_local_rows) ? r : -1; };
  if (t <= SEL_K) {
    int4 v;
    if (t < SEL_K) {
      const int pos = s_pos[t];
      const int pi = pos >= 0 ? s_ci[pos] : -1;
      if (sel_pools) sel_pools[(size_t)row * SEL_K + t] = pi;
      const int tk = pi * 4;
      v.x = pi >= 0 ? local(tk) : -1;
      v.y = pi >= 0 ? local(tk + 1) : -1;
      v.z = pi >= 0 ? local(tk + 2) : -1;
      v.w = pi >= 0 ? local(tk + 3) : -1;
    } else {
      v.x = local(cur - 3); v.y = local(cur - 2); v.z = local(cur - 1); v.w = local(cur);
    }
    out[t] = v;
  }
}

}  // namespace hk

HK_API size_t hk_dsa_select_region_bytes(int m, int n_ranks) {
  if (m <= 0 || n_ranks <= 0 || n_ranks > hk::SEL_MAX_RANKS) return 0;
  return hk::sel_region_bytes(m, n_ranks);
}

HK_API int hk_dsa_select_splitkv(const void* scores, int s_stride, int n_local_pools, int pool_base, int* local_idx,
                                 void* const* cand_bases, const void* local_cand_base, int n_ranks, int my_rank, int m, int k,
                                 const int* q_pos, int row_base, int n_local_rows, int* sel_pools, int* raw_local,
                                 const int* step_ctr, int max_wait_ms, int signal, int phases, void* stream) {
  using namespace hk;
  HK_REQUIRE(phases >= 1 && phases <= 3);
  HK_REQUIRE(scores && local_idx && cand_bases && local_cand_base && q_pos && raw_local && step_ctr);
  HK_REQUIRE(m > 0 && k >= 0 && k <= SEL_K && n_ranks >= 1 && n_ranks <= SEL_MAX_RANKS && my_rank >= 0 && my_rank < n_ranks);
  HK_REQUIRE(n_local_pools >= 0 && s_stride >= n_local_pools && pool_base >= 0 && row_base >= 0 && n_local_rows >= 0);
  HK_REQUIRE(max_wait_ms > 0 && max_wait_ms <= 10000 && aligned(local_cand_base, 256) && aligned(raw_local, 16));
  cudaStream_t s = as_stream(stream);
  if (phases & 1) {
    const int st = hk_dsa_topk(scores, s_stride, local_idx, m, n_local_pools, k, SEL_K, nullptr, 0, stream);
    if (st != HK_OK) return st;
    sel_publish_kernel<<<m, SEL_K, 0, s>>>((const uint16_t*)scores, s_stride, local_idx, pool_base, (char* const*)cand_bases,
                                           n_ranks, my_rank, m, step_ctr, signal);
    HK_LAUNCH_CHECK();
  }
  if (!(phases & 2)) return HK_OK;
  sel_select_kernel<<<m, TK_THREADS, 0, s>>>((const char*)local_cand_base, n_ranks, m, k, q_pos, row_base, n_local_rows,
                                             sel_pools, raw_local, step_ctr, (long long)max_wait_ms * 2000000LL,
                                             device_status_ptr());
  HK_LAUNCH_CHECK();
  return HK_OK;
}
