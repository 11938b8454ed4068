// DSA indexer scores on the 5th-generation tensor cores.
//   S[r][p] = 32^-1/2 * sum_h w[r][h] * relu(128^-1/2 * q[r][h] . pk[p]),  -inf where 4p+3 > q_pos[r]
// Interface of helios::attn::indexer_score (reference: src/cuda/attn/attn.cu:182-273, an
// mma.sync.m16n8k16 kernel with queries as M).
//
// Orientation: POOLS are the MMA M dimension (128 pooled keys per tile = 128 TMEM lanes) and
// (query row, head) pairs are N (up to 8 rows x 32 heads = 256 columns), K = 128.  That way the
// relu / head-weight / head-sum epilogue reads one TMEM lane per thread and never crosses lanes,
// and a decode step (one query row) is a single M128 N32 K128 tile per 32 KB of pooled keys: the
// kernel streams the key plane once from HBM (256 B per pool).  Both operands are K-major exactly
// as they sit in memory ([pool][128] and [row][head][128]); they are staged with 16-byte cp.async
// into the no-swizzle core-matrix layout (8 rows x 16 B contiguous per lane group: conflict-free).
#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime at first use)
#include <cuda_pipeline_primitives.h>

#include <cstdlib>
#include <cstring>

#include "hk_common.cuh"
#include "tc05.cuh"

namespace hk {

constexpr int IX_TILE_P = 128;   // pools per tile (MMA M)
constexpr int IX_RG = 8;         // query rows per MMA group (N = 32 * rows)
constexpr int IX_HEADS = 32;
constexpr uint32_t IX_LBO = 128;           // K-chunk stride: core matrices adjacent along K
constexpr uint32_t IX_SBO = 16 * 128;      // 8-row group stride: 16 K-chunks of 128 B
constexpr size_t IX_SMEM_A = (size_t)IX_TILE_P * IDX_DIM * 2;            // 32 KB
constexpr size_t IX_SMEM_B = (size_t)IX_RG * IX_HEADS * IDX_DIM * 2;     // 64 KB
constexpr size_t IX_SMEM = IX_SMEM_A + IX_SMEM_B + IX_RG * IX_HEADS * 4 + IX_RG * 4 + 64;

// Stage `nrows` rows of 128 16-bit elements (256 B each, contiguous in global memory) as a K-major
// tile.  Lane l of a warp handles row (l % 8) of an 8-row group and K-chunk (l / 8) + 4*j, so every
// quarter-warp writes one contiguous 128-byte core matrix.  Rows >= valid_rows are zero-filled.
__device__ __forceinline__ void stage_kmajor_rows(uint8_t* smem_tile, const uint16_t* gsrc,
                                                  int nrows, int valid_rows, int tid, int nthreads) {
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  const int r_in = lane & 7, kc0 = lane >> 3;
  // one warp-iteration covers 8 rows x 4 chunks; a row group needs 4 of them (16 chunks)
  const int items = (nrows / 8) * 4;
  for (int it = warp; it < items; it += nwarps) {
    const int grp = it >> 2, kc = kc0 + (it & 3) * 4;
    const int row = grp * 8 + r_in;
    uint8_t* dst = smem_tile + grp * IX_SBO + kc * IX_LBO + r_in * 16;
    if (row < valid_rows) {
      __pipeline_memcpy_async(dst, gsrc + (size_t)row * IDX_DIM + kc * 8, 16);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
}

template <int FMT>
__global__ __launch_bounds__(128) void indexer_tc_kernel(
    const uint16_t* __restrict__ q, const uint16_t* __restrict__ pk, const uint16_t* __restrict__ w,
    const int* __restrict__ q_pos, __half* __restrict__ scores, int m, int npools, int score_stride,
    int rows_per_cta, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sA = smem;
  uint8_t* sB = smem + IX_SMEM_A;
  float* w_sm = reinterpret_cast<float*>(sB + IX_SMEM_B);
  int* pos_sm = reinterpret_cast<int*>(w_sm + IX_RG * IX_HEADS);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int p0 = blockIdx.x * IX_TILE_P;
  const int r_begin = blockIdx.y * rows_per_cta;
  const int r_end = min(m, r_begin + rows_per_cta);

  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 256);
  stage_kmajor_rows(sA, pk + (size_t)p0 * IDX_DIM, IX_TILE_P, min(IX_TILE_P, npools - p0), tid, 128);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t a_addr = tc::smem_u32(sA), b_addr = tc::smem_u32(sB);
  const int p = p0 + tid;  // this thread's pool (TMEM lane tid)
  uint32_t parity = 0;

  for (int rg0 = r_begin; rg0 < r_end; rg0 += IX_RG) {
    const int nr = min(IX_RG, r_end - rg0);
    const int nb = nr * IX_HEADS;  // N of this group
    stage_kmajor_rows(sB, q + (size_t)rg0 * IX_HEADS * IDX_DIM, nb, nb, tid, 128);
    for (int i = tid; i < nb; i += 128) {
      const uint16_t wb = w[(size_t)rg0 * IX_HEADS + i];
      w_sm[i] = FMT == tc::FMT_BF16 ? bf16_bits_to_f(wb) : __half2float(__ushort_as_half(wb));
    }
    if (tid < nr) pos_sm[tid] = q_pos[rg0 + tid];
    __pipeline_commit();
    __pipeline_wait_prior(0);
    tc::fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      const uint32_t idesc = tc::make_idesc(IX_TILE_P, nb, FMT, FMT, false, false);
#pragma unroll
      for (int kk = 0; kk < IDX_DIM / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(a_addr + kk * 2 * IX_LBO, IX_LBO, IX_SBO);
        const uint64_t bd = tc::make_sdesc(b_addr + kk * 2 * IX_LBO, IX_LBO, IX_SBO);
        tc::mma_f16(tmem, ad, bd, idesc, kk > 0);
      }
      tc::mma_commit(&bar);
    }
    const bool ok = tc::mbar_wait(&bar, parity, &abort_flag, 1);
    parity ^= 1;
    tc::fence_after_sync();
    if (ok) {
      for (int rr = 0; rr < nr; rr++) {
        uint32_t c[32];
        tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + rr * IX_HEADS, c);
        tc::tmem_ld_wait();
        float tot = 0.f;
#pragma unroll
        for (int h = 0; h < IX_HEADS; h++) {
          const float d = __uint_as_float(c[h]) * 0.08838834764f;
          tot = fmaf(w_sm[rr * IX_HEADS + h], fmaxf(d, 0.f), tot);
        }
        if (p < npools) {
          const bool vis = p * POOL + POOL - 1 <= pos_sm[rr];
          scores[(size_t)(rg0 + rr) * score_stride + p] =
              vis ? __float2half_rn(tot * 0.17677669530f) : __ushort_as_half((unsigned short)0xfc00);
        }
      }
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
  }
  if (warp == 0) tc::tmem_dealloc(tmem, 256);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}


// ------------------------------------------------------------------------------------------------
// Decode form (at most 8 query rows = one N group): persistent CTAs stream the pooled-key plane.
// The query operand is staged once; key tiles of 128 pools (32 KB) are double buffered, fetched with
// fully coalesced 16-byte loads into registers while the previous tile is in the tensor pipe and the
// epilogue, then stored into a padded core-matrix layout (channel chunks 144 B apart, so the 8
// chunks a quarter-warp writes fall into different banks).
// ------------------------------------------------------------------------------------------------
constexpr uint32_t IXD_LBO = 144;                // K-chunk stride (128 B core matrix + 16 B pad)
constexpr uint32_t IXD_SBO = 16 * IXD_LBO;       // 8-row group stride = 2304
constexpr uint32_t IXD_TILE = 16 * IXD_SBO;      // 128 rows = 36864 B

template <int FMT>
__global__ __launch_bounds__(128) void indexer_tc_decode_kernel(
    const uint16_t* __restrict__ q, const uint16_t* __restrict__ pk, const uint16_t* __restrict__ w,
    const int* __restrict__ q_pos, __half* __restrict__ scores, int m, int npools, int score_stride,
    int n_tiles, uint32_t tmem_cols, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sA = smem;                              // 2 x IXD_TILE
  uint8_t* sB = smem + 2 * IXD_TILE;               // (4 m) groups x IXD_SBO
  const int nb = m * IX_HEADS;                     // N
  float* w_sm = reinterpret_cast<float*>(sB + (nb / 8) * IXD_SBO);
  int* pos_sm = reinterpret_cast<int*>(w_sm + IX_RG * IX_HEADS);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane >> 4, chunk = lane & 15;    // a warp instruction covers 2 rows x 16 chunks
  // a selection kernel launched as this grid's programmatic dependent may be placed now; it waits for this grid's
  // completion itself before it reads a score
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, tmem_cols);
  // query rows -> B operand
  for (int r2 = warp; r2 < nb / 2; r2 += 4) {
    const int row = r2 * 2 + sub;
    const uint4 v = *reinterpret_cast<const uint4*>(q + (size_t)row * IDX_DIM + chunk * 8);
    *reinterpret_cast<uint4*>(sB + (row >> 3) * IXD_SBO + chunk * IXD_LBO + (row & 7) * 16) = v;
  }
  for (int i = tid; i < nb; i += 128) {
    const uint16_t wb = w[i];
    w_sm[i] = FMT == tc::FMT_BF16 ? bf16_bits_to_f(wb) : __half2float(__ushort_as_half(wb));
  }
  if (tid < m) pos_sm[tid] = q_pos[tid];

  uint4 stage[16];
  auto fetch = [&](int tile) {                     // 128 rows x 256 B of one tile into registers
    const int p0 = tile * IX_TILE_P;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int row = (warp + 4 * j) * 2 + sub;
      stage[j] = (p0 + row < npools) ? ld_stream16(pk + (size_t)(p0 + row) * IDX_DIM + chunk * 8)
                                     : make_uint4(0, 0, 0, 0);
    }
  };
  auto stash = [&](int buf) {
    uint8_t* dst = sA + buf * IXD_TILE;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int row = (warp + 4 * j) * 2 + sub;
      *reinterpret_cast<uint4*>(dst + (row >> 3) * IXD_SBO + chunk * IXD_LBO + (row & 7) * 16) = stage[j];
    }
  };
  int tile = blockIdx.x;
  if (tile < n_tiles) {
    fetch(tile);
    stash(0);
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t b_addr = tc::smem_u32(sB);
  const uint32_t idesc = tc::make_idesc(IX_TILE_P, nb, FMT, FMT, false, false);
  uint32_t parity = 0;
  int buf = 0;
  for (; tile < n_tiles; tile += gridDim.x, buf ^= 1) {
    const int next = tile + gridDim.x;
    if (next < n_tiles) fetch(next);               // in flight during the MMA and the epilogue below
    if (tid == 0) {
      const uint64_t ad0 = tc::make_sdesc(tc::smem_u32(sA + buf * IXD_TILE), IXD_LBO, IXD_SBO);
      const uint64_t bd0 = tc::make_sdesc(b_addr, IXD_LBO, IXD_SBO);
#pragma unroll
      for (int kk = 0; kk < IDX_DIM / 16; kk++)
        tc::mma_f16(tmem, tc::sdesc_advance(ad0, kk * 2 * IXD_LBO), tc::sdesc_advance(bd0, kk * 2 * IXD_LBO), idesc, kk > 0);
      tc::mma_commit(&bar);
    }
    const bool ok = tc::mbar_wait(&bar, parity, &abort_flag, 1);
    parity ^= 1;
    tc::fence_after_sync();
    const int p = tile * IX_TILE_P + tid;          // this thread's pool (TMEM lane tid)
    if (ok) {
      for (int rr = 0; rr < m; rr++) {
        uint32_t c[32];
        tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + rr * IX_HEADS, c);
        tc::tmem_ld_wait();
        float tot = 0.f;
#pragma unroll
        for (int h = 0; h < IX_HEADS; h++) {
          const float d = __uint_as_float(c[h]) * 0.08838834764f;
          tot = fmaf(w_sm[rr * IX_HEADS + h], fmaxf(d, 0.f), tot);
        }
        if (p < npools) {
          const bool vis = p * POOL + POOL - 1 <= pos_sm[rr];
          scores[(size_t)rr * score_stride + p] =
              vis ? __float2half_rn(tot * 0.17677669530f) : __ushort_as_half((unsigned short)0xfc00);
        }
      }
    }
    if (next < n_tiles) stash(buf ^ 1);            // the other buffer was last read two MMAs ago
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
  }
  if (warp == 0) tc::tmem_dealloc(tmem, tmem_cols);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

}  // namespace hk

// device word that records a bounded wait giving up (read with hk_read_device_status)
__device__ int hk_g_status = 0;

HK_API int hk_read_device_status(int* host_out, int reset) {
  if (!host_out) return HK_ERR_INVALID;
  if (cudaMemcpyFromSymbol(host_out, hk_g_status, sizeof(int)) != cudaSuccess) return HK_ERR_CUDA;
  if (reset) {
    int z = 0;
    if (cudaMemcpyToSymbol(hk_g_status, &z, sizeof(int)) != cudaSuccess) return HK_ERR_CUDA;
  }
  return HK_OK;
}

namespace hk {
int* device_status_ptr() {
  static int* ptr[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, hk_g_status) != cudaSuccess) return nullptr;
    ptr[dev] = (int*)p;
  }
  return ptr[dev];
}
}  // namespace hk

#include "indexer_prefill.cuh"

HK_API int hk_indexer_score(const void* q_idx, const void* pool_k_nt, const void* w,
                            const int* q_pos, void* scores, int m, int npools, int score_stride,
                            int n_heads, int dtype, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_idx && pool_k_nt && w && q_pos && scores);
  HK_REQUIRE(m >= 0 && npools >= 0 && score_stride >= npools);
  HK_REQUIRE(dtype == HK_F16 || dtype == HK_BF16);
  HK_REQUIRE(aligned(q_idx, 16) && aligned(pool_k_nt, 16));
  if (n_heads != IX_HEADS) return HK_ERR_UNSUPPORTED;
  if (m == 0 || npools == 0) return HK_OK;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(indexer_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IX_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(indexer_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IX_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  const int tiles = (npools + IX_TILE_P - 1) / IX_TILE_P;
  if (m <= IX_RG) {
    // decode form: persistent CTAs over the pool tiles
    const int nb = m * IX_HEADS;
    const size_t smem = 2 * IXD_TILE + (size_t)(nb / 8) * IXD_SBO + IX_RG * IX_HEADS * 4 + IX_RG * 4 + 64;
    uint32_t cols = 32;
    while ((int)cols < nb) cols <<= 1;
    static bool dattr[64] = {false};
    if (dev >= 0 && dev < 64 && !dattr[dev]) {
      const int max_smem = (int)(2 * IXD_TILE + 32 * IXD_SBO + IX_RG * IX_HEADS * 4 + IX_RG * 4 + 64);
      if (cudaFuncSetAttribute(indexer_tc_decode_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
          cudaFuncSetAttribute(indexer_tc_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess)
        return HK_ERR_CUDA;
      dattr[dev] = true;
    }
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    int grid_x = per_sm * sm_count();
    if (grid_x > tiles) grid_x = tiles;
    cudaStream_t sd = as_stream(stream);
    int* std_ = device_status_ptr();
    if (dtype == HK_F16)
      indexer_tc_decode_kernel<0><<<grid_x, 128, smem, sd>>>((const uint16_t*)q_idx, (const uint16_t*)pool_k_nt, (const uint16_t*)w, q_pos, (__half*)scores, m, npools, score_stride, tiles, cols, std_);
    else
      indexer_tc_decode_kernel<1><<<grid_x, 128, smem, sd>>>((const uint16_t*)q_idx, (const uint16_t*)pool_k_nt, (const uint16_t*)w, q_pos, (__half*)scores, m, npools, score_stride, tiles, cols, std_);
    HK_LAUNCH_CHECK();
    return HK_OK;
  }
  if (m >= 32) {
    // many rows: the pipelined copy-engine kernel
    const int st = indexer_prefill_launch(q_idx, pool_k_nt, w, q_pos, scores, m, npools, score_stride, dtype, as_stream(stream));
    if (st != HK_ERR_UNSUPPORTED) return st;
  }
  // enough row groups per CTA to amortise the key tile, enough CTAs to cover the GPU twice
  int row_groups = (m + IX_RG - 1) / IX_RG;
  int want_y = (2 * sm_count() + tiles - 1) / tiles;
  if (want_y < 1) want_y = 1;
  if (want_y > row_groups) want_y = row_groups;
  int groups_per_cta = (row_groups + want_y - 1) / want_y;
  int rows_per_cta = groups_per_cta * IX_RG;
  dim3 grid(tiles, (m + rows_per_cta - 1) / rows_per_cta);
  cudaStream_t s = as_stream(stream);
  int* st = device_status_ptr();
  if (dtype == HK_F16)
    indexer_tc_kernel<0><<<grid, 128, IX_SMEM, s>>>((const uint16_t*)q_idx, (const uint16_t*)pool_k_nt, (const uint16_t*)w, q_pos, (__half*)scores, m, npools, score_stride, rows_per_cta, st);
  else
    indexer_tc_kernel<1><<<grid, 128, IX_SMEM, s>>>((const uint16_t*)q_idx, (const uint16_t*)pool_k_nt, (const uint16_t*)w, q_pos, (__half*)scores, m, npools, score_stride, rows_per_cta, st);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

// Scores, top-k and expansion of a decode step (at most 8 query rows) in one call: the scorer above, then the
// selection kernel with the expansion folded into its output writes, launched as the scorer's programmatic dependent
// (its CTAs are resident and waiting when the last score is written).  The reference runs four launches here
// (indexer_score -> dsa_topk -> pool_expand_row -> ..., src/engine/runner.cpp:620-630); this is two.
HK_API int hk_indexer_select(const void* q_idx, const void* pool_k_nt, const void* w, const int* q_pos, void* scores,
                             int* indices, int* raw_idx, int m, int npools, int score_stride, int n_heads, int dtype, int k,
                             void* stream) {
  using namespace hk;
  HK_REQUIRE(indices && raw_idx && m >= 0 && k >= 0 && k <= 512);
  if (m == 0) return HK_OK;
  if (npools == 0) return hk_dsa_topk_expand(scores, score_stride, indices, raw_idx, q_pos, m, 0, k, 0, stream);
  const int st = hk_indexer_score(q_idx, pool_k_nt, w, q_pos, scores, m, npools, score_stride, n_heads, dtype, stream);
  if (st != HK_OK) return st;
  return hk_dsa_topk_expand(scores, score_stride, indices, raw_idx, q_pos, m, npools, k, m <= IX_RG ? 1 : 0, stream);
}
