// DSA indexer scores for MANY query rows (prefill), pipelined: same arithmetic and orientation as indexer_tc_kernel
// (pools = MMA M = TMEM lanes, (row, head) pairs = N, K = 128), but the operands arrive as tensor copies in the
// 128-byte-swizzle layout and the roles are split.  A CTA owns 16 query rows (two groups of 8 rows = two N = 256
// operands, 128 KB, loaded ONCE) and streams pool tiles of 128 pools (32 KB, two stages) past them:
//   warp 8     producer: the two query groups, then one pool tile per step
//   warp 9     issues, per pool tile, M128 N256 K128 for group 0 and for group 1 (8 tcgen05.mma each, converged warp,
//              elected lane) into the two accumulators (2 x 256 TMEM columns)
//   warps 0-7  epilogue of group 0 while group 1 is in the tensor pipe and vice versa: relu, head weights, head sum
//              (one TMEM lane = one pool per thread; warps w and w + 4 share a lane quarter and take four of the
//              group's eight rows each, all four in registers at once: with one row at a time and one warp per
//              scheduler the 32-step sum of a row ran as one exposed dependency chain), masked fp16 store
// Why this shape: the serial kernel re-staged the 64 KB query group for every pool tile with per-thread 16-byte copies
// (the load/store unit holds those to about 13 B per cycle and SM); a first pipelined form that still streamed the
// query groups past a resident pool tile moved 64 KB through L2 per 8.4 MFLOP and ran at the L2's bandwidth (400-500
// TFLOP/s).  Streaming the 32 KB pool tiles past 16 resident rows needs 32 KB per 16.8 MFLOP.
// Pool tiles that no row of the CTA may see yet (4p + 3 > position) are not computed: their scores are -inf.
// Interface of helios::attn::indexer_score (reference: src/cuda/attn/attn.cu:182-273).
#pragma once

namespace hk {

constexpr int IP_THREADS = 320;                               // 8 epilogue warps, producer warp, issuing warp
constexpr int IP_EPI = 256;
constexpr int IP_ROWS = 2 * IX_RG;                              // query rows per CTA
constexpr uint32_t IP_A_BLK = IX_TILE_P * 128;                  // one 64-channel block of a pool tile: 16 KB
constexpr uint32_t IP_B_BLK = IX_RG * IX_HEADS * 128;           // one 64-channel block of a query group: 32 KB
constexpr uint32_t IP_A_BYTES = 2 * IP_A_BLK, IP_B_BYTES = 2 * IP_B_BLK;
constexpr uint32_t IP_OFF_A = 2 * IP_B_BYTES;                   // two pool-tile stages behind the two query groups
constexpr uint32_t IP_OFF_W = IP_OFF_A + 2 * IP_A_BYTES;        // head weights [16][32] f32, positions [16]
constexpr size_t IP_SMEM = IP_OFF_W + IP_ROWS * IX_HEADS * 4 + IP_ROWS * 4 + 1024;   // + slack to align to 1 KB

__device__ __forceinline__ void ip_tma_rows(void* smem_dst, const CUtensorMap* tmap, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          tc::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(0), "r"(row), "r"(0), "r"(tc::smem_u32(bar))
      : "memory");
}

template <int FMT>
__global__ __launch_bounds__(IP_THREADS, 1) void indexer_tc_prefill_kernel(
    const __grid_constant__ CUtensorMap tmap_pk, const __grid_constant__ CUtensorMap tmap_q, const uint16_t* __restrict__ w,
    const int* __restrict__ q_pos, __half* __restrict__ scores, int m, int npools, int score_stride, int tiles_per_cta,
    int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t ip_smem_raw[];
  uint8_t* smem = ip_smem_raw + ((1024u - (tc::smem_u32(ip_smem_raw) & 1023u)) & 1023u);
  float* w_sm = reinterpret_cast<float*>(smem + IP_OFF_W);        // [16][32]
  int* pos_sm = reinterpret_cast<int*>(w_sm + IP_ROWS * IX_HEADS);   // [16]
  __shared__ uint64_t b_full, a_full[2], a_free[2], acc_full[2], acc_free[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp_u = tc::warp_index_uniform();
  const int r_begin = blockIdx.y * IP_ROWS;
  const int nr_total = min(IP_ROWS, m - r_begin);
  const int n_grp = nr_total > IX_RG ? 2 : 1;
  const int tiles_total = (npools + IX_TILE_P - 1) / IX_TILE_P;
  const int t0 = blockIdx.x * tiles_per_cta, t1 = min(tiles_total, t0 + tiles_per_cta);

  if (tid == 0) {
    tc::mbar_init(&b_full, 1);
#pragma unroll
    for (int b = 0; b < 2; b++) {
      tc::mbar_init(&a_full[b], 1);
      tc::mbar_init(&a_free[b], 1);
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_free[b], IP_EPI);
    }
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp_u == 0) tc::tmem_alloc(&tmem_slot, 512);
  for (int j = tid; j < nr_total * IX_HEADS; j += IP_THREADS) {
    const uint16_t wb = w[(size_t)r_begin * IX_HEADS + j];
    w_sm[j] = FMT == tc::FMT_BF16 ? bf16_bits_to_f(wb) : __half2float(__ushort_as_half(wb));
  }
  if (tid < IP_ROWS) pos_sm[tid] = tid < nr_total ? q_pos[r_begin + tid] : -1;
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  // tiles [t0, t_vis) are visible to at least one row of the CTA: tile t holds pools 128 t ..., the first of which
  // needs position >= 512 t + 3
  int max_pos = -1;
#pragma unroll
  for (int j = 0; j < IP_ROWS; j++) max_pos = max(max_pos, pos_sm[j]);
  const int t_vis = max_pos >= 3 ? max(t0, min(t1, (max_pos - 3) / (IX_TILE_P * POOL) + 1)) : t0;
  const int n_tiles = t_vis - t0;
  bool ok = true;

  if (warp_u == 8) {
    // ---- producer ----
    if (lane == 0 && n_tiles > 0) {
      tc::mbar_arrive_expect_tx(&b_full, 2 * IP_B_BYTES);
      ip_tma_rows(smem, &tmap_q, r_begin * IX_HEADS, &b_full);
      ip_tma_rows(smem + IP_B_BYTES, &tmap_q, (r_begin + IX_RG) * IX_HEADS, &b_full);
      for (int i = 0; i < n_tiles; i++) {
        const int s = i & 1;
        if (i >= 2) ok = tc::mbar_wait<20>(&a_free[s], ((i - 2) >> 1) & 1, &abort_flag, 11);
        if (!ok) break;
        tc::mbar_arrive_expect_tx(&a_full[s], IP_A_BYTES);
        ip_tma_rows(smem + IP_OFF_A + s * IP_A_BYTES, &tmap_pk, (t0 + i) * IX_TILE_P, &a_full[s]);
      }
    }
  } else if (warp_u == 9) {
    // ---- tensor-core issue: every lane runs the loop, the elected lane issues ----
    const uint32_t leader = tc::elect_one();
    auto wait_u = [&](uint64_t* bar, uint32_t parity, int code) {
      const bool done = tc::mbar_wait<20>(bar, parity, &abort_flag, code);
      return __all_sync(0xffffffffu, done) != 0;
    };
    const uint32_t idesc = tc::make_idesc(IX_TILE_P, IX_RG * IX_HEADS, FMT, FMT, false, false);
    if (n_tiles > 0) ok = wait_u(&b_full, 0, 12);
    for (int i = 0; i < n_tiles && ok; i++) {
      const int s = i & 1;
      ok = wait_u(&a_full[s], (i >> 1) & 1, 13) && ok;
      const uint64_t ad0 = tc::make_sdesc_sw128(tc::smem_u32(smem + IP_OFF_A + s * IP_A_BYTES), 16, 1024);
      for (int g = 0; g < n_grp && ok; g++) {
        if (i >= 1) ok = wait_u(&acc_free[g], (i - 1) & 1, 14) && ok;
        if (!ok) break;
        tc::fence_after_sync();
        const uint64_t bd0 = tc::make_sdesc_sw128(tc::smem_u32(smem + g * IP_B_BYTES), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < IDX_DIM / 16; kk++)
          tc::mma_f16_if(leader, tmem + g * 256, tc::sdesc_advance(ad0, (kk >> 2) * IP_A_BLK + (kk & 3) * 32),
                         tc::sdesc_advance(bd0, (kk >> 2) * IP_B_BLK + (kk & 3) * 32), idesc, kk > 0);
        tc::mma_commit_if(leader, &acc_full[g]);
      }
      tc::mma_commit_if(leader, &a_free[s]);       // both products have read the pool tile
    }
  } else {
    // ---- epilogue warps 0-7: TMEM lane = pool, warp w: lane quarter w % 4, rows 4 (w / 4) .. + 3 of the group ----
    const int lq = warp_u & 3, rhalf = warp_u >> 2;
    const int pl = lq * 32 + lane;                              // pool inside the tile
    for (int i = 0; i < n_tiles; i++) {
      const int p = (t0 + i) * IX_TILE_P + pl;
      for (int g = 0; g < n_grp; g++) {
        ok = tc::mbar_wait<20>(&acc_full[g], i & 1, &abort_flag, 15) && ok;
        tc::fence_after_sync();
        const int row0 = g * IX_RG + rhalf * 4;                 // first of this warp's four rows (CTA-relative)
        if (ok && row0 < nr_total) {
          uint32_t c[4][32];
#pragma unroll
          for (int u = 0; u < 4; u++) tc::tmem_ld32(tmem + ((uint32_t)(lq * 32) << 16) + g * 256 + (rhalf * 4 + u) * IX_HEADS, c[u]);
          tc::tmem_ld_wait();
          float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int h4 = 0; h4 < IX_HEADS / 4; h4++) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const float4 ww = reinterpret_cast<const float4*>(w_sm + (row0 + u) * IX_HEADS)[h4];
              // per row the same operation order as the serial kernel: d = c * 128^-1/2, tot += w * relu(d)
              tot[u] = fmaf(ww.x, fmaxf(__uint_as_float(c[u][4 * h4 + 0]) * 0.08838834764f, 0.f), tot[u]);
              tot[u] = fmaf(ww.y, fmaxf(__uint_as_float(c[u][4 * h4 + 1]) * 0.08838834764f, 0.f), tot[u]);
              tot[u] = fmaf(ww.z, fmaxf(__uint_as_float(c[u][4 * h4 + 2]) * 0.08838834764f, 0.f), tot[u]);
              tot[u] = fmaf(ww.w, fmaxf(__uint_as_float(c[u][4 * h4 + 3]) * 0.08838834764f, 0.f), tot[u]);
            }
          }
          if (p < npools) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              if (row0 + u < nr_total) {
                const bool vis = p * POOL + POOL - 1 <= pos_sm[row0 + u];
                scores[(size_t)(r_begin + row0 + u) * score_stride + p] =
                    vis ? __float2half_rn(tot[u] * 0.17677669530f) : __ushort_as_half((unsigned short)0xfc00);
              }
            }
          }
        }
        tc::fence_before_sync();
        tc::mbar_arrive(&acc_free[g]);
      }
    }
    // tiles that none of the rows may see yet
    for (int t = t_vis; t < t1; t++) {
      const int p = t * IX_TILE_P + pl;
      if (p < npools)
        for (int rr = rhalf; rr < nr_total; rr += 2)
          scores[(size_t)(r_begin + rr) * score_stride + p] = __ushort_as_half((unsigned short)0xfc00);
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (warp_u == 0) tc::tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

// tensor map over rows of 128 16-bit elements viewed as [row][2 blocks][64]: box {64, box_rows, 2}, 128-byte swizzle
static bool ip_encode_rows(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows, bool bf16) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
  if (!encode) return false;
  memset(map, 0, sizeof(*map));
  const cuuint64_t dims[3] = {64, rows, 2};
  const cuuint64_t strides[2] = {IDX_DIM * 2, 128};
  const cuuint32_t box[3] = {64, box_rows, 2};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims,
                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// returns HK_ERR_UNSUPPORTED when the copy-engine form cannot be set up (the caller then uses the serial kernel)
static int indexer_prefill_launch(const void* q_idx, const void* pool_k_nt, const void* w, const int* q_pos, void* scores, int m,
                                  int npools, int score_stride, int dtype, cudaStream_t s) {
  static const bool disabled = getenv("HK_INDEXER_SERIAL") != nullptr;    // debug switch: the serial kernel only
  if (disabled) return HK_ERR_UNSUPPORTED;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return HK_ERR_UNSUPPORTED;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(indexer_tc_prefill_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IP_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(indexer_tc_prefill_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IP_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  alignas(64) CUtensorMap map_pk, map_q;
  if (!ip_encode_rows(&map_pk, pool_k_nt, (uint64_t)npools, IX_TILE_P, dtype == HK_BF16) ||
      !ip_encode_rows(&map_q, q_idx, (uint64_t)m * IX_HEADS, IX_RG * IX_HEADS, dtype == HK_BF16))
    return HK_ERR_UNSUPPORTED;
  // grid = (pool splits, row pairs of 16): the number of pool splits with the fewest tile steps on the busiest SM
  const int tiles = (npools + IX_TILE_P - 1) / IX_TILE_P;
  const int pairs = (m + IP_ROWS - 1) / IP_ROWS;
  const int sms = sm_count();
  int best_split = 1;
  long best_cost = -1;
  for (int ns = 1; ns <= tiles && ns <= 64; ns++) {
    const int tps = (tiles + ns - 1) / ns;
    const long waves = ((long)pairs * ((tiles + tps - 1) / tps) + sms - 1) / sms;
    const long cost = waves * (tps + 3);                      // + the resident operand's load, in tile steps
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_split = ns; }
  }
  const int tiles_per_cta = (tiles + best_split - 1) / best_split;
  dim3 grid((tiles + tiles_per_cta - 1) / tiles_per_cta, pairs);
  const int rows_per_cta = tiles_per_cta;                      // (kernel argument: pool tiles per CTA)
  int* st = device_status_ptr();
  if (dtype == HK_F16)
    indexer_tc_prefill_kernel<0><<<grid, IP_THREADS, IP_SMEM, s>>>(map_pk, map_q, (const uint16_t*)w, q_pos, (__half*)scores, m, npools,
                                                                  score_stride, rows_per_cta, st);
  else
    indexer_tc_prefill_kernel<1><<<grid, IP_THREADS, IP_SMEM, s>>>(map_pk, map_q, (const uint16_t*)w, q_pos, (__half*)scores, m, npools,
                                                                  score_stride, rows_per_cta, st);
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

}  // namespace hk
