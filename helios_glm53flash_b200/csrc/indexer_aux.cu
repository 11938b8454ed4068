// DSA indexer, the small kernels: pooled-key writer, pool->token expansion and the scalar
// cross-check scorer.  Interfaces of helios::attn::kpool_write / pool_expand / pool_expand_row /
// indexer_score_legacy (reference: src/cuda/attn/attn.cu:134-158, :284-390).
#include "hk_common.cuh"
#include "kpool_common.cuh"

namespace hk {

// One CTA per pool touched by this call, one thread per channel (body: kpool_common.cuh).
__global__ __launch_bounds__(128) void kpool_write_kernel(
    const __half* __restrict__ ik, const __half* __restrict__ ig, __half* __restrict__ ring,
    int raw_rows, __half* __restrict__ pk_nt, const float* __restrict__ ape, int pos_start,
    int n_new, int first_pool) {
  kpool_one(ik, ig, ring, raw_rows, pk_nt, ape, pos_start, n_new, first_pool + blockIdx.x, threadIdx.x);
}

// raw[r][4i+j] = 4*pool_i + j if <= cur else -1; raw[r][4*n_sel + i] = cur-3+i (>= 0) - the tail
// is appended without de-duplication, exactly as the reference does.
__global__ void pool_expand_kernel(const int* __restrict__ pidx, const int* __restrict__ q_pos,
                                   int* __restrict__ raw, int cur_pos, int n_sel) {
  const int r = blockIdx.x;
  const int cur = q_pos ? q_pos[r] : cur_pos;
  int4* row = reinterpret_cast<int4*>(raw + (size_t)r * (n_sel * POOL + POOL));
  for (int i = threadIdx.x; i <= n_sel; i += blockDim.x) {
    int4 v;
    if (i < n_sel) {
      const int pi = pidx[(size_t)r * n_sel + i];
      const int t = pi * POOL;
      v.x = (pi >= 0 && t + 0 <= cur) ? t + 0 : -1;
      v.y = (pi >= 0 && t + 1 <= cur) ? t + 1 : -1;
      v.z = (pi >= 0 && t + 2 <= cur) ? t + 2 : -1;
      v.w = (pi >= 0 && t + 3 <= cur) ? t + 3 : -1;
    } else {
      v.x = cur - 3 >= 0 ? cur - 3 : -1;
      v.y = cur - 2 >= 0 ? cur - 2 : -1;
      v.z = cur - 1 >= 0 ? cur - 1 : -1;
      v.w = cur >= 0 ? cur : -1;
    }
    row[i] = v;
  }
}

// Scalar scorer over the transposed [128][pk_stride] plane: thread per pool, fp32 accumulation.
__global__ __launch_bounds__(256) void indexer_legacy_kernel(
    const __half* __restrict__ qi, const __half* __restrict__ pk, const __half* __restrict__ w,
    const int* __restrict__ q_pos, __half* __restrict__ scores, int npools, int pk_stride) {
  const int r = blockIdx.y;
  const int p = blockIdx.x * 256 + threadIdx.x;
  __shared__ __half q_sm[32 * 128];
  __shared__ float w_sm[32];
  for (int i = threadIdx.x; i < 32 * 128; i += 256) q_sm[i] = qi[(size_t)r * 32 * 128 + i];
  if (threadIdx.x < 32) w_sm[threadIdx.x] = __half2float(w[(size_t)r * 32 + threadIdx.x]);
  __syncthreads();
  if (p >= npools) return;
  if (p * POOL + POOL - 1 > q_pos[r]) {
    scores[(size_t)r * npools + p] = __ushort_as_half((unsigned short)0xfc00);
    return;
  }
  float kreg[128];
#pragma unroll
  for (int d = 0; d < 128; d++) kreg[d] = __half2float(pk[(size_t)d * pk_stride + p]);
  float total = 0.f;
  for (int h = 0; h < 32; h++) {
    float dot = 0.f;
#pragma unroll
    for (int d = 0; d < 128; d++) dot += kreg[d] * __half2float(q_sm[h * 128 + d]);
    dot *= 0.08838834764f;
    if (dot > 0.f) total += w_sm[h] * dot;
  }
  scores[(size_t)r * npools + p] = __float2half_rn(total * 0.17677669530f);
}

}  // namespace hk

HK_API int hk_kpool_write(const void* idx_k, const void* idx_g, void* raw_ring, int raw_rows,
                          void* pool_k_nt, const float* ape, int pos_start, int n_new,
                          void* stream) {
  using namespace hk;
  HK_REQUIRE(idx_k && idx_g && raw_ring && pool_k_nt && ape);
  HK_REQUIRE(raw_rows > 0 && pos_start >= 0 && n_new >= 0);
  if (n_new == 0) return HK_OK;
  // a completed pool reads back at most 3 rows written by earlier calls; they must still be there
  HK_REQUIRE(raw_rows >= n_new + (POOL - 1) || raw_rows >= pos_start + n_new);
  const int first_pool = pos_start / POOL;
  const int last_pool = (pos_start + n_new - 1) / POOL;
  kpool_write_kernel<<<last_pool - first_pool + 1, 128, 0, as_stream(stream)>>>(
      (const __half*)idx_k, (const __half*)idx_g, (__half*)raw_ring, raw_rows, (__half*)pool_k_nt,
      ape, pos_start, n_new, first_pool);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_pool_expand(const int* pool_idx, const int* q_pos, int* raw_idx, int m, int cur_pos,
                          int n_sel, void* stream) {
  using namespace hk;
  HK_REQUIRE(pool_idx && raw_idx && m >= 0 && n_sel > 0);
  HK_REQUIRE(aligned(raw_idx, 16));
  if (m == 0) return HK_OK;
  pool_expand_kernel<<<m, 256, 0, as_stream(stream)>>>(pool_idx, q_pos, raw_idx, cur_pos, n_sel);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_indexer_score_legacy(const void* q_idx, const void* pool_k, const void* w,
                                   const int* q_pos, void* scores, int m, int npools,
                                   int pk_stride, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_idx && pool_k && w && q_pos && scores && m >= 0 && npools >= 0 && pk_stride >= npools);
  if (m == 0 || npools == 0) return HK_OK;
  dim3 grid((npools + 255) / 256, m);
  indexer_legacy_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      (const __half*)q_idx, (const __half*)pool_k, (const __half*)w, q_pos, (__half*)scores, npools,
      pk_stride);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
