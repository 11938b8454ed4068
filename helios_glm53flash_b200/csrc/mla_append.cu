// The two small producers in front of the MLA / indexer caches:
//   * hk_mla_cache_append: RMS norm of the new compressed-KV rows (fp32 in, fp16 weight) written straight
//     into the latent cache at their positions (the reference normalises into a staging buffer and copies
//     it: aux::rms_norm + cudaMemcpyAsync, src/engine/runner.cpp:569-572);
//   * hk_layernorm_f16: layer norm with weight and bias over the indexer key rows
//     (glue::layernorm_f16, src/engine/glue2.cu:420-455).
// One warp per row.  The reference uses 128 threads per row (4 warps); a lane here plays the same lane of
// those four warps in turn and the four warp sums are combined in the reference's order
// ((s0 + s2) + (s1 + s3)), so the results are the same bits.
#include "hk_common.cuh"
#include "kpool_common.cuh"

namespace hk {
namespace {

__device__ __forceinline__ float4 half4_to_float4(uint2 r) {
  const __half2 a = *reinterpret_cast<const __half2*>(&r.x), b = *reinterpret_cast<const __half2*>(&r.y);
  return make_float4(__half2float(__low2half(a)), __half2float(__high2half(a)), __half2float(__low2half(b)),
                     __half2float(__high2half(b)));
}

__device__ __forceinline__ uint2 float4_to_half4(float4 v) {
  const __half2 a = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y));
  const __half2 b = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&a);
  r.y = *reinterpret_cast<const uint32_t*>(&b);
  return r;
}

// dim = 512, one warp: lane owns the float4 columns lane, lane + 32, lane + 64, lane + 96
__device__ __forceinline__ void append_row(const float* __restrict__ kv_row, const __half* __restrict__ ln_w,
                                           __half* __restrict__ dst_row, __half* __restrict__ dst2_row, float eps, int lane) {
  const float4* xr = reinterpret_cast<const float4*>(kv_row);
  float4 x[4];
  float s[4];
#pragma unroll
  for (int w = 0; w < 4; w++) x[w] = xr[w * 32 + lane];
#pragma unroll
  for (int w = 0; w < 4; w++) {
    float t = 0.f;
    t = fmaf(x[w].x, x[w].x, t);
    t = fmaf(x[w].y, x[w].y, t);
    t = fmaf(x[w].z, x[w].z, t);
    t = fmaf(x[w].w, x[w].w, t);
    s[w] = warp_sum(t);
  }
  const float sum = (s[0] + s[2]) + (s[1] + s[3]);
  const float rmf = rsqrtf(sum / (float)LATENT + eps) * 1.0f;
  uint2* dst = reinterpret_cast<uint2*>(dst_row);
  uint2* dst2 = dst2_row ? reinterpret_cast<uint2*>(dst2_row) : nullptr;
#pragma unroll
  for (int w = 0; w < 4; w++) {
    const float4 w4 = half4_to_float4(reinterpret_cast<const uint2*>(ln_w)[w * 32 + lane]);
    float4 o;
    o.x = x[w].x * w4.x * rmf;
    o.y = x[w].y * w4.y * rmf;
    o.z = x[w].z * w4.z * rmf;
    o.w = x[w].w * w4.w * rmf;
    const uint2 p = float4_to_half4(o);
    dst[w * 32 + lane] = p;
    if (dst2) dst2[w * 32 + lane] = p;
  }
}

__global__ void __launch_bounds__(256) mla_cache_append_kernel(const float* __restrict__ kv_pre,
                                                               const __half* __restrict__ ln_w,
                                                               __half* __restrict__ ckv, __half* __restrict__ ckv_new,
                                                               long long pos, int n, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= n) return;
  append_row(kv_pre + (size_t)row * LATENT, ln_w, ckv + (size_t)(pos + row) * LATENT,
             ckv_new ? ckv_new + (size_t)row * LATENT : nullptr, eps, lane);
}

// one warp; xr and yr may alias; y2 (optional) receives the same row (any address space)
__device__ __forceinline__ void layernorm_row(const __half* xr, const __half* __restrict__ w, const __half* __restrict__ b,
                                              __half* yr, __half* y2, int dim, float eps, int lane) {
  float s1[4], s2[4];
#pragma unroll
  for (int q = 0; q < 4; q++) {                            // lane `lane` of the reference's warp q
    float sum = 0, sq = 0;
    for (int i = q * 32 + lane; i < dim; i += 128) {
      float v = __half2float(xr[i]);
      sum += v; sq += v * v;
    }
    s1[q] = warp_sum(sum);
    s2[q] = warp_sum(sq);
  }
  const float a = (s1[0] + s1[2]) + (s1[1] + s1[3]), c = (s2[0] + s2[2]) + (s2[1] + s2[3]);
  const float m0 = a / dim, m1 = c / dim;
  float mean = m0, var = m1 - mean * mean;
  float inv = rsqrtf(var + eps);
  for (int i = lane; i < dim; i += 32) {
    float v = (__half2float(xr[i]) - mean) * inv * __half2float(w[i]) + __half2float(b[i]);
    const __half h = __float2half_rn(v);
    if (yr) yr[i] = h;
    if (y2) y2[i] = h;
  }
}

__global__ void __launch_bounds__(256) layernorm_f16_kernel(const __half* x, const __half* __restrict__ w,   // x and y may alias
                                                            const __half* __restrict__ b, __half* y,
                                                            int rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  layernorm_row(x + (size_t)row * dim, w, b, y + (size_t)row * dim, nullptr, dim, eps, lane);
}

// Everything an MLA layer does with ONE new token before its attention, in one launch of one CTA: the latent row is
// normalised into the cache (warp 0), the indexer key row is layer-normalised (warp 1, kept in shared memory), then
// the 128 threads write the key || gate row into the ring and, if this token completes its pool, the pooled key.  The
// reference's decode runs rms_norm + copy, layernorm_f16 and kpool_write here (src/engine/runner.cpp:569-584).
__global__ void __launch_bounds__(128) mla_decode_prologue_kernel(
    const float* __restrict__ kv_pre, const __half* __restrict__ ln_w, __half* __restrict__ ckv, float eps_rms,
    const __half* __restrict__ idx_k, const __half* __restrict__ knorm_w, const __half* __restrict__ knorm_b,
    __half* __restrict__ idx_kn, float eps_ln, const __half* __restrict__ idx_g, __half* __restrict__ ring, int raw_rows,
    __half* __restrict__ pk_nt, const float* __restrict__ ape, int pos, int* __restrict__ q_pos_out) {
  __shared__ __half s_kn[128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp == 0) append_row(kv_pre, ln_w, ckv + (size_t)pos * LATENT, nullptr, eps_rms, lane);
  if (warp == 1) layernorm_row(idx_k, knorm_w, knorm_b, idx_kn, s_kn, 128, eps_ln, lane);
  if (threadIdx.x == 64 && q_pos_out) *q_pos_out = pos;
  __syncthreads();
  kpool_one(s_kn, idx_g, ring, raw_rows, pk_nt, ape, pos, 1, pos / POOL, threadIdx.x);
}

}  // namespace
}  // namespace hk

HK_API int hk_mla_cache_append(const float* kv_pre, const void* ln_w_f16, void* ckv, void* ckv_new,
                               long long pos, int n, float epsilon, void* stream) {
  HK_REQUIRE(kv_pre && ln_w_f16 && ckv && pos >= 0 && n >= 0);
  HK_REQUIRE(hk::aligned(kv_pre, 16) && hk::aligned(ln_w_f16, 8) && hk::aligned(ckv, 8) &&
             (!ckv_new || hk::aligned(ckv_new, 8)));
  if (n == 0) return HK_OK;
  hk::mla_cache_append_kernel<<<(n + 7) / 8, 256, 0, hk::as_stream(stream)>>>(
      kv_pre, static_cast<const __half*>(ln_w_f16), static_cast<__half*>(ckv), static_cast<__half*>(ckv_new), pos, n,
      epsilon);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_layernorm_f16(const void* x, const void* w, const void* b, void* y, int rows, int dim,
                            float epsilon, void* stream) {
  HK_REQUIRE(x && w && b && y && rows >= 0 && dim > 0);
  if (rows == 0) return HK_OK;
  hk::layernorm_f16_kernel<<<(rows + 7) / 8, 256, 0, hk::as_stream(stream)>>>(
      static_cast<const __half*>(x), static_cast<const __half*>(w), static_cast<const __half*>(b),
      static_cast<__half*>(y), rows, dim, epsilon);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_mla_decode_prologue(const float* kv_pre, const void* ln_w_f16, void* ckv, float eps_rms, const void* idx_k,
                                  const void* knorm_w, const void* knorm_b, void* idx_kn, float eps_ln, const void* idx_g,
                                  void* raw_ring, int raw_rows, void* pool_k_nt, const float* ape, int pos, int* q_pos_out,
                                  void* stream) {
  HK_REQUIRE(kv_pre && ln_w_f16 && ckv && idx_k && knorm_w && knorm_b && idx_g && raw_ring && pool_k_nt && ape);
  HK_REQUIRE(pos >= 0 && raw_rows > 0 && (raw_rows >= hk::POOL || raw_rows >= pos + 1));
  HK_REQUIRE(hk::aligned(kv_pre, 16) && hk::aligned(ln_w_f16, 8) && hk::aligned(ckv, 8));
  hk::mla_decode_prologue_kernel<<<1, 128, 0, hk::as_stream(stream)>>>(
      kv_pre, static_cast<const __half*>(ln_w_f16), static_cast<__half*>(ckv), eps_rms, static_cast<const __half*>(idx_k),
      static_cast<const __half*>(knorm_w), static_cast<const __half*>(knorm_b), static_cast<__half*>(idx_kn), eps_ln,
      static_cast<const __half*>(idx_g), static_cast<__half*>(raw_ring), raw_rows, static_cast<__half*>(pool_k_nt), ape, pos,
      q_pos_out);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
