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

// dim = 512: lane owns the float4 columns lane, lane + 32, lane + 64, lane + 96
__global__ void __launch_bounds__(256) mla_cache_append_kernel(const float* __restrict__ kv_pre,
                                                               const __half* __restrict__ ln_w,
                                                               __half* __restrict__ ckv, __half* __restrict__ ckv_new,
                                                               long long pos, int n, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= n) return;
  const float4* xr = reinterpret_cast<const float4*>(kv_pre + (size_t)row * LATENT);
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
  uint2* dst = reinterpret_cast<uint2*>(ckv + (size_t)(pos + row) * LATENT);
  uint2* dst2 = ckv_new ? reinterpret_cast<uint2*>(ckv_new + (size_t)row * LATENT) : nullptr;
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

__global__ void __launch_bounds__(256) layernorm_f16_kernel(const __half* x, const __half* __restrict__ w,   // x and y may alias
                                                            const __half* __restrict__ b, __half* y,
                                                            int rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const __half* xr = x + (size_t)row * dim;
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
  __half* yr = y + (size_t)row * dim;
  for (int i = lane; i < dim; i += 32) {
    float v = (__half2float(xr[i]) - mean) * inv * __half2float(w[i]) + __half2float(b[i]);
    yr[i] = __float2half_rn(v);
  }
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
