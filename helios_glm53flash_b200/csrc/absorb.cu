// Absorbed MLA projections either side of the attention: q_lat = q_nope * W_uk (256 -> 512) and
// o = lat_out * W_uv^T (512 -> 256), per head, plus the one-off W_uv transpose.  Interfaces of
// helios::attn::q_latent / q_latent_t / o_absorb / o_absorb_t / wuv_transpose
// (reference: src/cuda/attn/attn.cu:12-130).  The entry points run the tensor-core GEMM of absorb_tc.cu;
// the plain CUDA-core kernels below (fp32 accumulation, one block per (row, head)) are the cross-check
// (HK_ABSORB_FORCE_SIMT=1) and the path for buffers the tensor copies cannot address (not 16-byte aligned).
#include <cstdlib>

#include "hk_common.cuh"

namespace hk {

int absorb_gemm_tc(const void* a, const void* b, void* out, int n_rows, int K, int n_out, bool b_mn,
                   uint64_t b_rows, uint64_t b_cols, int b_rows_per_head, int b_row_off, cudaStream_t s);

static bool absorb_force_simt() {
  static const bool v = getenv("HK_ABSORB_FORCE_SIMT") != nullptr;
  return v;
}

// kv_b is the raw [64*512][512] fp16 tensor: rows h*512 .. +255 = W_uk[h], +256 .. +511 = W_uv[h].
// grid (m, 64), 256 threads: thread t owns output columns 2t, 2t+1; q row staged in shared memory.
__global__ __launch_bounds__(256) void q_latent_kernel(const __half* __restrict__ qn,
                                                       const __half* __restrict__ kb,
                                                       __half* __restrict__ ql) {
  const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
  __shared__ float q_sm[256];
  q_sm[t] = __half2float(qn[((size_t)r * 64 + h) * 256 + t]);
  __syncthreads();
  const __half2* w = reinterpret_cast<const __half2*>(kb + (size_t)h * 512 * 512) + t;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
  for (int j = 0; j < 256; j++) {
    float2 wv = __half22float2(w[(size_t)j * 256]);
    a0 = fmaf(q_sm[j], wv.x, a0);
    a1 = fmaf(q_sm[j], wv.y, a1);
  }
  reinterpret_cast<__half2*>(ql + ((size_t)r * 64 + h) * 512)[t] = __floats2half2_rn(a0, a1);
}

// wuv_t[h][c][j] = kv_b[h*512 + 256 + j][c]   ([64][512][256])
__global__ __launch_bounds__(256) void wuv_transpose_kernel(const __half* __restrict__ kb,
                                                            __half* __restrict__ wt) {
  __shared__ __half tile[32][33];
  const int h = blockIdx.z, j0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) tile[i][tx] = kb[((size_t)h * 512 + 256 + j0 + i) * 512 + c0 + tx];
  __syncthreads();
  for (int i = ty; i < 32; i += 8) wt[((size_t)h * 512 + c0 + i) * 256 + j0 + tx] = tile[tx][i];
}

// o[r,h,j] = sum_c lat[r,h,c] * wuv_t[h][c][j]; grid (n, 64), 128 threads x 2 columns
__global__ __launch_bounds__(128) void o_absorb_t_kernel(const __half* __restrict__ lat,
                                                         const __half* __restrict__ wt,
                                                         __half* __restrict__ o) {
  const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
  __shared__ float l_sm[512];
  for (int i = t; i < 512; i += 128) l_sm[i] = __half2float(lat[((size_t)r * 64 + h) * 512 + i]);
  __syncthreads();
  const __half2* w = reinterpret_cast<const __half2*>(wt + (size_t)h * 512 * 256) + t;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
  for (int c = 0; c < 512; c++) {
    float2 wv = __half22float2(w[(size_t)c * 128]);
    a0 = fmaf(l_sm[c], wv.x, a0);
    a1 = fmaf(l_sm[c], wv.y, a1);
  }
  reinterpret_cast<__half2*>(o + ((size_t)r * 64 + h) * 256)[t] = __floats2half2_rn(a0, a1);
}

// same result from the untransposed weights: warp per output column, lanes stride the 512 latents
__global__ __launch_bounds__(256) void o_absorb_kernel(const __half* __restrict__ lat,
                                                       const __half* __restrict__ kb,
                                                       __half* __restrict__ o) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __shared__ float l_sm[512];
  for (int i = threadIdx.x; i < 512; i += 256) l_sm[i] = __half2float(lat[((size_t)r * 64 + h) * 512 + i]);
  __syncthreads();
  for (int j = wid; j < 256; j += 8) {
    const __half* wr = kb + ((size_t)h * 512 + 256 + j) * 512;
    float a = 0.f;
#pragma unroll
    for (int c = lane; c < 512; c += 32) a = fmaf(l_sm[c], __half2float(wr[c]), a);
    a = warp_sum(a);
    if (lane == 0) o[((size_t)r * 64 + h) * 256 + j] = __float2half_rn(a);
  }
}

}  // namespace hk

HK_API int hk_q_latent(const void* q_nope, const void* kv_b, void* q_lat, int m, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_nope && kv_b && q_lat && m >= 0);
  if (m == 0) return HK_OK;
  if (!absorb_force_simt()) {   // q_nope [m][64*256] x W_uk[h] = kv_b rows h*512 .. +255, [k][n] with n contiguous
    const int st = absorb_gemm_tc(q_nope, kv_b, q_lat, m, 256, 512, true, 64 * 512, 512, 512, 0, as_stream(stream));
    if (st != HK_ERR_UNSUPPORTED) return st;
  }
  q_latent_kernel<<<dim3(m, 64), 256, 0, as_stream(stream)>>>((const __half*)q_nope, (const __half*)kv_b, (__half*)q_lat);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_o_absorb(const void* lat_out, const void* kv_b, void* o, int m, void* stream) {
  using namespace hk;
  HK_REQUIRE(lat_out && kv_b && o && m >= 0);
  if (m == 0) return HK_OK;
  if (!absorb_force_simt()) {   // lat_out [m][64*512] x W_uv[h]^T: kv_b rows h*512+256 .. +511 are [n][k], k contiguous
    const int st = absorb_gemm_tc(lat_out, kv_b, o, m, 512, 256, false, 64 * 512, 512, 512, 256, as_stream(stream));
    if (st != HK_ERR_UNSUPPORTED) return st;
  }
  o_absorb_kernel<<<dim3(m, 64), 256, 0, as_stream(stream)>>>((const __half*)lat_out, (const __half*)kv_b, (__half*)o);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_wuv_transpose(const void* kv_b, void* wuv_t, void* stream) {
  using namespace hk;
  HK_REQUIRE(kv_b && wuv_t);
  wuv_transpose_kernel<<<dim3(16, 8, 64), 256, 0, as_stream(stream)>>>((const __half*)kv_b, (__half*)wuv_t);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_o_absorb_t(const void* lat_out, const void* wuv_t, void* o, int nrows, void* stream) {
  using namespace hk;
  HK_REQUIRE(lat_out && wuv_t && o && nrows >= 0);
  if (nrows == 0) return HK_OK;
  if (!absorb_force_simt()) {   // lat_out [n][64*512] x wuv_t[h] = [512 k][256 n], n contiguous
    const int st = absorb_gemm_tc(lat_out, wuv_t, o, nrows, 512, 256, true, 64 * 512, 256, 512, 0, as_stream(stream));
    if (st != HK_ERR_UNSUPPORTED) return st;
  }
  o_absorb_t_kernel<<<dim3(nrows, 64), 128, 0, as_stream(stream)>>>((const __half*)lat_out, (const __half*)wuv_t, (__half*)o);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
