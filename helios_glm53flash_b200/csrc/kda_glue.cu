// The elementwise producers and the consumer either side of the KDA recurrence:
//   * transpose + cast of the projected q|k|v rows (fp32, token-major) into the channel-major bf16 input
//     of the short convolution,
//   * gate preparation: beta = sigmoid(b), g = lower_bound * sigmoid(exp(a_log[h]) * (f + dt_bias)),
//   * gated RMS norm of the recurrence output: y = x * w * rsqrt(mean(x^2) + eps) * act(gate).
// All three are bound by HBM bandwidth: every element is read once and written once, with 16-byte
// accesses per lane wherever the layout allows.  The arithmetic keeps the reference's operation order
// (and this library is compiled with the same fast-math flags), so the results are the same bits.
#include "hk_common.cuh"
#include "kda_norm_common.cuh"

namespace hk {
namespace {

// ---------------------------------------------------------------------------------------------
// src [S][F] fp32 -> dst [F][S] bf16 (round to nearest even).  One CTA moves a 64 x 64 tile: rows of
// 256 B in, rows of 128 B out.
// ---------------------------------------------------------------------------------------------
constexpr int TT = 64;

__global__ void __launch_bounds__(256) transpose_cast_kernel(const float* __restrict__ src,
                                                             __nv_bfloat16* __restrict__ dst, int S, int F) {
  __shared__ float tile[TT][TT + 1];
  const int s0 = blockIdx.y * TT, f0 = blockIdx.x * TT;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; j++) {
    const int s = s0 + ty + 4 * j, f = f0 + tx;
    v[j] = (s < S && f < F) ? __ldg(src + (size_t)s * F + f) : 0.f;
  }
#pragma unroll
  for (int j = 0; j < 16; j++) tile[ty + 4 * j][tx] = v[j];
  __syncthreads();
  // lane -> two neighbouring tokens of one channel: a warp writes one 128-byte row of dst
  const int sp = threadIdx.x & 31, fr = threadIdx.x >> 5;
  const bool pair_ok = (S % 2 == 0);                      // 4-byte stores need even row starts
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int f = f0 + fr + 8 * j, s = s0 + 2 * sp;
    if (f >= F || s >= S) continue;
    const float a = tile[2 * sp][fr + 8 * j], b = tile[2 * sp + 1][fr + 8 * j];
    __nv_bfloat16* o = dst + (size_t)f * S + s;
    if (pair_ok) {
      *reinterpret_cast<__nv_bfloat162*>(o) = __halves2bfloat162(__float2bfloat16(a), __float2bfloat16(b));
    } else {
      o[0] = __float2bfloat16(a);
      if (s + 1 < S) o[1] = __float2bfloat16(b);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Gate preparation, four channels per thread.  g and f are [S][H][Dk] fp32, b and beta [S][H].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gate_kernel(const float* __restrict__ b, const float* __restrict__ f,
                                                   const float* __restrict__ dt_bias,
                                                   const float* __restrict__ a_log, float lb,
                                                   __nv_bfloat16* __restrict__ beta, float* __restrict__ g,
                                                   size_t n_quads, int HD4, int Dk4, size_t n_beta) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t i0 = first; i0 < n_quads; i0 += 4 * stride) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const size_t i = i0 + u * stride;
      raw[u] = i < n_quads ? ld_stream16(reinterpret_cast<const float4*>(f) + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const size_t i = i0 + u * stride;
      if (i >= n_quads) break;
      const int rem = (int)(i % HD4), hh = rem / Dk4;
      const float decay = __expf(__ldg(a_log + hh));
      const float4 bias = __ldg(reinterpret_cast<const float4*>(dt_bias) + rem);
      float4 o;
      o.x = gate_value(__uint_as_float(raw[u].x), bias.x, decay, lb);
      o.y = gate_value(__uint_as_float(raw[u].y), bias.y, decay, lb);
      o.z = gate_value(__uint_as_float(raw[u].z), bias.z, decay, lb);
      o.w = gate_value(__uint_as_float(raw[u].w), bias.w, decay, lb);
      reinterpret_cast<float4*>(g)[i] = o;
    }
  }
  for (size_t j = first; j < n_beta; j += stride)
    beta[j] = __float2bfloat16(1.0f / (1.0f + __expf(-b[j])));
}

// scalar form for head dims that are not a multiple of four
__global__ void __launch_bounds__(256) gate_scalar_kernel(const float* __restrict__ b, const float* __restrict__ f,
                                                          const float* __restrict__ dt_bias,
                                                          const float* __restrict__ a_log, float lb,
                                                          __nv_bfloat16* __restrict__ beta, float* __restrict__ g,
                                                          size_t n, int HD, int Dk, size_t n_beta) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t i = first; i < n; i += stride) {
    const int rem = (int)(i % HD);
    g[i] = gate_value(f[i], dt_bias[rem], __expf(a_log[rem / Dk]), lb);
  }
  for (size_t j = first; j < n_beta; j += stride)
    beta[j] = __float2bfloat16(1.0f / (1.0f + __expf(-b[j])));
}

// ---------------------------------------------------------------------------------------------
// Gated RMS norm.
// ---------------------------------------------------------------------------------------------
// dim <= 256: one warp per row, one group of four channels per lane (two when dim > 128: TWO), rows in a
// grid-stride loop.  A warp works on sets of ROWS rows and keeps two sets in registers: the loads of the
// next set are in flight while the current one is normalised, so that memory and arithmetic overlap
// inside every warp.
template <typename G, int ROWS, bool TWO>
struct NormRows {
  uint2 x0[ROWS], x1[ROWS];
  decltype(raw4(static_cast<const G*>(nullptr))) g0[ROWS], g1[ROWS];

  __device__ __forceinline__ void load(const __nv_bfloat16* __restrict__ x, const G* __restrict__ g, long long r0,
                                       long long rows, int dim, int lane, bool c0, bool c1) {
#pragma unroll
    for (int i = 0; i < ROWS; i++) {
      const long long r = r0 + i;
      const bool ok = r < rows;
      zero_raw(x0[i]); zero_raw(g0[i]);
      if (TWO) { zero_raw(x1[i]); zero_raw(g1[i]); }
      if (ok && c0) {
        x0[i] = raw4(x + r * dim + 4 * lane);
        g0[i] = raw4(g + r * dim + 4 * lane);
      }
      if (TWO && ok && c1) {
        x1[i] = raw4(x + r * dim + 4 * (lane + 32));
        g1[i] = raw4(g + r * dim + 4 * (lane + 32));
      }
    }
  }
};

template <typename W, typename Y, typename G, int ROWS, bool TWO>
__global__ void __launch_bounds__(256, 3) gated_rms_norm_warp_kernel(
    const __nv_bfloat16* __restrict__ x, const W* __restrict__ w, Y* __restrict__ y, const G* __restrict__ g,
    float eps, long long rows, int dim, float cbias, int w_groups, int gate_first, int gate_act) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long step = (((long long)gridDim.x * blockDim.x) >> 5) * ROWS;
  const int columns = dim >> 2;
  const bool c0 = lane < columns, c1 = TWO && lane + 32 < columns;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // one weight row for all rows (the usual case): kept in registers
  const float4 wf0 = (w_groups == 1 && c0) ? load4(w + 4 * lane) : zero4;
  const float4 wf1 = (w_groups == 1 && c1) ? load4(w + 4 * (lane + 32)) : zero4;

  auto compute = [&](const NormRows<G, ROWS, TWO>& set, long long r0) {
#pragma unroll
    for (int i = 0; i < ROWS; i++) {
      const long long r = r0 + i;
      if (r >= rows) break;                                // uniform over the warp
      const float4 xa = cvt4(set.x0[i]), ga = cvt4(set.g0[i]);
      const float4 xb = TWO ? cvt4(set.x1[i]) : zero4, gb = TWO ? cvt4(set.g1[i]) : zero4;
      float4 a0 = xa, a1 = xb;
      if (gate_first) {
        a0.x *= act_gate(ga.x, gate_act);
        a0.y *= act_gate(ga.y, gate_act);
        a0.z *= act_gate(ga.z, gate_act);
        a0.w *= act_gate(ga.w, gate_act);
        a1.x *= act_gate(gb.x, gate_act);
        a1.y *= act_gate(gb.y, gate_act);
        a1.z *= act_gate(gb.z, gate_act);
        a1.w *= act_gate(gb.w, gate_act);
      }
      float s = 0.f;
      if (c0) s = sum_squares(s, a0);
      if (c1) s = sum_squares(s, a1);
      s = warp_sum(s);
      const float rmf = rsqrtf(s / (float)dim + eps);
      const W* wr = w;
      if (w_groups != 1) wr += (size_t)(r % w_groups) * dim;
      if (c0) {
        const float4 w4 = w_groups == 1 ? wf0 : load4(wr + 4 * lane);
        store4(y + r * dim + 4 * lane, finish4(xa, w4, ga, rmf, cbias, gate_first, gate_act));
      }
      if (c1) {
        const float4 w4 = w_groups == 1 ? wf1 : load4(wr + 4 * (lane + 32));
        store4(y + r * dim + 4 * (lane + 32), finish4(xb, w4, gb, rmf, cbias, gate_first, gate_act));
      }
    }
  };

  NormRows<G, ROWS, TWO> even, odd;
  long long r0 = warp0 * ROWS;
  if (r0 < rows) even.load(x, g, r0, rows, dim, lane, c0, c1);
  while (r0 < rows) {
    if (r0 + step < rows) odd.load(x, g, r0 + step, rows, dim, lane, c0, c1);
    compute(even, r0);
    r0 += step;
    if (r0 >= rows) break;
    if (r0 + step < rows) even.load(x, g, r0 + step, rows, dim, lane, c0, c1);
    compute(odd, r0);
    r0 += step;
  }
}

// dim > 256: one CTA of 1024 threads per row, columns strided over the threads, two-level sum (lanes,
// then warps) in the same order as the one-warp form.
template <typename W, typename Y, typename G>
__global__ void __launch_bounds__(1024) gated_rms_norm_block_kernel(
    const __nv_bfloat16* __restrict__ x, const W* __restrict__ w, Y* __restrict__ y, const G* __restrict__ g,
    float eps, int dim, float cbias, int w_groups, int gate_first, int gate_act) {
  __shared__ float sums[32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const size_t row = blockIdx.x;
  const int columns = dim >> 2;
  const W* wr = w + (size_t)(row % w_groups) * dim;
  float s = 0.f;
  for (int c = t; c < columns; c += 1024) {
    float4 x4 = load4(x + row * dim + 4 * c);
    if (gate_first) {
      const float4 g4 = load4(g + row * dim + 4 * c);
      x4.x *= act_gate(g4.x, gate_act);
      x4.y *= act_gate(g4.y, gate_act);
      x4.z *= act_gate(g4.z, gate_act);
      x4.w *= act_gate(g4.w, gate_act);
    }
    s = sum_squares(s, x4);
  }
  s = warp_sum(s);
  if (lane == 0) sums[warp] = s;
  __syncthreads();
  s = warp_sum(sums[lane]);
  const float rmf = rsqrtf(s / (float)dim + eps);
  for (int c = t; c < columns; c += 1024) {
    const float4 x4 = load4(x + row * dim + 4 * c);
    const float4 g4 = load4(g + row * dim + 4 * c);
    store4(y + row * dim + 4 * c, finish4(x4, load4(wr + 4 * c), g4, rmf, cbias, gate_first, gate_act));
  }
}

template <typename W, typename Y, typename G>
int launch_gated_rms_norm(const void* x, const void* w, void* y, const void* g, long long rows, int dim,
                          float eps, float cbias, int w_groups, int gate_first, int gate_act,
                          cudaStream_t st) {
  auto xp = static_cast<const __nv_bfloat16*>(x);
  auto wp = static_cast<const W*>(w);
  auto yp = static_cast<Y*>(y);
  auto gp = static_cast<const G*>(g);
  if (dim <= 256) {
    const int rows_per_warp = dim <= 128 ? 4 : 2;
    const long long warps_needed = (rows + rows_per_warp - 1) / rows_per_warp;
    const long long ctas_needed = (warps_needed + 7) / 8;
    const long long cap = (long long)sm_count() * 3;       // resident CTAs only: every warp streams many row sets
    const int grid = (int)(ctas_needed < cap ? ctas_needed : cap);
    if (dim <= 128)
      gated_rms_norm_warp_kernel<W, Y, G, 4, false><<<grid, 256, 0, st>>>(xp, wp, yp, gp, eps, rows, dim, cbias,
                                                                         w_groups, gate_first, gate_act);
    else
      gated_rms_norm_warp_kernel<W, Y, G, 2, true><<<grid, 256, 0, st>>>(xp, wp, yp, gp, eps, rows, dim, cbias,
                                                                        w_groups, gate_first, gate_act);
  } else {
    gated_rms_norm_block_kernel<W, Y, G><<<(unsigned)rows, 1024, 0, st>>>(xp, wp, yp, gp, eps, dim, cbias, w_groups,
                                                                          gate_first, gate_act);
  }
  HK_LAUNCH_CHECK();
  return HK_OK;
}

}  // namespace
}  // namespace hk

HK_API int hk_kda_transpose_cast(void* dst_bf16, const float* src, int S, int F, void* stream) {
  HK_REQUIRE(dst_bf16 && src && S >= 0 && F >= 0);
  if (S == 0 || F == 0) return HK_OK;
  HK_REQUIRE((F + hk::TT - 1) / hk::TT <= 2147483647 && (S + hk::TT - 1) / hk::TT <= 65535);
  HK_REQUIRE(hk::aligned(dst_bf16, 4));
  dim3 grid((F + hk::TT - 1) / hk::TT, (S + hk::TT - 1) / hk::TT);
  hk::transpose_cast_kernel<<<grid, 256, 0, hk::as_stream(stream)>>>(src, static_cast<__nv_bfloat16*>(dst_bf16), S, F);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_kda_gate(const float* b, const float* f, const float* dt_bias, const float* a_log,
                       float lower_bound, void* beta_bf16, float* g, int S, int H, int Dk, void* stream) {
  HK_REQUIRE(b && f && dt_bias && a_log && beta_bf16 && g && S >= 0 && H > 0 && Dk > 0);
  if (S == 0) return HK_OK;
  const size_t n = (size_t)S * H * Dk, n_beta = (size_t)S * H;
  auto beta = static_cast<__nv_bfloat16*>(beta_bf16);
  const bool vec = Dk % 4 == 0 && hk::aligned(f, 16) && hk::aligned(g, 16) && hk::aligned(dt_bias, 16);
  const size_t items = vec ? n / 4 : n;
  const size_t want = (items + 255) / 256, cap = (size_t)hk::sm_count() * 32;
  const int grid = (int)(want < cap ? want : cap);
  if (vec)
    hk::gate_kernel<<<grid, 256, 0, hk::as_stream(stream)>>>(b, f, dt_bias, a_log, lower_bound, beta, g, n / 4,
                                                             H * Dk / 4, Dk / 4, n_beta);
  else
    hk::gate_scalar_kernel<<<grid, 256, 0, hk::as_stream(stream)>>>(b, f, dt_bias, a_log, lower_bound, beta, g, n,
                                                                    H * Dk, Dk, n_beta);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                          const float* a_log, float lower_bound, void* mixed_qkv_bf16, void* beta_bf16,
                          float* g, int S, int F, int H, int Dk, void* stream) {
  const int rc = hk_kda_transpose_cast(mixed_qkv_bf16, qkv, S, F, stream);
  if (rc != HK_OK) return rc;
  return hk_kda_gate(b, f, dt_bias, a_log, lower_bound, beta_bf16, g, S, H, Dk, stream);
}

HK_API int hk_gated_rms_norm(const void* x, const void* w, int w_type, void* y, int y_type, const void* g,
                             int g_type, long long rows, int dim, float epsilon, float constant_bias,
                             int w_groups, int gate_first, int gate_act, void* stream) {
  HK_REQUIRE(x && w && y && g && rows >= 0 && dim > 0 && dim % 4 == 0 && w_groups >= 1);
  HK_REQUIRE(gate_act == 0 || gate_act == 1);
  HK_REQUIRE(w_type == HK_F32 || w_type == HK_BF16);
  HK_REQUIRE(y_type == HK_F32 || y_type == HK_F16);
  HK_REQUIRE(g_type == HK_F32 || g_type == HK_BF16);
  HK_REQUIRE(hk::aligned(x, 8) && hk::aligned(w, w_type == HK_F32 ? 16 : 8) &&
             hk::aligned(y, y_type == HK_F32 ? 16 : 8) && hk::aligned(g, g_type == HK_F32 ? 16 : 8));
  if (rows == 0) return HK_OK;
  HK_REQUIRE(dim <= 256 || rows <= 2147483647LL);
  cudaStream_t st = hk::as_stream(stream);
#define HK_NORM_CASE(WT, W, YT, Y, GT, G)                                                                  \
  if (w_type == WT && y_type == YT && g_type == GT)                                                        \
    return hk::launch_gated_rms_norm<W, Y, G>(x, w, y, g, rows, dim, epsilon, constant_bias, w_groups,     \
                                              gate_first, gate_act, st);
  HK_NORM_CASE(HK_F32, float, HK_F16, __half, HK_BF16, __nv_bfloat16)
  HK_NORM_CASE(HK_F32, float, HK_F32, float, HK_BF16, __nv_bfloat16)
  HK_NORM_CASE(HK_BF16, __nv_bfloat16, HK_F16, __half, HK_BF16, __nv_bfloat16)
  HK_NORM_CASE(HK_BF16, __nv_bfloat16, HK_F32, float, HK_BF16, __nv_bfloat16)
  HK_NORM_CASE(HK_F32, float, HK_F16, __half, HK_F32, float)
  HK_NORM_CASE(HK_F32, float, HK_F32, float, HK_F32, float)
  HK_NORM_CASE(HK_BF16, __nv_bfloat16, HK_F16, __half, HK_F32, float)
  HK_NORM_CASE(HK_BF16, __nv_bfloat16, HK_F32, float, HK_F32, float)
#undef HK_NORM_CASE
  return HK_ERR_INVALID;
}
