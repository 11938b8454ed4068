// KDA short convolution: depthwise causal conv (window K) + SiLU over channel-major input, with a
// rolling window state.  Interface and arithmetic of helios::aux::cuda_causal_conv1d_update
// (reference: src/cuda/aux/gdn.cu:880-1023): fp32 fma chain k ascending, SiLU as a * 1/(1+exp(-a)),
// bf16 round-to-nearest output, state = last K inputs.
//
// Four kernels (the last one is the fused cast + convolution over token-major fp32 input, further below):
//   conv4_row_kernel   prefill with whole 16-token groups: K = 4, no history, seqlen % 16 == 0.  No
//                      shared memory: a lane keeps 2 channels x 16 (or 32) tokens in registers (32-byte reads
//                      per channel row, 128-byte warp stores per output row).
//   conv4_tile_kernel  other prefill lengths: a CTA transposes a [64 channel][128 token] tile
//                      through shared memory: 16-byte coalesced reads along tokens (the input is
//                      channel-major), 128-byte coalesced writes along channels (the output is
//                      token-major).  HBM-bound: 2 B read + 2 B written per channel-token.
//   conv_generic_kernel decode and every other case (any K <= 16, history, ragged shapes): one
//                      thread per channel; with seqlen = 1 its accesses are contiguous in channels.
#include "hk_common.cuh"

namespace hk {

constexpr int CONV_MAX_K = 16;
constexpr int CT_CH = 64;       // channels per tile
constexpr int CT_TOK = 128;     // tokens per tile
constexpr int CT_STRIDE = 138;  // bf16 elements per shared row: 8 halo slots + 128 tokens + 2 pad
                                // (69 words, odd, so channel-strided reads spread over the banks)

__device__ __forceinline__ float silu_fast(float a) { return a * (1.0f / (1.0f + __expf(-a))); }

template <bool ACT, bool VEC>
__global__ __launch_bounds__(256) void conv4_tile_kernel(
    const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ state,
    const int* __restrict__ slots, const __nv_bfloat16* __restrict__ weight,
    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int dim, int seqlen,
    int state_size) {
  __shared__ __align__(16) __nv_bfloat16 xs[CT_CH * CT_STRIDE];
  const int d0 = blockIdx.x * CT_CH;
  const int s0 = blockIdx.y * CT_TOK;
  const int b = blockIdx.z;
  const int tid = threadIdx.x;
  const __nv_bfloat16* xb = x + ((size_t)b * dim + d0) * seqlen;

  // ---- stage the tile: rows = channels, 8 tokens per 16-byte load ----
  if (VEC) {
    for (int idx = tid; idx < CT_CH * (CT_TOK / 8); idx += 256) {
      int r = idx >> 4, c = idx & 15;
      int s = s0 + c * 8;
      if (s < seqlen) {
        uint4 v = ld_stream16(xb + (size_t)r * seqlen + s);
        uint32_t* dst = reinterpret_cast<uint32_t*>(xs + r * CT_STRIDE + 8 + c * 8);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
      }
    }
  } else {
    for (int idx = tid; idx < CT_CH * CT_TOK; idx += 256) {
      int r = idx >> 7, c = idx & 127;
      int s = s0 + c;
      if (s < seqlen) xs[r * CT_STRIDE + 8 + c] = xb[(size_t)r * seqlen + s];
    }
  }
  // ---- halo (3 tokens before the tile) and, in the first tile, the state update ----
  if (tid < CT_CH) {
    const int r = tid;
    __nv_bfloat16* hrow = xs + r * CT_STRIDE + 5;
    if (s0 == 0) {
      const int slot = slots ? slots[b] : b;
      __nv_bfloat16* st = state + ((size_t)slot * dim + d0 + r) * state_size;
      __nv_bfloat16 old[4] = {st[0], st[1], st[2], st[3]};
      hrow[0] = old[1]; hrow[1] = old[2]; hrow[2] = old[3];
      // new window = last 4 entries of [old(4) | x(seqlen)]
#pragma unroll
      for (int k = 0; k < 4; k++) {
        int src_t = seqlen + k;
        st[k] = (src_t < 4) ? old[src_t] : xb[(size_t)r * seqlen + (src_t - 4)];
      }
    } else {
#pragma unroll
      for (int h = 0; h < 3; h++) hrow[h] = xb[(size_t)r * seqlen + (s0 - 3 + h)];
    }
  }
  __syncthreads();

  // ---- compute: lane owns 2 adjacent channels, warp owns 16 consecutive tokens ----
  const int lane = tid & 31, wid = tid >> 5;
  const int c0 = lane * 2;
  const uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)(d0 + c0) * 4);
  const float w00 = bf16lo(wv.x), w01 = bf16hi(wv.x), w02 = bf16lo(wv.y), w03 = bf16hi(wv.y);
  const float w10 = bf16lo(wv.z), w11 = bf16hi(wv.z), w12 = bf16lo(wv.w), w13 = bf16hi(wv.w);
  float b0 = 0.f, b1 = 0.f;
  if (bias) {
    b0 = __bfloat162float(bias[d0 + c0]);
    b1 = __bfloat162float(bias[d0 + c0 + 1]);
  }
  const __nv_bfloat16* r0 = xs + c0 * CT_STRIDE + 8;
  const __nv_bfloat16* r1 = r0 + CT_STRIDE;
  const int t0 = wid * 16;
  float a0 = __bfloat162float(r0[t0 - 3]), a1 = __bfloat162float(r0[t0 - 2]), a2 = __bfloat162float(r0[t0 - 1]);
  float e0 = __bfloat162float(r1[t0 - 3]), e1 = __bfloat162float(r1[t0 - 2]), e2 = __bfloat162float(r1[t0 - 1]);
  __nv_bfloat16* ob = out + ((size_t)b * seqlen) * dim + d0 + c0;
#pragma unroll 4
  for (int t = t0; t < t0 + 16; t++) {
    if (s0 + t >= seqlen) break;
    float a3 = __bfloat162float(r0[t]), e3 = __bfloat162float(r1[t]);
    float y0 = fmaf(w03, a3, fmaf(w02, a2, fmaf(w01, a1, fmaf(w00, a0, b0))));
    float y1 = fmaf(w13, e3, fmaf(w12, e2, fmaf(w11, e1, fmaf(w10, e0, b1))));
    if (ACT) {
      y0 = silu_fast(y0);
      y1 = silu_fast(y1);
    }
    __nv_bfloat162 pk;
    pk.x = __float2bfloat16_rn(y0);
    pk.y = __float2bfloat16_rn(y1);
    *reinterpret_cast<__nv_bfloat162*>(ob + (size_t)(s0 + t) * dim) = pk;
    a0 = a1; a1 = a2; a2 = a3;
    e0 = e1; e1 = e2; e2 = e3;
  }
}

// Prefill with whole 16-token groups (seqlen % 16 == 0): no shared memory at all.  A lane owns 2 adjacent
// channels and 16 consecutive tokens: it reads 32 contiguous bytes per channel row (full sectors), keeps
// the 19 inputs per channel in registers and writes 4 bytes per token, so that a warp's store covers 128
// contiguous bytes of one output row.  Same arithmetic as above, about half the instructions per output.
template <bool ACT, int NG>   // NG groups of 16 consecutive tokens per lane
__global__ __launch_bounds__(256) void conv4_row_kernel(
    const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ state,
    const int* __restrict__ slots, const __nv_bfloat16* __restrict__ weight,
    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int dim, int seqlen,
    int state_size) {
  constexpr int NT = 16 * NG;                                // tokens per lane
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CT_CH + lane * 2;
  const int t0 = (blockIdx.y * 8 + wid) * NT;
  const int b = blockIdx.z;
  if (t0 >= seqlen) return;                                  // warp-uniform
  const __nv_bfloat16* r0 = x + ((size_t)b * dim + c0) * seqlen;
  const __nv_bfloat16* r1 = r0 + seqlen;
  uint4 ra[2 * NG], re[2 * NG];                              // all loads of the lane are issued before any use
#pragma unroll
  for (int j = 0; j < 2 * NG; j++) {
    ra[j] = ld_stream16(r0 + t0 + 8 * j);
    re[j] = ld_stream16(r1 + t0 + 8 * j);
  }
  float xa[NT + 3], xe[NT + 3];                              // inputs t0-3 .. t0+NT-1 of the two channels
  if (t0 == 0) {
    // the first group takes its 3 predecessors from the window state and rolls the state forward
    const int slot = slots ? slots[b] : b;
    __nv_bfloat16* st0 = state + ((size_t)slot * dim + c0) * state_size;
    __nv_bfloat16* st1 = st0 + state_size;
#pragma unroll
    for (int h = 0; h < 3; h++) {
      xa[h] = __bfloat162float(st0[h + 1]);
      xe[h] = __bfloat162float(st1[h + 1]);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {                            // seqlen >= 16: the new window is the last 4 inputs
      st0[k] = r0[seqlen - 4 + k];
      st1[k] = r1[seqlen - 4 + k];
    }
  } else {
    const uint2 pa = *reinterpret_cast<const uint2*>(r0 + t0 - 4);   // tokens t0-4 .. t0-1
    const uint2 pe = *reinterpret_cast<const uint2*>(r1 + t0 - 4);
    xa[0] = bf16hi(pa.x); xa[1] = bf16lo(pa.y); xa[2] = bf16hi(pa.y);
    xe[0] = bf16hi(pe.x); xe[1] = bf16lo(pe.y); xe[2] = bf16hi(pe.y);
  }
#pragma unroll
  for (int j = 0; j < 2 * NG; j++) {
    const uint32_t wa[4] = {ra[j].x, ra[j].y, ra[j].z, ra[j].w};
    const uint32_t we[4] = {re[j].x, re[j].y, re[j].z, re[j].w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      xa[3 + 8 * j + 2 * i] = bf16lo(wa[i]); xa[4 + 8 * j + 2 * i] = bf16hi(wa[i]);
      xe[3 + 8 * j + 2 * i] = bf16lo(we[i]); xe[4 + 8 * j + 2 * i] = bf16hi(we[i]);
    }
  }
  const uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)c0 * 4);
  const float w00 = bf16lo(wv.x), w01 = bf16hi(wv.x), w02 = bf16lo(wv.y), w03 = bf16hi(wv.y);
  const float w10 = bf16lo(wv.z), w11 = bf16hi(wv.z), w12 = bf16lo(wv.w), w13 = bf16hi(wv.w);
  float b0 = 0.f, b1 = 0.f;
  if (bias) {
    b0 = __bfloat162float(bias[c0]);
    b1 = __bfloat162float(bias[c0 + 1]);
  }
  __nv_bfloat16* ob = out + ((size_t)b * seqlen + t0) * dim + c0;
#pragma unroll
  for (int i = 0; i < NT; i++) {
    float y0 = fmaf(w03, xa[i + 3], fmaf(w02, xa[i + 2], fmaf(w01, xa[i + 1], fmaf(w00, xa[i], b0))));
    float y1 = fmaf(w13, xe[i + 3], fmaf(w12, xe[i + 2], fmaf(w11, xe[i + 1], fmaf(w10, xe[i], b1))));
    if (ACT) {
      y0 = silu_fast(y0);
      y1 = silu_fast(y1);
    }
    __nv_bfloat162 pk;
    pk.x = __float2bfloat16_rn(y0);
    pk.y = __float2bfloat16_rn(y1);
    *reinterpret_cast<__nv_bfloat162*>(ob + (size_t)i * dim) = pk;
  }
}

template <bool ACT, bool HISTORY>
__global__ __launch_bounds__(256) void conv_generic_kernel(
    const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ state,
    const int* __restrict__ slots, const __nv_bfloat16* __restrict__ weight,
    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int dim, int seqlen,
    int state_size, int K) {
  const int d = blockIdx.x * 256 + threadIdx.x;
  if (d >= dim) return;
  const int b = blockIdx.y;
  const int slot = slots ? slots[b] : b;
  const __nv_bfloat16* x_d = x + ((size_t)b * dim + d) * seqlen;
  __nv_bfloat16* st = state + ((size_t)slot * dim + d) * state_size;
  float w[CONV_MAX_K], old[CONV_MAX_K], win[CONV_MAX_K];
#pragma unroll
  for (int k = 0; k < CONV_MAX_K; k++)
    if (k < K) {
      w[k] = __bfloat162float(weight[(size_t)d * K + k]);
      old[k] = __bfloat162float(st[k]);
    }
#pragma unroll
  for (int k = 0; k < CONV_MAX_K - 1; k++)
    if (k < K - 1) win[k] = old[k + 1];
  const float bias_d = bias ? __bfloat162float(bias[d]) : 0.0f;
  for (int s = 0; s < seqlen; s++) {
    float cur = __bfloat162float(x_d[s]);
    float acc = bias_d;
#pragma unroll
    for (int k = 0; k < CONV_MAX_K; k++)
      if (k < K) acc = fmaf(w[k], (k == K - 1) ? cur : win[k], acc);
    if (ACT) acc = silu_fast(acc);
    out[((size_t)b * seqlen + s) * dim + d] = __float2bfloat16_rn(acc);
#pragma unroll
    for (int k = 0; k < CONV_MAX_K - 1; k++)
      if (k < K - 1) win[k] = (k == K - 2) ? cur : win[k + 1];
  }
  if (!HISTORY) {
#pragma unroll
    for (int k = 0; k < CONV_MAX_K; k++)
      if (k < K) {
        int src_t = seqlen + k;
        float v = (src_t < K) ? old[src_t] : __bfloat162float(x_d[src_t - K]);
        st[k] = __float2bfloat16_rn(v);
      }
  } else {
    int total = K + seqlen;
    int write_size = state_size < total ? state_size : total;
    int dst_start = state_size - write_size, src_start = total - write_size;
    for (int j = 0; j < write_size; j++) {
      int src_t = src_start + j;
      float v = (src_t < K) ? old[src_t] : __bfloat162float(x_d[src_t - K]);
      st[dst_start + j] = __float2bfloat16_rn(v);
    }
  }
}


// Cast + convolution in one pass over TOKEN-major fp32 input (the projection's own output layout): the
// transposed bf16 copy that the channel-major kernels read is never made.  A thread owns 4 adjacent
// channels (one 16-byte load per token; a warp reads 512 contiguous bytes of a token row and writes 256)
// and walks CR_TOK consecutive tokens with the three previous inputs in registers.  Inputs are rounded
// to bf16 first, so the result equals transpose-cast followed by the channel-major convolution, bit for
// bit.  x [bsz][seqlen][dim] f32, out [bsz][seqlen][dim] bf16, state [slots][dim][4] bf16.
constexpr int CR_TOK = 64;

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <bool ACT>
__global__ __launch_bounds__(128) void conv4_cast_rows_kernel(
    const float* __restrict__ x, __nv_bfloat16* __restrict__ state, const int* __restrict__ slots,
    const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ bias,
    __nv_bfloat16* __restrict__ out, int dim, int seqlen) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 4;
  if (c >= dim) return;
  const int s0 = blockIdx.y * CR_TOK, b = blockIdx.z;
  const int s1 = min(s0 + CR_TOK, seqlen);
  const float* xb = x + (size_t)b * seqlen * dim + c;
  float w[4][4], bs[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const uint4 w01 = *reinterpret_cast<const uint4*>(weight + (size_t)c * 4);
    const uint4 w23 = *reinterpret_cast<const uint4*>(weight + (size_t)c * 4 + 8);
    const uint32_t ww[8] = {w01.x, w01.y, w01.z, w01.w, w23.x, w23.y, w23.z, w23.w};
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
      w[ch][0] = bf16lo(ww[2 * ch]); w[ch][1] = bf16hi(ww[2 * ch]);
      w[ch][2] = bf16lo(ww[2 * ch + 1]); w[ch][3] = bf16hi(ww[2 * ch + 1]);
    }
    if (bias) {
#pragma unroll
      for (int ch = 0; ch < 4; ch++) bs[ch] = __bfloat162float(bias[c + ch]);
    }
  }
  float h0[4], h1[4], h2[4];                                // inputs s-3, s-2, s-1 of the four channels
  if (s0 == 0) {
    // the first segment takes its predecessors from the window state and rolls the state forward
    const int slot = slots ? slots[b] : b;
    __nv_bfloat16* st = state + ((size_t)slot * dim + c) * 4;
    const uint4 o01 = *reinterpret_cast<const uint4*>(st), o23 = *reinterpret_cast<const uint4*>(st + 8);
    const uint32_t ow[8] = {o01.x, o01.y, o01.z, o01.w, o23.x, o23.y, o23.z, o23.w};
    uint32_t nw[8];
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
      const float old[4] = {bf16lo(ow[2 * ch]), bf16hi(ow[2 * ch]), bf16lo(ow[2 * ch + 1]), bf16hi(ow[2 * ch + 1])};
      h0[ch] = old[1]; h1[ch] = old[2]; h2[ch] = old[3];
      float nv[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {                          // new window = last 4 of [old | x]
        const int src_t = seqlen + k;
        nv[k] = src_t < 4 ? old[src_t] : xb[(size_t)(src_t - 4) * dim + ch];
      }
      nw[2 * ch] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(nv[0])) |
                   ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(nv[1])) << 16);
      nw[2 * ch + 1] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(nv[2])) |
                       ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(nv[3])) << 16);
    }
    *reinterpret_cast<uint4*>(st) = make_uint4(nw[0], nw[1], nw[2], nw[3]);
    *reinterpret_cast<uint4*>(st + 8) = make_uint4(nw[4], nw[5], nw[6], nw[7]);
  } else {
    const float4 p0 = *reinterpret_cast<const float4*>(xb + (size_t)(s0 - 3) * dim);
    const float4 p1 = *reinterpret_cast<const float4*>(xb + (size_t)(s0 - 2) * dim);
    const float4 p2 = *reinterpret_cast<const float4*>(xb + (size_t)(s0 - 1) * dim);
    h0[0] = round_bf16(p0.x); h0[1] = round_bf16(p0.y); h0[2] = round_bf16(p0.z); h0[3] = round_bf16(p0.w);
    h1[0] = round_bf16(p1.x); h1[1] = round_bf16(p1.y); h1[2] = round_bf16(p1.z); h1[3] = round_bf16(p1.w);
    h2[0] = round_bf16(p2.x); h2[1] = round_bf16(p2.y); h2[2] = round_bf16(p2.z); h2[3] = round_bf16(p2.w);
  }
  __nv_bfloat16* ob = out + (size_t)b * seqlen * dim + c;
  for (int t0 = s0; t0 < s1; t0 += 8) {
    uint4 raw[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
      raw[j] = t0 + j < s1 ? ld_stream16(xb + (size_t)(t0 + j) * dim) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (t0 + j >= s1) break;
      const float cur[4] = {round_bf16(__uint_as_float(raw[j].x)), round_bf16(__uint_as_float(raw[j].y)),
                            round_bf16(__uint_as_float(raw[j].z)), round_bf16(__uint_as_float(raw[j].w))};
      float y[4];
#pragma unroll
      for (int ch = 0; ch < 4; ch++) {
        y[ch] = fmaf(w[ch][3], cur[ch], fmaf(w[ch][2], h2[ch], fmaf(w[ch][1], h1[ch], fmaf(w[ch][0], h0[ch], bs[ch]))));
        if (ACT) y[ch] = silu_fast(y[ch]);
        h0[ch] = h1[ch]; h1[ch] = h2[ch]; h2[ch] = cur[ch];
      }
      uint2 pk;
      pk.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y[1])) << 16);
      pk.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y[3])) << 16);
      *reinterpret_cast<uint2*>(ob + (size_t)(t0 + j) * dim) = pk;
    }
  }
}

}  // namespace hk

HK_API int hk_kda_cast_conv(const float* x, void* conv_state, const int* slots, const void* weight,
                            const void* bias, void* out, int bsz, int dim, int seqlen, int activation,
                            void* stream) {
  using namespace hk;
  HK_REQUIRE(x && conv_state && weight && out);
  HK_REQUIRE(bsz > 0 && bsz <= 65535 && dim > 0 && dim % 4 == 0 && seqlen > 0);
  HK_REQUIRE((seqlen + CR_TOK - 1) / CR_TOK <= 65535);
  HK_REQUIRE(aligned(x, 16) && aligned(conv_state, 16) && aligned(weight, 16) && aligned(out, 8));
  dim3 grid((dim / 4 + 127) / 128, (seqlen + CR_TOK - 1) / CR_TOK, bsz);
  auto st = (__nv_bfloat16*)conv_state;
  auto w = (const __nv_bfloat16*)weight;
  auto bs = (const __nv_bfloat16*)bias;
  auto o = (__nv_bfloat16*)out;
  if (activation) conv4_cast_rows_kernel<true><<<grid, 128, 0, as_stream(stream)>>>(x, st, slots, w, bs, o, dim, seqlen);
  else            conv4_cast_rows_kernel<false><<<grid, 128, 0, as_stream(stream)>>>(x, st, slots, w, bs, o, dim, seqlen);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_conv1d_update(const void* x, void* conv_state, const int* slots, const void* weight,
                            const void* bias, void* out, int bsz, int dim, int seqlen,
                            int state_size, int K, int activation, int history, void* stream) {
  using namespace hk;
  HK_REQUIRE(x && conv_state && weight && out);
  HK_REQUIRE(bsz > 0 && dim > 0 && seqlen > 0);
  HK_REQUIRE(K >= 1 && K <= CONV_MAX_K && state_size >= K);
  auto xs = (const __nv_bfloat16*)x;
  auto st = (__nv_bfloat16*)conv_state;
  auto w = (const __nv_bfloat16*)weight;
  auto bs = (const __nv_bfloat16*)bias;
  auto o = (__nv_bfloat16*)out;
  cudaStream_t s = as_stream(stream);

  const bool tile_ok = (K == 4) && !history && (dim % CT_CH == 0) && seqlen >= 16 &&
                       aligned(weight, 16) && aligned(out, 4);
  if (tile_ok && seqlen % 16 == 0 && aligned(x, 16)) {
    // one 16-token group per lane: two groups (NG = 2) measured slower (419 vs 367 us at 32K tokens), fewer warps per SM

    dim3 grid(dim / CT_CH, (seqlen + CT_TOK - 1) / CT_TOK, bsz);
    if (activation) conv4_row_kernel<true, 1><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
    else            conv4_row_kernel<false, 1><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
  } else if (tile_ok) {
    dim3 grid(dim / CT_CH, (seqlen + CT_TOK - 1) / CT_TOK, bsz);
    const bool vec = (seqlen % 8 == 0) && aligned(x, 16);
    if (activation) {
      if (vec) conv4_tile_kernel<true, true><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
      else     conv4_tile_kernel<true, false><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
    } else {
      if (vec) conv4_tile_kernel<false, true><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
      else     conv4_tile_kernel<false, false><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size);
    }
  } else {
    dim3 grid((dim + 255) / 256, bsz);
    if (activation) {
      if (history) conv_generic_kernel<true, true><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size, K);
      else         conv_generic_kernel<true, false><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size, K);
    } else {
      if (history) conv_generic_kernel<false, true><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size, K);
      else         conv_generic_kernel<false, false><<<grid, 256, 0, s>>>(xs, st, slots, w, bs, o, dim, seqlen, state_size, K);
    }
  }
  HK_LAUNCH_CHECK();
  return HK_OK;
}
