// KDA / gated-delta-rule recurrence, one token at a time: the decode step, short sequences and the
// history (rewindable) mode.  Interface and arithmetic of
// helios::aux::cuda_recurrent_gated_delta_rule (reference: src/cuda/aux/gdn.cu:555-866).
//
// Layout of the work: one CTA per (batch item, head, slice of NV value-columns).  The CTA's
// [D x NV] slice of the fp32 state lives in REGISTERS for the whole call (the reference re-reads and
// re-writes it from global memory on every token), so a decode step moves each state byte exactly
// once in and once out - the HBM floor of 2*H*D*D*4 bytes per layer-step - and a multi-token call
// costs state traffic only once.  Thread (kg, j) owns column j and the D/KG consecutive k-rows of
// group kg; the k-reduction is the sum of the KG group sums taken in ascending order, which for
// D = 128, NV = 32 is exactly the reference's 4 x 32 order (gdn.cu:683-705).
#include "hk_common.cuh"
#include "kda_norm_common.cuh"

namespace hk {

template <int D, int NV, bool CW, bool HIST>
__global__ __launch_bounds__(128) void kda_recurrent_kernel(
    const __nv_bfloat16* __restrict__ mixed_qkv, const float* __restrict__ g,
    const __nv_bfloat16* __restrict__ beta, float* __restrict__ state,
    __nv_bfloat16* __restrict__ out, float* __restrict__ out_f32, int seqlen, int Hk, int Hv,
    float scale, const int* __restrict__ slots, int history_stride) {
  constexpr int KG = 128 / NV;   // k-groups per CTA
  constexpr int RPT = D / KG;    // state rows per thread
  constexpr int NW = D / 32;     // warps that carry q/k channels
  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * NV;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = tid % NV, kg = tid / NV;
  const int group = Hv / Hk, k_head = head / group;
  const size_t row = (size_t)2 * Hk * D + (size_t)Hv * D;
  const size_t head_state = (size_t)D * D;
  const size_t state_size = (size_t)Hv * head_state;
  const int slot = slots ? slots[b] : b;
  float* slot_state = state + (size_t)slot * history_stride * state_size;
  float* my_state = slot_state + head * head_state + (size_t)(kg * RPT) * D + v0 + j;

  const __nv_bfloat16* tok = mixed_qkv + (size_t)b * seqlen * row;
  const float* gp = g + (size_t)b * seqlen * Hv * (CW ? D : 1) + (size_t)head * (CW ? D : 1);
  const __nv_bfloat16* bp = beta + (size_t)b * seqlen * Hv + head;
  const size_t out_base = ((size_t)b * seqlen * Hv + head) * D + v0 + j;

  __shared__ float sh_q[D], sh_k[D], sh_d[D];
  __shared__ float sh_red[2][4];
  __shared__ float sh_part[2][KG][NV];

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; i++) S[i] = my_state[(size_t)i * D];

  // software prefetch of the next token's operands
  float nq = 0.f, nk = 0.f, ng = 0.f, nv, nb;
  if (tid < D) {
    nq = __bfloat162float(tok[(size_t)k_head * D + tid]);
    nk = __bfloat162float(tok[(size_t)(Hk + k_head) * D + tid]);
    if (CW) ng = gp[tid];
  }
  if (!CW) ng = gp[0];
  nv = __bfloat162float(tok[(size_t)2 * Hk * D + (size_t)head * D + v0 + j]);
  nb = __bfloat162float(bp[0]);

  for (int s = 0; s < seqlen; s++) {
    float q = nq, k = nk, gv = ng, v = nv, beta_h = nb;
    if (s + 1 < seqlen) {
      const __nv_bfloat16* nt = tok + (size_t)(s + 1) * row;
      if (tid < D) {
        nq = __bfloat162float(nt[(size_t)k_head * D + tid]);
        nk = __bfloat162float(nt[(size_t)(Hk + k_head) * D + tid]);
        if (CW) ng = gp[(size_t)(s + 1) * Hv * D + tid];
      }
      if (!CW) ng = gp[(size_t)(s + 1) * Hv];
      nv = __bfloat162float(nt[(size_t)2 * Hk * D + (size_t)head * D + v0 + j]);
      nb = __bfloat162float(bp[(size_t)(s + 1) * Hv]);
    }
    // ---- L2 normalisation of q and k over the D channels ----
    float sq = warp_sum(q * q), sk = warp_sum(k * k);
    if (lane == 0 && warp < NW) {
      sh_red[0][warp] = sq;
      sh_red[1][warp] = sk;
    }
    __syncthreads();
    if (tid < D) {
      float tq = 0.f, tk = 0.f;
#pragma unroll
      for (int w = 0; w < NW; w++) {
        tq += sh_red[0][w];
        tk += sh_red[1][w];
      }
      sh_q[tid] = q * rsqrtf(tq + 1e-6f);
      sh_k[tid] = k * rsqrtf(tk + 1e-6f);
      if (CW) sh_d[tid] = __expf(gv);
    }
    __syncthreads();
    // ---- kv_j = sum_c k_c d_c S[c][j] (the state is read decayed when channelwise) ----
    const float g_h = CW ? 1.0f : __expf(gv);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < RPT; i++) {
      const int c = kg * RPT + i;
      if (CW) sum = sum + sh_k[c] * sh_d[c] * S[i];
      else    sum = sum + sh_k[c] * S[i];
    }
    sh_part[0][kg][j] = sum;
    __syncthreads();
    float kv = 0.f;
#pragma unroll
    for (int p = 0; p < KG; p++) kv = __fadd_rn(kv, sh_part[0][p][j]);
    const float vp = v - kv * g_h;
    // ---- S <- S*decay + k v' beta ;  o_j = sum_c q_c S[c][j] ----
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < RPT; i++) {
      const int c = kg * RPT + i;
      float st = S[i] * (CW ? sh_d[c] : g_h) + sh_k[c] * vp * beta_h;
      S[i] = st;
      o = o + sh_q[c] * st;
    }
    sh_part[1][kg][j] = o;
    if (HIST) {
      // step s writes history slot s+1; the last step writes the final slot 0
      float* dst = (s == seqlen - 1) ? my_state : my_state + (size_t)(s + 1) * state_size;
#pragma unroll
      for (int i = 0; i < RPT; i++) dst[(size_t)i * D] = S[i];
    }
    __syncthreads();
    if (kg == 0) {
      float tot = 0.f;
#pragma unroll
      for (int p = 0; p < KG; p++) tot = __fadd_rn(tot, sh_part[1][p][j]);
      tot *= scale;
      const size_t oi = out_base + (size_t)s * Hv * D;
      out[oi] = __float2bfloat16_rz(tot);
      if (out_f32) out_f32[oi] = tot;
    }
  }
  if (!HIST) {
#pragma unroll
    for (int i = 0; i < RPT; i++) my_state[(size_t)i * D] = S[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Decode step with the short convolution inside: x -> conv(K = 4) + SiLU -> bf16 q|k|v -> recurrence, one launch.
// The reference runs cuda_causal_conv1d_update and cuda_recurrent_gated_delta_rule back to back for every decoded
// token (src/engine/runner.cpp:443-471); at 2-3 us per launch the pair is bound by launch latency, not by the 4 MB
// of state.  Same grid as the recurrence, (batch, head, value slice): every CTA convolves the head's 128 q and 128 k
// channels itself (from the window state as it was before the call) and the value channels of its slice; the rolling
// window of the q / k channels is written back once, by whichever slice of the head is the LAST to have read it (a
// ticket counter per (batch, head) in caller memory; nobody waits for anybody).  Arithmetic and rounding are those of
// the two separate kernels, so results are bit-identical to calling them in turn.
// ---------------------------------------------------------------------------------------------
// window and taps of one channel arrive as one 8-byte load each
__device__ __forceinline__ float conv4_silu_bf16(uint2 st, uint2 w, float bias, float cur) {
  // fp32 fma chain over the window [st1, st2, st3, x], taps ascending; SiLU as a / (1 + exp(-a)); rounded to bf16
  float acc = bias;
  acc = fmaf(bf16lo(w.x), bf16hi(st.x), acc);
  acc = fmaf(bf16hi(w.x), bf16lo(st.y), acc);
  acc = fmaf(bf16lo(w.y), bf16hi(st.y), acc);
  acc = fmaf(bf16hi(w.y), cur, acc);
  acc = acc * (1.0f / (1.0f + __expf(-acc)));
  return __bfloat162float(__float2bfloat16_rn(acc));
}
// new window [st1, st2, st3, x]
__device__ __forceinline__ uint2 conv4_rolled(uint2 st, __nv_bfloat16 cur) {
  uint2 r;
  r.x = (st.x >> 16) | (st.y << 16);
  r.y = (st.y >> 16) | ((uint32_t)__bfloat16_as_ushort(cur) << 16);
  return r;
}

template <int NV>
__global__ __launch_bounds__(128) void kda_decode_conv_kernel(
    const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ conv_w,
    const __nv_bfloat16* __restrict__ conv_bias, const float* __restrict__ g, const __nv_bfloat16* __restrict__ beta,
    float* __restrict__ state, __nv_bfloat16* __restrict__ out, float* __restrict__ out_f32,
    __nv_bfloat16* __restrict__ conv_out, int H, float scale, const int* __restrict__ slots, int* __restrict__ tickets) {
  constexpr int D = 128;
  constexpr int KG = 128 / NV, RPT = D / KG;
  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * NV;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = tid % NV, kg = tid / NV;
  const int dim = 3 * H * D;
  const int slot = slots ? slots[b] : b;
  float* my_state = state + ((size_t)slot * H + head) * D * D + (size_t)(kg * RPT) * D + v0 + j;
  __shared__ float sh_q[D], sh_k[D], sh_d[D];
  __shared__ float sh_red[2][4];
  __shared__ float sh_part[2][KG][NV];
  __shared__ int sh_last;

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; i++) S[i] = my_state[(size_t)i * D];

  // ---- short convolution of this head's q and k channels (thread = channel) and of this slice's value channel j ----
  const __nv_bfloat16* xb = x + (size_t)b * dim;                       // [dim][1]
  __nv_bfloat16* cs = conv_state + (size_t)slot * dim * 4;
  const int cq = head * D + tid, ck = (H + head) * D + tid, cv = (2 * H + head) * D + v0 + j;
  const __nv_bfloat16 xq = xb[cq], xk = xb[ck], xv = xb[cv];
  const uint2 sq4 = *reinterpret_cast<const uint2*>(cs + (size_t)cq * 4), wq4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)cq * 4));
  const uint2 sk4 = *reinterpret_cast<const uint2*>(cs + (size_t)ck * 4), wk4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)ck * 4));
  const uint2 sv4 = *reinterpret_cast<const uint2*>(cs + (size_t)cv * 4), wv4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)cv * 4));
  const float q = conv4_silu_bf16(sq4, wq4, conv_bias ? __bfloat162float(conv_bias[cq]) : 0.f, __bfloat162float(xq));
  const float k = conv4_silu_bf16(sk4, wk4, conv_bias ? __bfloat162float(conv_bias[ck]) : 0.f, __bfloat162float(xk));
  const float v = conv4_silu_bf16(sv4, wv4, conv_bias ? __bfloat162float(conv_bias[cv]) : 0.f, __bfloat162float(xv));
  const float gv = g[((size_t)b * H + head) * D + tid];
  const float beta_h = __bfloat162float(beta[(size_t)b * H + head]);

  // ---- L2 normalisation of q and k over the D channels ----
  float sq = warp_sum(q * q), sk = warp_sum(k * k);
  if (lane == 0) {
    sh_red[0][warp] = sq;
    sh_red[1][warp] = sk;
  }
  __syncthreads();
  {
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      tq += sh_red[0][w];
      tk += sh_red[1][w];
    }
    sh_q[tid] = q * rsqrtf(tq + 1e-6f);
    sh_k[tid] = k * rsqrtf(tk + 1e-6f);
    sh_d[tid] = __expf(gv);
  }
  // every thread of this CTA has read the old q / k window (first barrier): thread 0 takes a ticket now and looks at it
  // at the end of the kernel, so the round trip of the atomic runs under the recurrence
  int ticket = 0;
  if (tid == 0) ticket = atomicAdd(tickets + (size_t)b * H + head, 1);
  __syncthreads();
  // the value window of this slice is private to the CTA: every thread has read it (barrier above)
  if (kg == 0) {
    *reinterpret_cast<uint2*>(cs + (size_t)cv * 4) = conv4_rolled(sv4, xv);
    if (conv_out) conv_out[(size_t)b * dim + cv] = __float2bfloat16_rn(v);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const int c = kg * RPT + i;
    sum = sum + sh_k[c] * sh_d[c] * S[i];
  }
  sh_part[0][kg][j] = sum;
  __syncthreads();
  float kv = 0.f;
#pragma unroll
  for (int p = 0; p < KG; p++) kv = __fadd_rn(kv, sh_part[0][p][j]);
  const float vp = v - kv;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const int c = kg * RPT + i;
    const float st = S[i] * sh_d[c] + sh_k[c] * vp * beta_h;
    S[i] = st;
    o = o + sh_q[c] * st;
  }
  sh_part[1][kg][j] = o;
  __syncthreads();
  if (kg == 0) {
    float tot = 0.f;
#pragma unroll
    for (int p = 0; p < KG; p++) tot = __fadd_rn(tot, sh_part[1][p][j]);
    tot *= scale;
    const size_t oi = ((size_t)b * H + head) * D + v0 + j;
    out[oi] = __float2bfloat16_rz(tot);
    if (out_f32) out_f32[oi] = tot;
  }
#pragma unroll
  for (int i = 0; i < RPT; i++) my_state[(size_t)i * D] = S[i];
  // The slice that drew the last ticket knows that every slice of the head has read the q / k window: it rolls the
  // window and leaves the counter at zero for the next call.
  if (tid == 0) {
    const int last = ticket == (int)gridDim.z - 1;
    if (last) tickets[(size_t)b * H + head] = 0;
    sh_last = last;
  }
  __syncthreads();
  if (sh_last) {
    *reinterpret_cast<uint2*>(cs + (size_t)cq * 4) = conv4_rolled(sq4, xq);
    *reinterpret_cast<uint2*>(cs + (size_t)ck * 4) = conv4_rolled(sk4, xk);
    if (conv_out) {
      conv_out[(size_t)b * dim + cq] = __float2bfloat16_rn(q);
      conv_out[(size_t)b * dim + ck] = __float2bfloat16_rn(k);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The whole KDA layer of a decoded token in ONE launch: cast of the projected q|k|v row, gate preparation, short
// convolution, recurrence, gated RMS norm.  The reference's decode runs kda_transpose_cast, kda_gate,
// cuda_causal_conv1d_update, cuda_recurrent_gated_delta_rule and gated_rms_norm here (src/engine/runner.cpp:433-489);
// at 2-3 us per launch, over 34 layers, the launches are most of a decode step.  Same grid and arithmetic as
// kda_decode_conv_kernel with, in front, x = bf16(x32) and g = gate_value(f), beta = bf16(sigmoid(b)) computed in
// place, and behind it the norm of the head's 128 outputs, done by whichever value slice of the head is the LAST to
// have written its outputs (second ticket counter; it reads the other slices' bf16 outputs from L2).  Every value is
// formed by the same operations as in the separate kernels: results are bit-identical to the five-call sequence.
// ---------------------------------------------------------------------------------------------
template <int NV>
__global__ __launch_bounds__(128) void kda_decode_layer_kernel(
    const float* __restrict__ x32, __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ conv_w,
    const __nv_bfloat16* __restrict__ conv_bias, const float* __restrict__ f, const float* __restrict__ bgate,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, float lower_bound, float* __restrict__ state,
    __nv_bfloat16* out, float* __restrict__ out_f32, const void* __restrict__ norm_w, int w_bf16,
    const void* __restrict__ gate_out, int g_bf16, void* __restrict__ y, int y_f16, float eps, float cbias, int gate_act, int H,
    float scale, const int* __restrict__ slots, int* __restrict__ tickets) {
  constexpr int D = 128;
  constexpr int KG = 128 / NV, RPT = D / KG;
  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * NV;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j = tid % NV, kg = tid / NV;
  const int dim = 3 * H * D;
  const int slot = slots ? slots[b] : b;
  const size_t bh = (size_t)b * H + head;
  float* my_state = state + ((size_t)slot * H + head) * D * D + (size_t)(kg * RPT) * D + v0 + j;
  __shared__ float sh_q[D], sh_k[D], sh_d[D];
  __shared__ float sh_red[2][4];
  __shared__ float sh_part[2][KG][NV];
  __shared__ int sh_last, sh_last2;

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; i++) S[i] = my_state[(size_t)i * D];

  const float* xb = x32 + (size_t)b * dim;
  __nv_bfloat16* cs = conv_state + (size_t)slot * dim * 4;
  const int cq = head * D + tid, ck = (H + head) * D + tid, cv = (2 * H + head) * D + v0 + j;
  const __nv_bfloat16 xq = __float2bfloat16(xb[cq]), xk = __float2bfloat16(xb[ck]), xv = __float2bfloat16(xb[cv]);
  const uint2 sq4 = *reinterpret_cast<const uint2*>(cs + (size_t)cq * 4), wq4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)cq * 4));
  const uint2 sk4 = *reinterpret_cast<const uint2*>(cs + (size_t)ck * 4), wk4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)ck * 4));
  const uint2 sv4 = *reinterpret_cast<const uint2*>(cs + (size_t)cv * 4), wv4 = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)cv * 4));
  const float q = conv4_silu_bf16(sq4, wq4, conv_bias ? __bfloat162float(conv_bias[cq]) : 0.f, __bfloat162float(xq));
  const float k = conv4_silu_bf16(sk4, wk4, conv_bias ? __bfloat162float(conv_bias[ck]) : 0.f, __bfloat162float(xk));
  const float v = conv4_silu_bf16(sv4, wv4, conv_bias ? __bfloat162float(conv_bias[cv]) : 0.f, __bfloat162float(xv));
  const float gv = gate_value(f[bh * D + tid], __ldg(dt_bias + head * D + tid), __expf(__ldg(a_log + head)), lower_bound);
  const float beta_h = __bfloat162float(__float2bfloat16(1.0f / (1.0f + __expf(-bgate[bh]))));

  float sq = warp_sum(q * q), sk = warp_sum(k * k);
  if (lane == 0) {
    sh_red[0][warp] = sq;
    sh_red[1][warp] = sk;
  }
  __syncthreads();
  {
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      tq += sh_red[0][w];
      tk += sh_red[1][w];
    }
    sh_q[tid] = q * rsqrtf(tq + 1e-6f);
    sh_k[tid] = k * rsqrtf(tk + 1e-6f);
    sh_d[tid] = __expf(gv);
  }
  int ticket = 0;
  if (tid == 0) ticket = atomicAdd(tickets + bh, 1);
  __syncthreads();
  if (kg == 0) *reinterpret_cast<uint2*>(cs + (size_t)cv * 4) = conv4_rolled(sv4, xv);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const int c = kg * RPT + i;
    sum = sum + sh_k[c] * sh_d[c] * S[i];
  }
  sh_part[0][kg][j] = sum;
  __syncthreads();
  float kv = 0.f;
#pragma unroll
  for (int p = 0; p < KG; p++) kv = __fadd_rn(kv, sh_part[0][p][j]);
  const float vp = v - kv;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const int c = kg * RPT + i;
    const float st = S[i] * sh_d[c] + sh_k[c] * vp * beta_h;
    S[i] = st;
    o = o + sh_q[c] * st;
  }
  sh_part[1][kg][j] = o;
  __syncthreads();
  if (kg == 0) {
    float tot = 0.f;
#pragma unroll
    for (int p = 0; p < KG; p++) tot = __fadd_rn(tot, sh_part[1][p][j]);
    tot *= scale;
    const size_t oi = bh * D + v0 + j;
    out[oi] = __float2bfloat16_rz(tot);
    if (out_f32) out_f32[oi] = tot;
    __threadfence();                       // the outputs of this slice are visible before its second ticket is drawn
  }
#pragma unroll
  for (int i = 0; i < RPT; i++) my_state[(size_t)i * D] = S[i];
  __syncthreads();
  if (tid == 0) {
    const int last = ticket == (int)gridDim.z - 1;
    if (last) tickets[bh] = 0;
    sh_last = last;
    int* t2 = tickets + (size_t)gridDim.x * H + bh;
    const int last2 = atomicAdd(t2, 1) == (int)gridDim.z - 1;
    if (last2) *t2 = 0;
    sh_last2 = last2;
  }
  __syncthreads();
  if (sh_last) {
    *reinterpret_cast<uint2*>(cs + (size_t)cq * 4) = conv4_rolled(sq4, xq);
    *reinterpret_cast<uint2*>(cs + (size_t)ck * 4) = conv4_rolled(sk4, xk);
  }
  if (sh_last2 && warp == 0) {
    // gated RMS norm of the head's 128 outputs: lane = four channels, as the one-warp-per-row norm kernel
    __threadfence();
    const uint2 xr = __ldcg(reinterpret_cast<const uint2*>(out + bh * D) + lane);
    const float4 xa = make_float4(bf16lo(xr.x), bf16hi(xr.x), bf16lo(xr.y), bf16hi(xr.y));
    const float4 ga = g_bf16 ? load4(reinterpret_cast<const __nv_bfloat16*>(gate_out) + bh * D + 4 * lane)
                             : load4(reinterpret_cast<const float*>(gate_out) + bh * D + 4 * lane);
    const float4 w4 = w_bf16 ? load4(reinterpret_cast<const __nv_bfloat16*>(norm_w) + 4 * lane)
                             : load4(reinterpret_cast<const float*>(norm_w) + 4 * lane);
    float s = warp_sum(sum_squares(0.f, xa));
    const float rmf = rsqrtf(s / (float)D + eps);
    const float4 r = finish4(xa, w4, ga, rmf, cbias, false, gate_act);
    if (y_f16) store4(reinterpret_cast<__half*>(y) + bh * D + 4 * lane, r);
    else store4(reinterpret_cast<float*>(y) + bh * D + 4 * lane, r);
  }
}

template <int NV>
static int launch_decode_conv(const __nv_bfloat16* x, __nv_bfloat16* conv_state, const __nv_bfloat16* w, const __nv_bfloat16* bias,
                              const float* g, const __nv_bfloat16* beta, float* state, __nv_bfloat16* out, float* out_f32,
                              __nv_bfloat16* conv_out, int bsz, int H, const int* slots, int* tickets, cudaStream_t s) {
  kda_decode_conv_kernel<NV><<<dim3(bsz, H, 128 / NV), 128, 0, s>>>(x, conv_state, w, bias, g, beta, state, out, out_f32, conv_out,
                                                                    H, 1.0f / sqrtf(128.0f), slots, tickets);
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

template <int D, int NV>
static int launch_recurrent(const __nv_bfloat16* qkv, const float* g, const __nv_bfloat16* beta,
                            float* state, __nv_bfloat16* out, float* out_f32, int bsz, int seqlen,
                            int Hk, int Hv, int history_stride, const int* slots, bool cw,
                            bool hist, cudaStream_t s) {
  dim3 grid(bsz, Hv, D / NV);
  const float scale = 1.0f / sqrtf((float)D);
#define HK_RL(CWV, HV)                                                                             \
  kda_recurrent_kernel<D, NV, CWV, HV><<<grid, 128, 0, s>>>(qkv, g, beta, state, out, out_f32,    \
                                                            seqlen, Hk, Hv, scale, slots,          \
                                                            history_stride)
  if (cw) { if (hist) HK_RL(true, true); else HK_RL(true, false); }
  else    { if (hist) HK_RL(false, true); else HK_RL(false, false); }
#undef HK_RL
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

}  // namespace hk

HK_API int hk_kda_recurrent(const void* mixed_qkv, const float* g, const void* beta, float* state,
                            void* out, float* out_f32, int bsz, int seqlen, int num_k_heads,
                            int num_v_heads, int k_head_dim, int v_head_dim, int history_stride,
                            const int* slots, int channelwise, int history, void* stream) {
  using namespace hk;
  HK_REQUIRE(mixed_qkv && g && beta && state && out);
  HK_REQUIRE(bsz > 0 && seqlen > 0 && num_k_heads > 0 && num_v_heads > 0 && history_stride >= 1);
  HK_REQUIRE(num_v_heads % num_k_heads == 0);
  if (history) HK_REQUIRE(history_stride >= seqlen);  // slots 1..seqlen-1 are written
  if (k_head_dim != v_head_dim) return HK_ERR_UNSUPPORTED;
  if (channelwise && k_head_dim != 128) return HK_ERR_INVALID;  // as the reference launcher
  auto q = (const __nv_bfloat16*)mixed_qkv;
  auto bt = (const __nv_bfloat16*)beta;
  auto o = (__nv_bfloat16*)out;
  cudaStream_t s = as_stream(stream);
  // narrower column slices when the (batch x head) count alone cannot cover the SMs
  const bool narrow = (long)bsz * num_v_heads * 4 < sm_count();
  if (k_head_dim == 128) {
    return narrow ? launch_recurrent<128, 16>(q, g, bt, state, o, out_f32, bsz, seqlen, num_k_heads,
                                              num_v_heads, history_stride, slots, channelwise,
                                              history, s)
                  : launch_recurrent<128, 32>(q, g, bt, state, o, out_f32, bsz, seqlen, num_k_heads,
                                              num_v_heads, history_stride, slots, channelwise,
                                              history, s);
  }
  if (k_head_dim == 64)
    return launch_recurrent<64, 32>(q, g, bt, state, o, out_f32, bsz, seqlen, num_k_heads,
                                    num_v_heads, history_stride, slots, channelwise, history, s);
  return HK_ERR_UNSUPPORTED;
}

HK_API int hk_kda_decode_step(const void* x, void* conv_state, const void* conv_weight, const void* conv_bias, const float* g,
                              const void* beta, float* rec_state, void* out, float* out_f32, void* conv_out, int bsz,
                              int num_heads, const int* slots, int* tickets, void* stream) {
  using namespace hk;
  HK_REQUIRE(x && conv_state && conv_weight && g && beta && rec_state && out && tickets);
  HK_REQUIRE(bsz > 0 && bsz <= 65535 && num_heads > 0 && num_heads <= 65535);
  auto xb = (const __nv_bfloat16*)x;
  auto cs = (__nv_bfloat16*)conv_state;
  auto cw = (const __nv_bfloat16*)conv_weight;
  auto cb = (const __nv_bfloat16*)conv_bias;
  auto bt = (const __nv_bfloat16*)beta;
  auto o = (__nv_bfloat16*)out;
  auto co = (__nv_bfloat16*)conv_out;
  cudaStream_t s = as_stream(stream);
  const bool narrow = (long)bsz * num_heads * 4 < sm_count();
  return narrow ? launch_decode_conv<16>(xb, cs, cw, cb, g, bt, rec_state, o, out_f32, co, bsz, num_heads, slots, tickets, s)
                : launch_decode_conv<32>(xb, cs, cw, cb, g, bt, rec_state, o, out_f32, co, bsz, num_heads, slots, tickets, s);
}

HK_API int hk_kda_decode_layer(const float* x32, void* conv_state, const void* conv_weight, const void* conv_bias, const float* f,
                               const float* b, const float* dt_bias, const float* a_log, float lower_bound, float* rec_state,
                               void* out, float* out_f32, const void* norm_w, int w_type, const void* gate_out, int g_type, void* y,
                               int y_type, float epsilon, float constant_bias, int gate_act, int bsz, int num_heads,
                               const int* slots, int* tickets, void* stream) {
  using namespace hk;
  HK_REQUIRE(x32 && conv_state && conv_weight && f && b && dt_bias && a_log && rec_state && out && norm_w && gate_out && y && tickets);
  HK_REQUIRE(bsz > 0 && bsz <= 65535 && num_heads > 0 && num_heads <= 65535);
  HK_REQUIRE(w_type == HK_F32 || w_type == HK_BF16);
  HK_REQUIRE(y_type == HK_F32 || y_type == HK_F16);
  HK_REQUIRE(g_type == HK_F32 || g_type == HK_BF16);
  HK_REQUIRE(gate_act == 0 || gate_act == 1);
  HK_REQUIRE(aligned(out, 8) && aligned(norm_w, w_type == HK_F32 ? 16 : 8) && aligned(y, y_type == HK_F32 ? 16 : 8) &&
             aligned(gate_out, g_type == HK_F32 ? 16 : 8));
  cudaStream_t s = as_stream(stream);
  const float scale = 1.0f / sqrtf(128.0f);
  const bool narrow = (long)bsz * num_heads * 4 < sm_count();
#define HK_DL(NV)                                                                                                          \
  kda_decode_layer_kernel<NV><<<dim3(bsz, num_heads, 128 / NV), 128, 0, s>>>(                                              \
      x32, (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)conv_weight, (const __nv_bfloat16*)conv_bias, f, b, dt_bias, a_log,  \
      lower_bound, rec_state, (__nv_bfloat16*)out, out_f32, norm_w, w_type == HK_BF16, gate_out, g_type == HK_BF16, y,        \
      y_type == HK_F16, epsilon, constant_bias, gate_act, num_heads, scale, slots, tickets)
  if (narrow) HK_DL(16); else HK_DL(32);
#undef HK_DL
  HK_LAUNCH_CHECK();
  return HK_OK;
}
