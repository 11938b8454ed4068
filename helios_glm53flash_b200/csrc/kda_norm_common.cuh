// Element helpers of the gated RMS norm  y = x * w * rsqrt(mean(x^2) + eps) * act(gate), shared by the stand-alone norm
// kernels and by the decode-step kernel that applies the norm to its own output.  Operation order as in
// helios::aux::gated_rms_norm (reference: src/cuda/aux/norm.cu:294-468).
#pragma once
#include "hk_common.cuh"

namespace hk {

// decay gate of one channel: lower_bound * sigmoid(exp(a_log[h]) * (f + dt_bias))  (glue::kda_gate, reference:
// src/engine/glue2.cu:340-368)
__device__ __forceinline__ float gate_value(float f, float bias, float decay, float lb) {
  return lb * (1.0f / (1.0f + __expf(-(decay * (f + bias)))));
}

__device__ __forceinline__ float act_gate(float v, int gate_act) {
  const float r = __fdividef(1.0f, 1.0f + __expf(-v));
  return gate_act == 1 ? r : v * r;                       // 1: sigmoid, 0: SiLU
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
}
__device__ __forceinline__ float4 load4_stream(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float4 load4_stream(const __nv_bfloat16* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
}
// raw (unconverted) 4-element pieces: fewer live registers while several rows are in flight
__device__ __forceinline__ float4 raw4(const float* p) { return load4_stream(p); }
__device__ __forceinline__ uint2 raw4(const __nv_bfloat16* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
__device__ __forceinline__ float4 cvt4(float4 v) { return v; }
__device__ __forceinline__ float4 cvt4(uint2 r) { return make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y)); }
__device__ __forceinline__ void zero_raw(float4& v) { v = make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void zero_raw(uint2& v) { v = make_uint2(0u, 0u); }

__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__half* p, float4 v) {
  const __half2 a = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y));
  const __half2 b = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&a);
  r.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

__device__ __forceinline__ float4 finish4(float4 x4, float4 w4, float4 g4, float rmf, float cbias,
                                          bool gate_first, int gate_act) {
  if (cbias != 0.0f) {
    w4.x += cbias;
    w4.y += cbias;
    w4.z += cbias;
    w4.w += cbias;
  }
  if (gate_first) {
    x4.x *= act_gate(g4.x, gate_act);
    x4.y *= act_gate(g4.y, gate_act);
    x4.z *= act_gate(g4.z, gate_act);
    x4.w *= act_gate(g4.w, gate_act);
  }
  x4.x = x4.x * w4.x * rmf;
  x4.y = x4.y * w4.y * rmf;
  x4.z = x4.z * w4.z * rmf;
  x4.w = x4.w * w4.w * rmf;
  if (!gate_first) {
    x4.x *= act_gate(g4.x, gate_act);
    x4.y *= act_gate(g4.y, gate_act);
    x4.z *= act_gate(g4.z, gate_act);
    x4.w *= act_gate(g4.w, gate_act);
  }
  return x4;
}

__device__ __forceinline__ float sum_squares(float s, float4 v) {
  s = fmaf(v.x, v.x, s);
  s = fmaf(v.y, v.y, s);
  s = fmaf(v.z, v.z, s);
  s = fmaf(v.w, v.w, s);
  return s;
}

}  // namespace hk
