// Shared host/device helpers of libhelios_b200 (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/helios_b200.h"

#if defined(__CUDA_ARCH__) && !defined(__CUDA_ARCH_FEAT_SM100_ALL)
#error "libhelios_b200 is written for sm_100a only (compile with -gencode arch=compute_100a,code=sm_100a)"
#endif

#define HK_API extern "C" __attribute__((visibility("default")))

#define HK_REQUIRE(cond)                    \
  do {                                      \
    if (!(cond)) return HK_ERR_INVALID;     \
  } while (0)

#define HK_LAUNCH_CHECK()                                        \
  do {                                                           \
    if (cudaPeekAtLastError() != cudaSuccess) return HK_ERR_CUDA; \
  } while (0)

namespace hk {

constexpr int LATENT = 512;     // MLA latent width (ckv row, absorbed query row)
constexpr int IDX_DIM = 128;    // indexer head dim
constexpr int POOL = 4;         // tokens per pooled indexer key

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// device word (per device) where kernels record that a bounded wait gave up; see hk_read_device_status
int* device_status_ptr();

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float bf16_bits_to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// 16-byte read-only load that does not allocate in L1 (streaming data touched once)
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace hk
