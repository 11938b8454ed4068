// Self test of the tcgen05 / TMEM helper layer (tc05.cuh): one CTA computes D = A * B with fp16
// operands staged in the no-swizzle canonical layouts (or, per operand, the 128-byte-swizzle layouts
// a TMA tensor copy with 128-byte rows produces) and dumps the raw TMEM accumulator
// (all 128 lanes x N columns), so the host can check both the arithmetic and the row <-> lane
// mapping of each instruction shape.
#include "hk_common.cuh"
#include "tc05.cuh"

namespace hk {

__global__ __launch_bounds__(128) void tc05_selftest_kernel(const __half* __restrict__ A,
                                                            const __half* __restrict__ B,
                                                            float* __restrict__ D, int M, int N,
                                                            int K, int flags, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const bool a_sw = flags & 4, b_sw = flags & 8;   // 128-byte swizzle: rows of 128 B, 16-byte chunk c of row r at c ^ (r % 8)
  // the offset-swap diagnostics exist for the no-swizzle layouts only: a swapped stride offset of a
  // swizzled tile would point past the operand region
  const bool b_mn = flags & 1, a_mn = flags & 2, swap_a = (flags & 0x100) && !a_sw, swap_b = (flags & 0x200) && !b_sw;
  const bool converged_issue = flags & 0x400;   // issue from the whole of warp 0 with one elected lane (tc::mma_f16_if)
  const int tid = threadIdx.x, warp = tc::warp_index_uniform();
  uint8_t* sA = smem;
  uint8_t* sB = smem + 128 * 128 * 2;
  const uint32_t kchunks = K / 8;
  // K direction contiguous core matrices (LBO = 128 B), M/N groups of 8 rows kchunks*128 B apart
  const uint32_t lbo_a = 128, sbo_a = kchunks * 128;
  const uint32_t lbo_b = 128, sbo_b = kchunks * 128;

  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 256);
  // zero both operand regions so rows beyond M read as zero
  for (int i = tid; i < (128 * 128 * 2 + 256 * 128 * 2) / 16; i += 128)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  // swizzled forms: K-major = [K block of 64][row][128 B], block stride rows*128; MN-major =
  // [MN block of 64][k][128 B], block stride K*128 (the leading-dimension byte offset of the descriptor)
  const uint32_t blk_a = a_mn ? K * 128 : 128 * 128, blk_b = b_mn ? K * 128 : 256 * 128;
  if (a_sw) {
    const int inner = a_mn ? M / 8 : (int)kchunks, outer = a_mn ? K : M;   // outer = 128-byte row index
    for (int i = tid; i < outer * inner; i += 128) {
      const int r = i / inner, c = i % inner;
      const uint4 v = *reinterpret_cast<const uint4*>(A + (size_t)r * inner * 8 + c * 8);
      *reinterpret_cast<uint4*>(sA + tc::sw128_off(r, c, blk_a)) = v;
    }
  } else if (!a_mn) {
    for (int i = tid; i < M * (int)kchunks; i += 128) {
      int r = i / kchunks, kc = i % kchunks;
      uint4 v = *reinterpret_cast<const uint4*>(A + (size_t)r * K + kc * 8);
      *reinterpret_cast<uint4*>(sA + tc::kmajor_off(r, kc, lbo_a, sbo_a)) = v;
    }
  } else {  // A given as [K][M]
    const int mchunks = M / 8;
    for (int i = tid; i < K * mchunks; i += 128) {
      int k = i / mchunks, mc = i % mchunks;
      uint4 v = *reinterpret_cast<const uint4*>(A + (size_t)k * M + mc * 8);
      *reinterpret_cast<uint4*>(sA + tc::mnmajor_off(k, mc, lbo_a, sbo_a)) = v;
    }
  }
  if (b_sw) {
    const int inner = b_mn ? N / 8 : (int)kchunks, outer = b_mn ? K : N;
    for (int i = tid; i < outer * inner; i += 128) {
      const int r = i / inner, c = i % inner;
      const uint4 v = *reinterpret_cast<const uint4*>(B + (size_t)r * inner * 8 + c * 8);
      *reinterpret_cast<uint4*>(sB + tc::sw128_off(r, c, blk_b)) = v;
    }
  } else if (!b_mn) {
    for (int i = tid; i < N * (int)kchunks; i += 128) {
      int r = i / kchunks, kc = i % kchunks;
      uint4 v = *reinterpret_cast<const uint4*>(B + (size_t)r * K + kc * 8);
      *reinterpret_cast<uint4*>(sB + tc::kmajor_off(r, kc, lbo_b, sbo_b)) = v;
    }
  } else {
    const int nchunks = N / 8;
    for (int i = tid; i < K * nchunks; i += 128) {
      int k = i / nchunks, nc = i % nchunks;
      uint4 v = *reinterpret_cast<const uint4*>(B + (size_t)k * N + nc * 8);
      *reinterpret_cast<uint4*>(sB + tc::mnmajor_off(k, nc, lbo_b, sbo_b)) = v;
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (warp == 0) {
    // both issue forms run the same loop: every lane of warp 0 computes the (warp-uniform) descriptors; either
    // lane 0 alone issues from a diverged branch, or an elected lane issues from the converged warp
    const uint32_t leader = converged_issue ? tc::elect_one() : (uint32_t)(tid == 0);
    const uint32_t idesc = tc::make_idesc(M, N, tc::FMT_F16, tc::FMT_F16, a_mn, b_mn);
    for (int kk = 0; kk < K / 16; kk++) {
      uint64_t ad = swap_a ? tc::make_sdesc(tc::smem_u32(sA) + kk * 2 * lbo_a, sbo_a, lbo_a)
                           : tc::make_sdesc(tc::smem_u32(sA) + kk * 2 * lbo_a, lbo_a, sbo_a);
      uint64_t bd = swap_b ? tc::make_sdesc(tc::smem_u32(sB) + kk * 2 * lbo_b, sbo_b, lbo_b)
                           : tc::make_sdesc(tc::smem_u32(sB) + kk * 2 * lbo_b, lbo_b, sbo_b);
      // swizzled: K-major steps 32 B inside the 128-byte row and one block per 64 K; MN-major steps
      // two 8-row atoms (2 KB) per 16 K.  Leading offset = block stride, stride offset = 1 KB atom.
      if (a_sw) {
        const uint32_t st = tc::smem_u32(sA) + (a_mn ? kk * 2048 : (kk >> 2) * blk_a + (kk & 3) * 32);
        ad = swap_a ? tc::make_sdesc_sw128(st, 1024, blk_a) : tc::make_sdesc_sw128(st, blk_a, 1024);
      }
      if (b_sw) {
        const uint32_t st = tc::smem_u32(sB) + (b_mn ? kk * 2048 : (kk >> 2) * blk_b + (kk & 3) * 32);
        bd = swap_b ? tc::make_sdesc_sw128(st, 1024, blk_b) : tc::make_sdesc_sw128(st, blk_b, 1024);
      }
      if (converged_issue) tc::mma_f16_if(leader, tmem, ad, bd, idesc, kk > 0);
      else if (leader) tc::mma_f16(tmem, ad, bd, idesc, kk > 0);
    }
    if (converged_issue) tc::mma_commit_if(leader, &bar);
    else if (leader) tc::mma_commit(&bar);
    __syncwarp();
  }
  const bool ok = tc::mbar_wait(&bar, 0, &abort_flag, 1);
  tc::fence_after_sync();
  if (ok) {
    for (int c0 = 0; c0 < N; c0 += 16) {
      uint32_t r[16];
      tc::tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
      tc::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; j++) D[(size_t)tid * N + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 256);
  if (tid == 0) status[0] = abort_flag;
}


#ifdef HK_DIAG   // measurement aid of the diagnostic build only (not part of the product ABI)
// Issue-rate probe: `count` products (K = 16 each, operands cycling through a zeroed K = 128 tile, all
// accumulated into one TMEM tile) are issued back to back, then committed and waited for.  cycles[0] = clock64
// ticks until the last product was issued, cycles[1] = until all had completed.  converged = 0: issued by one
// thread inside a diverged branch; 1: by the whole of warp 0 with an elected lane (tc::mma_f16_if).
__global__ __launch_bounds__(128) void tc05_issue_probe_kernel(int M, int N, int converged, int count,
                                                               long long* __restrict__ cycles, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tc::warp_index_uniform();
  for (int i = tid; i < (128 * 128 * 2 + 256 * 128 * 2) / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 256);
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (warp == 0) {
    const uint32_t idesc = tc::make_idesc(M, N, tc::FMT_F16, tc::FMT_F16, false, false);
    const uint64_t ad0 = tc::make_sdesc(tc::smem_u32(smem), 128, 2048);
    const uint64_t bd0 = tc::make_sdesc(tc::smem_u32(smem + 128 * 128 * 2), 128, 2048);
    long long t0 = 0, t1 = 0;
    if (converged) {
      const uint32_t leader = tc::elect_one();
      t0 = clock64();
#pragma unroll 1
      for (int it = 0; it < count / 8; it++) {
#pragma unroll
        for (int kk = 0; kk < 8; kk++)
          tc::mma_f16_if(leader, tmem, tc::sdesc_advance(ad0, kk * 256), tc::sdesc_advance(bd0, kk * 256), idesc, true);
      }
      t1 = clock64();
      tc::mma_commit_if(leader, &bar);
    } else if (tid == 0) {
      t0 = clock64();
#pragma unroll 1
      for (int it = 0; it < count / 8; it++) {
#pragma unroll
        for (int kk = 0; kk < 8; kk++)
          tc::mma_f16(tmem, tc::sdesc_advance(ad0, kk * 256), tc::sdesc_advance(bd0, kk * 256), idesc, true);
      }
      t1 = clock64();
      tc::mma_commit(&bar);
    }
    __syncwarp();
    const bool ok = tc::mbar_wait(&bar, 0, &abort_flag, 1);       // every lane waits
    const long long t2 = clock64();
    if (tid == 0) {
      cycles[0] = t1 - t0;
      cycles[1] = t2 - t0;
      status[0] = ok ? 0 : abort_flag;
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 256);
}

#endif  // HK_DIAG

}  // namespace hk

HK_API int hk_tc05_selftest(const void* a_f16, const void* b_f16, float* d, int M, int N, int K,
                            int b_layout, int* status, void* stream) {
  using namespace hk;
  HK_REQUIRE(a_f16 && b_f16 && d && status);
  HK_REQUIRE((M == 64 || M == 128) && N >= 16 && N <= 256 && N % 16 == 0 && K >= 16 && K <= 128 &&
             K % 16 == 0);
  const size_t smem = 128 * 128 * 2 + 256 * 128 * 2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(tc05_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  tc05_selftest_kernel<<<1, 128, smem, as_stream(stream)>>>((const __half*)a_f16,
                                                            (const __half*)b_f16, d, M, N, K,
                                                            b_layout, status);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

#ifdef HK_DIAG
extern "C" __attribute__((visibility("default"))) int hk_debug_tc05_issue_probe(int M, int N, int converged, int count, long long* cycles, int* status, void* stream) {
  using namespace hk;
  HK_REQUIRE(cycles && status);
  HK_REQUIRE((M == 64 || M == 128) && N >= 16 && N <= 256 && N % 16 == 0 && count >= 8 && count <= 65536 && count % 8 == 0);
  const size_t smem = 128 * 128 * 2 + 256 * 128 * 2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(tc05_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  tc05_issue_probe_kernel<<<1, 128, smem, as_stream(stream)>>>(M, N, converged, count, cycles, status);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
#endif  // HK_DIAG
