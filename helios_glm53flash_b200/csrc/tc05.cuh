// Blackwell (sm_100a) tensor-core plumbing used by the dense kernels of this library: tcgen05.mma
// with shared-memory operands and TMEM accumulators, TMEM allocation and loads, mbarriers with
// BOUNDED waits, and bulk (TMA engine) global->shared copies.  Inline PTX only.
//
// Operand layouts.  All operands use the no-swizzle ("interleaved") canonical layouts, built from
// 8 x 16-byte core matrices, because the kernels here fill shared memory themselves (gathered rows,
// register-computed operands) or copy pre-arranged tiles with one bulk copy:
//   K-major  (row r of M/N, element k of K):   off = (r/8)*SBO + (k/8)*LBO + (r%8)*16 + (k%8)*2
//   MN-major (element n of M/N, row k of K):   off = (n/8)*SBO + (k/8)*LBO + (k%8)*16 + (n%8)*2
// i.e. in both cases SBO strides the M/N direction and LBO strides the K direction, both in bytes,
// multiples of 16.  One tcgen05.mma.kind::f16 consumes K = 16 elements = two core matrices along K.
#pragma once
#include <cstdint>

namespace hk {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------------------------------
// mbarrier (shared::cta), bounded waits
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// raises the byte count the barrier's current phase waits for, without arriving
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking phase test.  mbarrier.try_wait may SUSPEND the thread for a system-dependent time (measured
// here: well over a thousand cycles) before it reports "not yet", so it is the wrong instruction for
// "is it ready? otherwise do something else first"; test_wait returns at once.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Cycle budget of one wait (~1 s at 2 GHz).  A wait that expires records `code` in *abort_flag
// (shared memory, CTA-wide); once the flag is set every later wait returns at once, so a kernel
// with a broken dependency still terminates within about one budget and reports where it gave up.
constexpr long long MBAR_WAIT_CYCLES = 2000000000LL;

// SLEEP_NS > 0 backs the poll off with nanosleep: for long waits of warps that share an SM with
// copy-issuing warps (every poll is a shared-memory pipeline operation).
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (*abort_flag) return false;
    if (mbar_try_wait(bar, parity)) return true;
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    if (clock64() - t0 > MBAR_WAIT_CYCLES) {
      *abort_flag = code;
      return false;
    }
  }
}

// ------------------------------------------------------------------------------------------
// bulk copy global -> shared through the TMA engine (untiled form: both addresses 16-byte
// aligned, size a multiple of 16), completion counted on an mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// bulk copy shared -> global through the TMA engine (both addresses 16-byte aligned, size a multiple of 16), tracked
// by the issuing thread's bulk groups: commit, then wait until the engine has finished READING shared memory (the
// source may be rewritten) - the global writes complete asynchronously and are flushed at kernel end
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Ask the TMA engine to pull a contiguous global range into L2 (no destination, no completion to wait
// for): address 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void prefetch_l2(const void* gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem), "r"(bytes) : "memory");
}

// 16-byte asynchronous copy global -> shared that bypasses L1 (cp.async.cg).  The .ca form allocates
// an L1 line per request; in kernels that give almost all of the SM's 256 KB to shared memory the few
// KB left for L1 cap the bytes in flight and with them the copy rate.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma operand reads)
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// TMEM
// ------------------------------------------------------------------------------------------
// Whole-warp calls.  ncols: power of two, 32..512.  The address lands in *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
// `taddr` = tmem base | (first lane << 16) | first column; the lane must be the warp's own quarter
// (32 * (warp index % 4)).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 64 consecutive 32-bit columns spread over the WHOLE warp (shape 16x256b, 8 repeats): the
// natural read-back of an M = 64 accumulator, whose rows occupy lanes 0-15 of each lane quarter.
// Thread t holds rows t/4 and t/4 + 8; in repeat j (columns 8j .. 8j+7) it holds columns
// 8j + 2(t%4) and 8j + 2(t%4) + 1:  r[4j] = (row t/4, col), r[4j+1] = (row t/4, col+1),
// r[4j+2] = (row t/4+8, col), r[4j+3] = (row t/4+8, col+1).
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// the same shape with 4 and 2 repeats (32 and 16 columns); r points at 16 / 8 registers
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}

// ------------------------------------------------------------------------------------------
// descriptors
// ------------------------------------------------------------------------------------------
enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1 };

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
//   bits [4,6) D format (1 = f32) | [7,10) A format | [10,13) B format | 15 A MN-major |
//   16 B MN-major | [17,23) N >> 3 | [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(uint32_t M, uint32_t N, uint32_t a_fmt,
                                                  uint32_t b_fmt, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Shared-memory matrix descriptor, no swizzle: start address, LBO (K direction) and SBO (M/N
// direction) in 16-byte units, descriptor version 1 (Blackwell) in bits [46,48).
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes,
                                               uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// 128-byte-swizzle descriptor (layout type 2 in bits [61,64)): rows of 128 bytes, atoms of 8 rows
// (1 KB, the stride offset); the tile base must be 1 KB aligned.  K-major operands ignore the leading
// offset; MN-major operands use it as the distance between blocks of 64 M/N elements.
__device__ __forceinline__ uint64_t make_sdesc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return make_sdesc(smem_addr, lbo_bytes, sbo_bytes) | ((uint64_t)2 << 61);
}

// byte offset of 16-byte chunk `c` of 128-byte row `r` in a 128-byte-swizzled tile whose blocks of
// 8 chunks (64 elements of the contiguous dimension) are `block_bytes` apart
__device__ __forceinline__ uint32_t sw128_off(int r, int c, uint32_t block_bytes) {
  return (uint32_t)(c >> 3) * block_bytes + (uint32_t)r * 128 + (uint32_t)(((c & 7) ^ (r & 7)) << 4);
}

// descriptor of the same tile advanced by `bytes` (start-address field only; no carry into LBO for
// the offsets used here: shared addresses stay below 256 KB = 14 bits of 16-byte units)
__device__ __forceinline__ uint64_t sdesc_advance(uint64_t desc, uint32_t bytes) {
  return desc + (uint64_t)(bytes >> 4);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// ---- issue from a CONVERGED warp ----
// A tcgen05.mma takes its descriptors from uniform registers.  Inside `if (threadIdx.x == 0)` the compiler
// cannot treat them as warp-uniform and moves every operand across for every instruction: the issuing
// thread then spends about 47 cycles per MMA whatever its shape (measured: M64 N16 ... M128 N64 all 47
// cycles per instruction, the tensor pipe idle in between).  Issued by a whole warp whose index is provably
// uniform (warp_index_uniform) with one elected lane as the predicate, the same instructions go out every
// 24 (M64 N16), 29 (M64 N48), 41 (M128 N32), 49 (M128 N64, M64 N96) cycles; shapes with N >= 128 are bound
// by the tensor pipe either way (N / 2 cycles for M = 64 and M = 128 alike).
__device__ __forceinline__ int warp_index_uniform() {
  return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
}
// nonzero in exactly one lane of a fully active warp
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred;
}
// executed by every lane of the warp; only the lane with leader != 0 issues
__device__ __forceinline__ void mma_f16_if(uint32_t leader, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void mma_commit_if(uint32_t leader, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)),
      "r"(leader)
      : "memory");
}

// Arrive on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// byte offset of a 16-byte chunk inside a no-swizzle operand tile
__device__ __forceinline__ uint32_t kmajor_off(uint32_t row, uint32_t kchunk, uint32_t lbo,
                                               uint32_t sbo) {
  return (row >> 3) * sbo + kchunk * lbo + (row & 7) * 16;
}
__device__ __forceinline__ uint32_t mnmajor_off(uint32_t k, uint32_t nchunk, uint32_t lbo,
                                                uint32_t sbo) {
  return nchunk * sbo + (k >> 3) * lbo + (k & 7) * 16;
}

}  // namespace tc
}  // namespace hk
