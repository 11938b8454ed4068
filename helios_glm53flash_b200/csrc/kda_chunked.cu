// Chunked KDA prefill (gated delta rule with channelwise decay), chunk = 64 tokens, dk = dv = 128.
// The reference has no chunked kernel: its prefill runs the per-token recurrence with seqlen = n
// (src/engine/runner.cpp:468-471 -> src/cuda/aux/gdn.cu:555-749).  This file computes the same
// function in two kernels.
//
// Math, per head, for a chunk with incoming state S0 [128 k][128 v] (q^, k^ = L2-normalised rows,
// G_t = inclusive cumulative log-decay inside the chunk, all exponentials below have arguments <= 0
// except inside one 16-token sub-block):
//   A_ts = sum_c k^_t k^_s e^{G_t-G_s} (s<t),  B_ts = sum_c q^_t k^_s e^{G_t-G_s} (s<=t)
//   T = (I + A diag(beta))^-1                      K+ = k^ e^{G_t},  Q+ = q^ e^{G_t}
//   W = T K+,  Uloc = T V                           Kt = beta_t k^_t e^{G_last-G_t}
//   U = Uloc - W S0                                 (delta-rule residuals of the whole chunk)
//   O = scale (Q+ S0 + (B diag(beta)) U)            S' = diag(e^{G_last}) S0 + Kt^T U
//
// Kernel 1 (kda_chunk_prep_kernel) is parallel over every (batch, head, chunk): it builds A and B
// on the warp-level tensor cores in TF32 with per-16-token re-basing of the exponents (the
// triangular 16x16 blocks are smaller than a tcgen05 tile and need fp32 exponent range), inverts the
// unit-triangular system in fp32, and runs the dense W|Uloc = T [K+|V] product as ONE
// tcgen05 M128 N256 K64 contraction.  It writes, per chunk, operand tiles that are already in the
// shared-memory layout kernel 2 needs (74,240 bytes).
// Kernel 2 (kda_chunk_scan_kernel) walks the chunks of one (batch, head, 32-column value slice) in
// order.  The fp32 state slice stays in registers; per chunk it pulls the 60 KB of operands with TMA
// bulk copies (three stages in flight) and issues three tcgen05 contractions with TMEM accumulators:
// [W;Q+] S0 (M128 N32 K128), [0;B beta] U (accumulated onto the Q+ S0 rows) and Kt^T U (M128 N32 K64).
#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime at first use)
#include <cuda_pipeline_primitives.h>

#include <cstring>

#include "hk_common.cuh"
#include "tc05.cuh"

namespace hk {

constexpr int KC = 64;                    // chunk length
constexpr int KD = 128;                   // head dim (k and v)
constexpr int KNV = 32;                   // value columns per scan CTA
constexpr int KVS = KD / KNV;             // value slices

// ---- per-chunk workspace unit (bytes); every tile is in its final shared-memory layout ----
constexpr uint32_t U_WQ = 0;              // fp16 A operand, K-major, rows 0-63 W, 64-127 Q+ ; K = 128 channels
constexpr uint32_t U_BB = 32768;          // fp16 A operand rows (t), K = 64 (s): B_ts beta_s
constexpr uint32_t U_KT = 40960;          // fp16 A operand rows = 128 channels, K = 64 tokens: Kt^T
constexpr uint32_t U_UL = 57344;          // fp16 Uloc as [4 slices][64 tokens][32]
constexpr uint32_t U_DEC = 73728;         // f32 e^{G_last}[128]
constexpr uint32_t U_BYTES = 74240;

// K-major tile with K = 128 (16 chunks): LBO 128, SBO 2048; with K = 64 (8 chunks): LBO 128, SBO 1024
constexpr uint32_t LBO = 128;
constexpr uint32_t SBO_K128 = 2048;
constexpr uint32_t SBO_K64 = 1024;

__device__ __forceinline__ uint32_t f2tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---- flags in global memory (fused form): release / acquire at GPU scope, bounded polls ----
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_gpu(int* p, int v) {
  asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// orders this thread's generic-proxy accesses with its async-proxy accesses (bulk copies) in every state space
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded poll of a flag in global memory until it is at least `want`.  Returns false once the CTA has given up
// (this wait or an earlier one) or another CTA has raised the launch-wide abort word.
__device__ __forceinline__ bool poll_flag_ge(const int* flag, int want, volatile int* abort_flag, int* g_abort, int code) {
  if (ld_acquire_gpu(flag) >= want) return true;
  const long long t0 = clock64();
  for (;;) {
    if (*abort_flag) return false;
    if (ld_acquire_gpu(flag) >= want) return true;
    __nanosleep(64);
    if (ld_relaxed_gpu(g_abort) != 0 || clock64() - t0 > tc::MBAR_WAIT_CYCLES) {
      *abort_flag = code;
      atomicExch(g_abort, code);
      return false;
    }
  }
}

// =================================================================================================
// kernel 1: per-chunk preparation.  256 threads, 104 KB of shared memory: two CTAs per SM, so the
// serial stages of one chunk overlap with another chunk's.
// =================================================================================================
constexpr int P1_LD = 132;                               // fp32 row pitch (conflict-free fragment loads)
constexpr int P1_LDH = 136;                              // 16-bit row pitch of raw k
constexpr int P1_LDA = 68;                               // fp32 row pitch of the 64x64 matrices
constexpr uint32_t P1_KP = 0;                            // fp16 K+ = first half of the B operand [K+|V] (16 KB)
constexpr uint32_t P1_G = 16384;                         // f32 [64][132] cumulative log decay, then R  (later: V half of the B operand)
constexpr uint32_t P1_KR = P1_G + KC * P1_LD * 4;        // X = inverse, f32 [64][68]
constexpr uint32_t P1_L = P1_KR + KC * P1_LDH * 2;       // raw bf16 v rows as loaded (16 KB), then the T operand (16 KB)
constexpr uint32_t P1_A = P1_L + 2 * 16 * P1_LD * 4;     // f32 [64][68] N = A beta (strictly lower); upper blocks = scratch
constexpr uint32_t P1_P = P1_A + KC * P1_LDA * 4;     // f32 [4][128] G_last - (sum before each 16-token block)
constexpr uint32_t P1_EP = P1_P + 2048;                  // f32 [4][128] e^{sum before the block}
constexpr uint32_t P1_BETA = P1_EP + 2048;               // f32 [64]
constexpr uint32_t P1_RK = P1_BETA + 256;                // f32 [64] 1 / |k_t|
constexpr uint32_t P1_DD = P1_RK + 256;                  // f32 [6][128] decay between the starts of two blocks
constexpr uint32_t P1_TOT = P1_DD + 3072;                // f32 [4][128] log-decay total of each block
constexpr uint32_t P1_SMEM = P1_TOT + 2048;
static_assert(KC * P1_LD * 4 >= 16384 && 2 * 16 * P1_LD * 4 >= 16384 && KC * P1_LDH * 2 == KC * P1_LDA * 4, "aliases");

// Optional stage timeline (diagnostic build, -DHK_DIAG): one preparation worker and one scan CTA stamp clock64 at
// their stage boundaries; hk_debug_kda_trace copies the stamps to the host.
#ifdef HK_DIAG
__device__ long long hk_kda_trace[128];
// stamps go to shared memory and are copied out once per unit.  A stamp placed after a barrier is taken when the
// stamping warp ARRIVES there (the clock read is not held back by the barrier): the intervals are that warp's own
// work, not the stage's length - the slowest warp of a stage shows up in the NEXT interval.
__shared__ long long hk_kda_stamps[16];
#define KT_TRACE(slot) do { if (ctx.trace && ctx.tid == 0) hk_kda_stamps[slot] = clock64(); } while (0)
#define KT_FLUSH() do { if (ctx.trace && ctx.tid == 0) { for (int q_ = 0; q_ < 16; q_++) hk_kda_trace[q_] = hk_kda_stamps[q_]; } } while (0)
#define KS_TRACE(slot, ch) do { if (threadIdx.x == 0 && blockIdx.x == 1 && (ch) == 100) hk_kda_trace[32 + (slot)] = clock64(); } while (0)
#define KS_TRACE_AT(slot, ch, want) do { if (threadIdx.x == 0 && blockIdx.x == 1 && (ch) == (want)) hk_kda_trace[32 + (slot)] = clock64(); } while (0)
#else
#define KS_TRACE_AT(slot, ch, want) do { } while (0)
#define KT_TRACE(slot) do { } while (0)
#define KT_FLUSH() do { } while (0)
#define KS_TRACE(slot, ch) do { } while (0)
#endif

// 16 x 16 block product on the warp-level tensor cores: acc += L R with L, R fp32 in shared memory (row
// pitch P1_LDA).  Each operand is split into a TF32 head and a TF32 tail and the three significant
// partial products are accumulated in fp32, which keeps the result at fp32-class accuracy.
__device__ __forceinline__ void block16_mma(const float* __restrict__ L, const float* __restrict__ R,
                                            float (&acc)[2][4], int lane) {
  const int g8 = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int ks = 0; ks < 2; ks++) {
    const float af[4] = {L[g8 * P1_LDA + 8 * ks + tig], L[(g8 + 8) * P1_LDA + 8 * ks + tig],
                         L[g8 * P1_LDA + 8 * ks + tig + 4], L[(g8 + 8) * P1_LDA + 8 * ks + tig + 4]};
    uint32_t ah[4], al[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      ah[e] = f2tf32(af[e]);
      al[e] = f2tf32(af[e] - __uint_as_float(ah[e]));
    }
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
      const float b0 = R[(8 * ks + tig) * P1_LDA + 8 * nt + g8], b1 = R[(8 * ks + tig + 4) * P1_LDA + 8 * nt + g8];
      const uint32_t b0h = f2tf32(b0), b1h = f2tf32(b1);
      const uint32_t b0l = f2tf32(b0 - __uint_as_float(b0h)), b1l = f2tf32(b1 - __uint_as_float(b1h));
      mma_tf32(acc[nt], al, b0h, b1h);
      mma_tf32(acc[nt], ah, b0l, b1l);
      mma_tf32(acc[nt], ah, b0h, b1h);
    }
  }
}

// writes sign * acc (fragment rows g8, g8 + 8; columns 8 nt + 2 tig, + 1) to a 16 x 16 block
__device__ __forceinline__ void block16_store(float* __restrict__ D, const float (&acc)[2][4], float sign, int lane) {
  const int g8 = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 2; nt++) {
    *reinterpret_cast<float2*>(D + g8 * P1_LDA + 8 * nt + 2 * tig) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
    *reinterpret_cast<float2*>(D + (g8 + 8) * P1_LDA + 8 * nt + 2 * tig) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
  }
}

// Stage 4 of the preparation kernel for one warp: rows 16 ib .. 16 ib + 15 of A (k warps) or B (q warps)
// against the column blocks jb <= ib.  v = this thread's left-operand fragment values (rows g8, g8 + 8;
// channel 32 m + 8 tig + j at index 8 m + j).  k-step ks of the m16n8k8 product contracts the channel
// pairs (32 m + 8 tig + j, + 1), j = 2 (ks % 4), m = ks / 4, in MMA k slots tig and tig + 4.
__device__ __forceinline__ void prep_ab_block(const int ib, const float (&v)[2][32], bool is_q, const float* __restrict__ sR,
                                              const float* __restrict__ sDD, const float* __restrict__ sBeta,
                                              float* __restrict__ sA, uint8_t* __restrict__ unit, int g8, int tig) {
  // one code path for all row blocks (column blocks jb > ib are skipped by warp-uniform branches): four
  // specialised copies of this fully unrolled body would not fit the instruction cache
  float acc[4][2][4];
#pragma unroll
  for (int jb = 0; jb < 4; jb++)
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[jb][nt][e] = 0.f;
  const float* dd_base = sDD + (ib * (ib - 1) / 2) * KD;
  // two k-steps per pass: the R rows are read 16 bytes at a time (4 channels = both channel pairs of the
  // two k-steps), which with the 132-float row pitch is free of bank conflicts (a quarter-warp covers
  // rows g8, g8 + 1 and the four tig: 4 g8 + 8 tig are eight different 4-bank groups)
#pragma unroll
  for (int kp = 0; kp < 8; kp++) {
    const int m = kp >> 1, j = (kp & 1) * 4;
    const int c0 = 32 * m + 8 * tig + j;
    uint32_t a0[4], a1[4];
    a0[0] = f2tf32(v[0][8 * m + j]); a0[1] = f2tf32(v[1][8 * m + j]);
    a0[2] = f2tf32(v[0][8 * m + j + 1]); a0[3] = f2tf32(v[1][8 * m + j + 1]);
    a1[0] = f2tf32(v[0][8 * m + j + 2]); a1[1] = f2tf32(v[1][8 * m + j + 2]);
    a1[2] = f2tf32(v[0][8 * m + j + 3]); a1[3] = f2tf32(v[1][8 * m + j + 3]);
#pragma unroll
    for (int jb = 0; jb < 4; jb++) {
      if (jb <= ib) {
        float4 dd = make_float4(1.f, 1.f, 1.f, 1.f);
        if (jb < ib) dd = *reinterpret_cast<const float4*>(dd_base + jb * KD + c0);
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const float4 r4 = *reinterpret_cast<const float4*>(sR + (jb * 16 + nt * 8 + g8) * P1_LD + c0);
          mma_tf32(acc[jb][nt], a0, f2tf32(r4.x * dd.x), f2tf32(r4.y * dd.y));
          mma_tf32(acc[jb][nt], a1, f2tf32(r4.z * dd.z), f2tf32(r4.w * dd.w));
        }
      }
    }
  }
  // accumulator fragment: rows t = 16 ib + g8 (+8), columns s = 16 jb + 8 nt + 2 tig (+1)
#pragma unroll
  for (int jb = 0; jb < 4; jb++) {
    if (jb > ib) continue;
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
      const int s0 = jb * 16 + nt * 8 + tig * 2;
      const float b0 = sBeta[s0], b1 = sBeta[s0 + 1];
#pragma unroll
      for (int hrow = 0; hrow < 2; hrow++) {
        const int t = ib * 16 + g8 + hrow * 8;
        if (!is_q) {            // N = A beta, strictly lower
          if (s0 < t) sA[t * P1_LDA + s0] = acc[jb][nt][2 * hrow] * b0;
          if (s0 + 1 < t) sA[t * P1_LDA + s0 + 1] = acc[jb][nt][2 * hrow + 1] * b1;
        } else {                // B beta, lower including the diagonal, fp16 operand tile
          const float v0 = s0 <= t ? acc[jb][nt][2 * hrow] * b0 : 0.f;
          const float v1 = s0 + 1 <= t ? acc[jb][nt][2 * hrow + 1] * b1 : 0.f;
          *reinterpret_cast<uint32_t*>(unit + U_BB + (t >> 3) * SBO_K64 + (s0 >> 3) * LBO + (t & 7) * 16 + (s0 & 7) * 2) =
              pack_h2(v0, v1);
        }
      }
    }
  }
}

// What one preparation worker (256 threads) needs besides the tensors: its shared memory, its completion barrier
// for the tensor-core product, its 256 TMEM columns and how it synchronises.  SUB = false: the worker is a whole
// CTA (__syncthreads); SUB = true: it is one half of a 512-thread CTA and uses the named barrier `bar_id`.
struct PrepCtx {
  uint8_t* smem;
  uint64_t* bar;
  uint32_t bar_parity;
  volatile int* abort_flag;
  uint32_t tmem;
  int tid;
  int bar_id;
  bool trace;
  // fused form only: the ring slot this unit is written to must have been drained (flag >= want); thread 0 sampled
  // the flag at the start of the unit (slot_seen) and polls, with a bound, only if that was too early
  const int* slot_flag;
  int slot_want, slot_seen;
  int* g_abort;
};
template <bool SUB>
__device__ __forceinline__ void prep_sync(const PrepCtx& ctx) {
  if (SUB) asm volatile("bar.sync %0, 256;" ::"r"(ctx.bar_id) : "memory");
  else __syncthreads();
}

// One (batch, head, chunk) unit of the preparation.
// GATED: `g` holds the raw gate projection f and `beta_in` the raw fp32 b; the kernel applies
//   g = lower_bound * sigmoid(exp(a_log[head]) * (f + dt_bias[head][channel])),  beta = bf16(sigmoid(b))
// itself (the arithmetic of the reference's separate gate kernel, src/engine/glue2.cu:347-360), so the
// fp32 gate tensor is never written to or read back from memory.
// (pf_head, pf_chunk): a unit whose input rows this worker asks the copy engine to pull into L2 (pf_chunk < 0: none).
template <bool GATED, bool SUB>
__device__ __forceinline__ void prep_unit(
    const PrepCtx& ctx, const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ g,
    const void* __restrict__ beta_in, uint8_t* __restrict__ unit, int seqlen, int H, int head, int chunk, int b,
    int pf_head, int pf_chunk, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
    float lower_bound) {
  uint8_t* smem = ctx.smem;
  float* sG = reinterpret_cast<float*>(smem + P1_G);
  float* sA = reinterpret_cast<float*>(smem + P1_A);
  float* sGLP = reinterpret_cast<float*>(smem + P1_P);
  float* sTot = reinterpret_cast<float*>(smem + P1_TOT);
  float* sEP = reinterpret_cast<float*>(smem + P1_EP);
  float* sBeta = reinterpret_cast<float*>(smem + P1_BETA);
  float* sDD = reinterpret_cast<float*>(smem + P1_DD);
  float* sETot = sTot;                                     // e^{block total}: overwrites the totals once the tables are built
  float* sEGLN = sGLP;                                     // e^{G_last - (sum up to the END of the block)}
  uint8_t* sKV = smem + P1_KP;                             // [K+ | V] fp16 B operand; the V half aliases sG, valid after the A/B stage
  float* sX = reinterpret_cast<float*>(smem + P1_KR);      // alias, valid after the A/B stage
  uint8_t* sT = smem + P1_L;                               // raw v rows, then the T operand (valid after the conversion of v)

  const int tid = ctx.tid, lane = tid & 31, warp = tid >> 5;
  const int t0 = chunk * KC;
  const int n_valid = min(KC, seqlen - t0);
  const size_t row = (size_t)3 * H * KD;
  const __nv_bfloat16* tok0 = qkv + ((size_t)b * seqlen + t0) * row;
  const float* g0 = g + (((size_t)b * seqlen + t0) * H + head) * KD;

  KT_TRACE(0);
  // L2 prefetch of the input rows of a later unit (about one wave of workers ahead): its q, k, v rows (256 B each)
  // and g rows (512 B), one request per thread.  That unit's own loads then mostly hit L2.
  {
    const int pt = pf_chunk * KC + (tid & 63);
    if (pf_chunk >= 0 && pt < seqlen) {
      const __nv_bfloat16* ptok = qkv + ((size_t)b * seqlen + pt) * row;
      const int part = tid >> 6;                          // 0: q, 1: k, 2: v, 3: g
      if (part < 3) tc::prefetch_l2(ptok + (size_t)(part * H + pf_head) * KD, KD * 2);
      else tc::prefetch_l2(g + (((size_t)b * seqlen + pt) * H + pf_head) * KD, KD * 4);
    }
  }
  // ---- stage 1: loads.  Ownership for stages 1-4 is the TF32 MMA fragment layout, so that the left
  //      operands of the A/B products never pass through shared memory: warp -> (16-token row block ib,
  //      k or q), lane = 4*g8 + tig owns rows 16 ib + g8 and + 8 and, of every 32 channels, the 8
  //      starting at 8 tig (one 16-byte piece).  Block ib has ib+1 column blocks of work and the k warps
  //      carry the exponentials of stage 3: every scheduler partition gets one k warp and one q warp
  //      whose row blocks add up to the same work.
  const int g8 = lane >> 2, tig = lane & 3;
  const bool is_q = warp >> 2;                              // warps 0-3: k rows, warps 4-7: q rows
  const int ib = is_q ? 3 - (warp & 3) : (warp & 3);        // partition s hosts k block s and q block 3 - s
  float v[2][32];                                           // [row half][4 pieces x 8 channels]
  {
    uint4 raw[2][4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int t = 16 * ib + g8 + 8 * h;
      const __nv_bfloat16* src = tok0 + (size_t)t * row + (size_t)(is_q ? head : H + head) * KD + 8 * tig;
#pragma unroll
      for (int m = 0; m < 4; m++)
        raw[h][m] = t < n_valid ? *reinterpret_cast<const uint4*>(src + 32 * m) : make_uint4(0, 0, 0, 0);
    }
    // g rows straight to shared memory (warp w: tokens w, w+8, ...; lane: 4 channels)
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int t = warp + 8 * i;
      float* gdst = sG + t * P1_LD + lane * 4;
      if (t < n_valid) __pipeline_memcpy_async(gdst, g0 + (size_t)t * H * KD + lane * 4, 16);
      else *reinterpret_cast<float4*>(gdst) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __pipeline_commit();
    // v rows (raw bf16) are parked where the T operand goes later; chunk cc of row t sits at cc ^ (t % 8)
    // so that the conversion pass (8 rows of one chunk per quarter-warp) is free of bank conflicts.  (The product
    // T V needs both operands in ONE 16-bit format: a kind::f16 product of an fp16 T with the bf16 rows as they
    // were loaded is rejected by the hardware as an illegal instruction.)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int i = tid + 256 * j, t = i >> 4, cc = i & 15;
      uint8_t* vdst = sT + t * 256 + ((cc ^ (t & 7)) << 4);
      if (t < n_valid) __pipeline_memcpy_async(vdst, tok0 + (size_t)t * row + (size_t)(2 * H + head) * KD + cc * 8, 16);
      else *reinterpret_cast<uint4*>(vdst) = make_uint4(0, 0, 0, 0);
    }
    __pipeline_commit();
    if (tid < KC) {
      float bv = 0.f;
      if (tid < n_valid) {
        const size_t bi = ((size_t)b * seqlen + t0 + tid) * H + head;
        if (GATED) bv = __bfloat162float(__float2bfloat16(1.0f / (1.0f + __expf(-static_cast<const float*>(beta_in)[bi]))));
        else bv = __bfloat162float(static_cast<const __nv_bfloat16*>(beta_in)[bi]);
      }
      sBeta[tid] = bv;
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int t = 16 * ib + g8 + 8 * h;
      float ss = 0.f;
#pragma unroll
      for (int m = 0; m < 4; m++) {
        const uint32_t w4[4] = {raw[h][m].x, raw[h][m].y, raw[h][m].z, raw[h][m].w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float lo = bf16lo(w4[e]), hi = bf16hi(w4[e]);
          v[h][8 * m + 2 * e] = lo;
          v[h][8 * m + 2 * e + 1] = hi;
          ss = fmaf(lo, lo, fmaf(hi, hi, ss));
        }
      }
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float rn = rsqrtf(ss + 1e-6f);                  // L2 normalisation of the q / k row
#pragma unroll
      for (int e = 0; e < 32; e++) v[h][e] *= rn;
    }
  }
  KT_TRACE(1);
  __pipeline_wait_prior(1);                                 // g has landed; the v rows may still be in flight
  if (GATED) {
    // every thread turns the pieces it copied itself (tokens warp, warp + 8, ...; 4 channels) into gates
    const float decay = __expf(__ldg(a_log + head));
    const float4 bias = __ldg(reinterpret_cast<const float4*>(dt_bias + (size_t)head * KD) + lane);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int t = warp + 8 * i;
      if (t < n_valid) {
        float4* gp = reinterpret_cast<float4*>(sG + t * P1_LD + lane * 4);
        float4 fv = *gp;
        fv.x = lower_bound * (1.0f / (1.0f + __expf(-(decay * (fv.x + bias.x)))));
        fv.y = lower_bound * (1.0f / (1.0f + __expf(-(decay * (fv.y + bias.y)))));
        fv.z = lower_bound * (1.0f / (1.0f + __expf(-(decay * (fv.z + bias.z)))));
        fv.w = lower_bound * (1.0f / (1.0f + __expf(-(decay * (fv.w + bias.w)))));
        *gp = fv;
      }
    }
  }
  // fused form: the ring slot must have been drained before the first write to the unit (all of them follow)
  if (SUB && tid == 0 && ctx.slot_seen < ctx.slot_want)
    poll_flag_ge(ctx.slot_flag, ctx.slot_want, ctx.abort_flag, ctx.g_abort, 20);
  prep_sync<SUB>(ctx);

  KT_TRACE(2);
  {
  // blocks of B beta above the diagonal are never computed: they are zeros in the workspace tile
  if (tid < 192) {
    const int blk = tid >> 5, e = tid & 31;             // 6 blocks x (16 rows x 2 chunks)
    const int zi = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
    const int zj = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);
    const int t = zi * 16 + (e >> 1), sc = zj * 2 + (e & 1);
    *reinterpret_cast<uint4*>(unit + U_BB + (t >> 3) * SBO_K64 + sc * LBO + (t & 7) * 16) = make_uint4(0, 0, 0, 0);
  }
  }
  // ---- stage 2: log-decay sums per channel.  x_t = inclusive sum INSIDE the 16-token block (in place
  //      over g), block totals, then the per-block tables: e^{P_blk} (P = sum before the block),
  //      G_last - P_blk, the decay between two block starts, and the chunk decay e^{G_last}. ----
  {
    const int c = tid & 127, b0 = (tid >> 7) * 2;
    float a0 = 0.f, a1 = 0.f;
    float* p0 = sG + (16 * b0) * P1_LD + c;
    float* p1 = p0 + 16 * P1_LD;
#pragma unroll
    for (int t = 0; t < 16; t++) {
      a0 += p0[t * P1_LD]; p0[t * P1_LD] = a0;
      a1 += p1[t * P1_LD]; p1[t * P1_LD] = a1;
    }
    sTot[b0 * KD + c] = a0;
    sTot[(b0 + 1) * KD + c] = a1;
  }
  prep_sync<SUB>(ctx);
  // The k warps (threads 0-127, one channel each) build the per-block tables while the q warps scale their rows by
  // e^{x}, which needs x only.
  if (!is_q) {
    const float t0s = sTot[tid], t1s = sTot[KD + tid], t2s = sTot[2 * KD + tid], t3s = sTot[3 * KD + tid];
    const float P1v = t0s, P2v = P1v + t1s, P3v = P2v + t2s, GL = P3v + t3s;
    // for Kt: decay from a token to the end of ITS block is e^{tot - x} = e^{-x} e^{tot} (each factor within fp32
    // range for |x| <= 85), the decay over the LATER blocks is e^{G_last - P_next} (may underflow: then Kt is 0)
    sEGLN[tid] = __expf(GL - P1v); sEGLN[KD + tid] = __expf(GL - P2v); sEGLN[2 * KD + tid] = __expf(GL - P3v); sEGLN[3 * KD + tid] = 1.f;
    sETot[tid] = __expf(t0s); sETot[KD + tid] = __expf(t1s); sETot[2 * KD + tid] = __expf(t2s); sETot[3 * KD + tid] = __expf(t3s);
    sEP[tid] = 1.f; sEP[KD + tid] = __expf(P1v); sEP[2 * KD + tid] = __expf(P2v); sEP[3 * KD + tid] = __expf(P3v);
    // pair (ib, jb < ib) at index ib (ib - 1) / 2 + jb: e^{P_ib - P_jb}
    sDD[tid] = __expf(t0s);
    sDD[KD + tid] = __expf(t0s + t1s); sDD[2 * KD + tid] = __expf(t1s);
    sDD[3 * KD + tid] = __expf(t0s + t1s + t2s); sDD[4 * KD + tid] = __expf(t1s + t2s); sDD[5 * KD + tid] = __expf(t2s);
    reinterpret_cast<float*>(unit + U_DEC)[tid] = __expf(GL);
  }
  else {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const float* xr = sG + (16 * ib + g8 + 8 * h) * P1_LD + 8 * tig;
#pragma unroll
      for (int m = 0; m < 4; m++) {
        const float4 x0 = *reinterpret_cast<const float4*>(xr + 32 * m), x1 = *reinterpret_cast<const float4*>(xr + 32 * m + 4);
        v[h][8 * m + 0] *= __expf(fmaxf(x0.x, -85.f)); v[h][8 * m + 1] *= __expf(fmaxf(x0.y, -85.f));
        v[h][8 * m + 2] *= __expf(fmaxf(x0.z, -85.f)); v[h][8 * m + 3] *= __expf(fmaxf(x0.w, -85.f));
        v[h][8 * m + 4] *= __expf(fmaxf(x1.x, -85.f)); v[h][8 * m + 5] *= __expf(fmaxf(x1.y, -85.f));
        v[h][8 * m + 6] *= __expf(fmaxf(x1.z, -85.f)); v[h][8 * m + 7] *= __expf(fmaxf(x1.w, -85.f));
      }
    }
  }
  prep_sync<SUB>(ctx);

  KT_TRACE(3);
  KT_TRACE(4);
  // ---- stage 3: the q warps have read x; the k warps turn it into the RIGHT operand R[s][c] = k^_s e^{-x_s} (in
  //      place, fp32: up to e^85) and scale their own rows by e^{x}; the q warps emit Q+ = q^ e^{G_t} (fp16 tile
  //      rows 64..127) ----
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const int t = 16 * ib + g8 + 8 * h;
    float* xr = sG + t * P1_LD + 8 * tig;
#pragma unroll
    for (int m = 0; m < 4; m++) {
      if (!is_q) {
        float4 x0 = *reinterpret_cast<const float4*>(xr + 32 * m), x1 = *reinterpret_cast<const float4*>(xr + 32 * m + 4);
        float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w}, r8[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const float xc = fmaxf(xs[e], -85.f);
          r8[e] = v[h][8 * m + e] * __expf(-xc);
          v[h][8 * m + e] *= __expf(xc);
        }
        *reinterpret_cast<float4*>(xr + 32 * m) = make_float4(r8[0], r8[1], r8[2], r8[3]);
        *reinterpret_cast<float4*>(xr + 32 * m + 4) = make_float4(r8[4], r8[5], r8[6], r8[7]);
      } else {
        const float* ep = sEP + ib * KD + 32 * m + 8 * tig;
        const float4 e0 = *reinterpret_cast<const float4*>(ep), e1 = *reinterpret_cast<const float4*>(ep + 4);
        uint4 p;
        p.x = pack_h2(v[h][8 * m + 0] * e0.x, v[h][8 * m + 1] * e0.y); p.y = pack_h2(v[h][8 * m + 2] * e0.z, v[h][8 * m + 3] * e0.w);
        p.z = pack_h2(v[h][8 * m + 4] * e1.x, v[h][8 * m + 5] * e1.y); p.w = pack_h2(v[h][8 * m + 6] * e1.z, v[h][8 * m + 7] * e1.w);
        *reinterpret_cast<uint4*>(unit + U_WQ + ((64 + t) >> 3) * SBO_K128 + (4 * m + tig) * LBO + (t & 7) * 16) = p;
      }
    }
  }
  prep_sync<SUB>(ctx);

  KT_TRACE(5);
  // ---- stage 4: A and B on the warp-level tensor cores (TF32).  Every warp multiplies its own 16
  //      rows (fragments from registers) with the R rows of the column blocks jb <= ib; R of an earlier
  //      block is moved from its own reference P_jb to P_ib by the pair decay while it is loaded.  The
  //      contraction runs over the channels in the order the registers hold them. ----
  prep_ab_block(ib, v, is_q, sG, sDD, sBeta, sA, unit, g8, tig);
  // Kt^T tile (rows = channels, K = tokens) from R: Kt[t][c] = beta_t R[t][c] e^{tot_blk} e^{G_last - P_next}, no
  // exponentials; all eight warps, a thread = 8 tokens of one channel = one 16-byte piece of the tile
  for (int i = tid; i < KD * (KC / 8); i += 256) {
    const int c = i & 127, tg = i >> 7;
    const float et = sETot[(tg >> 1) * KD + c], en = sEGLN[(tg >> 1) * KD + c];
    float kt[8];
#pragma unroll
    for (int u8 = 0; u8 < 8; u8++) {
      const int t = tg * 8 + u8;
      kt[u8] = sBeta[t] * (sG[t * P1_LD + c] * et) * en;
    }
    uint4 p;
    p.x = pack_h2(kt[0], kt[1]); p.y = pack_h2(kt[2], kt[3]); p.z = pack_h2(kt[4], kt[5]); p.w = pack_h2(kt[6], kt[7]);
    *reinterpret_cast<uint4*>(unit + U_KT + (c >> 3) * SBO_K64 + tg * LBO + (c & 7) * 16) = p;
  }
  if (!is_q) {
    // K+ = k^ e^{G_t}: first half of the [K+ | V] operand
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int t = 16 * ib + g8 + 8 * h;
#pragma unroll
      for (int m = 0; m < 4; m++) {
        const float* ep = sEP + ib * KD + 32 * m + 8 * tig;
        const float4 e0 = *reinterpret_cast<const float4*>(ep), e1 = *reinterpret_cast<const float4*>(ep + 4);
        uint4 p;
        p.x = pack_h2(v[h][8 * m + 0] * e0.x, v[h][8 * m + 1] * e0.y); p.y = pack_h2(v[h][8 * m + 2] * e0.z, v[h][8 * m + 3] * e0.w);
        p.z = pack_h2(v[h][8 * m + 4] * e1.x, v[h][8 * m + 5] * e1.y); p.w = pack_h2(v[h][8 * m + 6] * e1.z, v[h][8 * m + 7] * e1.w);
        *reinterpret_cast<uint4*>(sKV + (4 * m + tig) * 1024 + (t >> 3) * 128 + (t & 7) * 16) = p;
      }
    }
  }
  __pipeline_wait_prior(0);                                 // v rows
  prep_sync<SUB>(ctx);
  KT_TRACE(6);

  // from here on sG is dead: the V half of sKV, sX and (after the conversion) sT take their place

  // ---- stage 5: V -> B operand columns 128..255 (bf16 -> fp16), then the blocked inverse X = (I + N)^-1 in fp32
  //      and its fp16 copy T as the A operand.  The conversion needs no barrier of its own: the inverse works on sA
  //      and sX only, and the T operand is written (5c) after the barriers of the inverse. ----
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = tid + 256 * j;
    const int t = (i & 7) + ((i >> 7) << 3), cc = (i >> 3) & 15;
    const uint4 vr = *reinterpret_cast<const uint4*>(sT + t * 256 + ((cc ^ (t & 7)) << 4));   // bf16 -> fp16
    uint4 p;
    p.x = pack_h2(bf16lo(vr.x), bf16hi(vr.x)); p.y = pack_h2(bf16lo(vr.y), bf16hi(vr.y));
    p.z = pack_h2(bf16lo(vr.z), bf16hi(vr.z)); p.w = pack_h2(bf16lo(vr.w), bf16hi(vr.w));
    *reinterpret_cast<uint4*>(sKV + (16 + cc) * 1024 + (t >> 3) * 128 + (t & 7) * 16) = p;
  }
  KT_TRACE(7);
  // 5a: the four diagonal 16x16 blocks, one warp each, lane = column: x_r = delta - sum_{s<r} N[r][s] x_s
  if (warp < 4 && lane < 16) {
    const int ib = warp;
    float x[16];
#pragma unroll
    for (int r = 0; r < 16; r++) {
      float a0 = (r == lane) ? 1.f : 0.f, a1 = 0.f;
      const float* nrow = sA + (ib * 16 + r) * P1_LDA + ib * 16;
#pragma unroll
      for (int s = 0; s < r; s++) {
        if (s & 1) a1 = fmaf(-nrow[s], x[s], a1);
        else a0 = fmaf(-nrow[s], x[s], a0);
      }
      x[r] = a0 + a1;
    }
#pragma unroll
    for (int r = 0; r < 16; r++) sX[(ib * 16 + r) * P1_LDA + ib * 16 + lane] = x[r];
  }
  prep_sync<SUB>(ctx);
  KT_TRACE(8);
  // 5b: off-diagonal blocks.  M_im = X_ii N_im for the six pairs i > m (kept in the unused mirror block
  //     (m, i) of sA), then by distance d = i - j: X_ij = - sum_{m=j}^{i-1} M_im X_mj.  One warp per
  //     16x16 block, products on the warp-level tensor cores with split operands (fp32-class accuracy).
  if (warp < 6) {
    const int i = warp < 1 ? 1 : (warp < 3 ? 2 : 3), m = warp - (i * (i - 1)) / 2;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    block16_mma(sX + (i * 16) * P1_LDA + i * 16, sA + (i * 16) * P1_LDA + m * 16, acc, lane);
    block16_store(sA + (m * 16) * P1_LDA + i * 16, acc, 1.f, lane);
  }
  prep_sync<SUB>(ctx);
#pragma unroll 1
  for (int d = 1; d < 4; d++) {
    if (warp < 4 - d) {
      const int i = d + warp, j = warp;
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int m = j; m < i; m++)
        block16_mma(sA + (m * 16) * P1_LDA + i * 16, sX + (m * 16) * P1_LDA + j * 16, acc, lane);
      block16_store(sX + (i * 16) * P1_LDA + j * 16, acc, -1.f, lane);
    }
    prep_sync<SUB>(ctx);
  }
  KT_TRACE(9);
  // 5c: T = fp16(X) as the K-major A operand (K = 64): lanes = 8 rows x 4 chunks.  Rows 64..127 of the
  //     operand are never produced: zero, so the unused TMEM lanes stay finite
  for (int i = tid; i < 8192 / 16; i += 256) reinterpret_cast<uint4*>(sT + 8192)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < KC * (KC / 8); i += 256) {
    const int t = (i & 7) + ((i >> 6) << 3), jc = (i >> 3) & 7;
    uint4 p = make_uint4(0, 0, 0, 0);                      // blocks above the diagonal are never computed: zeros
    if ((jc >> 1) <= (t >> 4)) {
      const float4 v0 = *reinterpret_cast<const float4*>(sX + t * P1_LDA + jc * 8);
      const float4 v1 = *reinterpret_cast<const float4*>(sX + t * P1_LDA + jc * 8 + 4);
      p.x = pack_h2(v0.x, v0.y); p.y = pack_h2(v0.z, v0.w); p.z = pack_h2(v1.x, v1.y); p.w = pack_h2(v1.z, v1.w);
    }
    *reinterpret_cast<uint4*>(sT + (t >> 3) * SBO_K64 + jc * LBO + (t & 7) * 16) = p;
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  prep_sync<SUB>(ctx);
  tc::fence_after_sync();

  KT_TRACE(10);
  // ---- stage 6: [W | Uloc] = T [K+ | V] : tcgen05 M128 N256 K64, fp16 in, fp32 TMEM accumulators ----
  const uint32_t tmem = ctx.tmem;
  if (tid == 0) {
    const uint32_t idesc = tc::make_idesc(128, 256, tc::FMT_F16, tc::FMT_F16, false, true);
    const uint32_t a_addr = tc::smem_u32(sT), b_addr = tc::smem_u32(sKV);
#pragma unroll
    for (int kk = 0; kk < KC / 16; kk++) {
      const uint64_t ad = tc::make_sdesc(a_addr + kk * 2 * LBO, LBO, SBO_K64);
      const uint64_t bd = tc::make_sdesc(b_addr + kk * 2 * 128, 128, 1024);
      tc::mma_f16(tmem, ad, bd, idesc, kk > 0);
    }
    tc::mma_commit(ctx.bar);
  }
  // one warp polls the barrier (with a back-off); the others park at the block barrier instead of spending
  // issue slots that the other CTA of this SM can use
  if (warp == 0) tc::mbar_wait<64>(ctx.bar, ctx.bar_parity, ctx.abort_flag, 1);
  prep_sync<SUB>(ctx);
  const bool ok = *ctx.abort_flag == 0;
  tc::fence_after_sync();
  KT_TRACE(11);
  // ---- stage 7: epilogue. Lanes 0-63 are the tokens; warps 0,1 take W, warps 4,5 take Uloc ----
  if (ok && (warp & 3) < 2) {
    const int t = (warp & 3) * 32 + lane;
    const bool second = warp >= 4;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (second ? 128 : 0);
#pragma unroll
    for (int c0 = 0; c0 < KD; c0 += 32) {
      uint32_t r[32];
      tc::tmem_ld32(lane_addr + c0, r);
      tc::tmem_ld_wait();
      uint4 p[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        p[u].x = pack_h2(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
        p[u].y = pack_h2(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
        p[u].z = pack_h2(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
        p[u].w = pack_h2(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
      }
      if (!second) {
#pragma unroll
        for (int u = 0; u < 4; u++)
          *reinterpret_cast<uint4*>(unit + U_WQ + (t >> 3) * SBO_K128 + (c0 / 8 + u) * LBO + (t & 7) * 16) = p[u];
      } else {
        uint4* dst = reinterpret_cast<uint4*>(unit + U_UL + (c0 / KNV) * (KC * KNV * 2) + t * (KNV * 2));
#pragma unroll
        for (int u = 0; u < 4; u++) dst[u] = p[u];
      }
    }
  }
  tc::fence_before_sync();
  prep_sync<SUB>(ctx);
  KT_TRACE(12);
}

template <bool GATED>
__global__ __launch_bounds__(256, 2) void kda_chunk_prep_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ g,
    const void* __restrict__ beta_in, uint8_t* __restrict__ ws, int seqlen, int H,
    int n_chunks, int prefetch_dist, int* __restrict__ status, const float* __restrict__ dt_bias,
    const float* __restrict__ a_log, float lower_bound) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  // heads are the fastest grid dimension: CTAs that run together read the same tokens, i.e. whole
  // contiguous rows of the activations
  const int head = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  // units are chunk-major: the CTAs that run together (same chunks, all heads) touch adjacent units, in
  // this kernel and in the scan, so their traffic spreads over all memory channels
  uint8_t* unit = ws + (((size_t)b * n_chunks + chunk) * H + head) * U_BYTES;
  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (tid < 32) tc::tmem_alloc(&tmem_slot, 256);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // the CTA that runs `prefetch_dist` blocks later (blocks are scheduled in linear order, heads fastest)
  const long long lin = (long long)blockIdx.y * H + blockIdx.x + prefetch_dist;
  const int pchunk = (int)(lin / H);
  PrepCtx ctx{smem, &bar, 0u, &abort_flag, tmem_slot, tid, 0, false, nullptr, 0, 0, nullptr};
  prep_unit<GATED, false>(ctx, qkv, g, beta_in, unit, seqlen, H, head, chunk, b, (int)(lin % H),
                          (prefetch_dist > 0 && pchunk < n_chunks) ? pchunk : -1, dt_bias, a_log, lower_bound);
  if (tid < 32) tc::tmem_dealloc(tmem_slot, 256);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

// =================================================================================================
// kernel 2: sequential scan over the chunks of one (batch, head, value slice)
// =================================================================================================
constexpr uint32_t S_WQ = 0;              // 32768
constexpr uint32_t S_BB = 32768;          // 16384: rows 0-63 zero (never overwritten), rows 64-127 = B beta
constexpr uint32_t S_KT = 49152;          // 16384
constexpr uint32_t S_UL = 65536;          // 4096
constexpr uint32_t S_DEC = 69632;         // 512
constexpr uint32_t S_STAGE = 70144;
constexpr uint32_t S_TX = 32768 + 8192 + 16384 + 4096 + 512;  // bytes landing per stage
constexpr int S_NSTAGE = 3;               // operand stages in flight: two chunks of lead time for the bulk copies
constexpr uint32_t P2_S = S_NSTAGE * S_STAGE;  // fp16 B operand: state slice [128 k][32], MN-major, 8 KB
constexpr uint32_t P2_U = P2_S + 8192;    // fp16 B operand: U [64 tokens][32], MN-major, 4 KB
constexpr uint32_t P2_SMEM = P2_U + 4096;

__global__ __launch_bounds__(128, 1) void kda_chunk_scan_kernel(
    const uint8_t* __restrict__ ws, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
    float* __restrict__ out_f32, int seqlen, int H, int n_chunks, const int* __restrict__ slots,
    float scale, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[S_NSTAGE];
  __shared__ uint64_t mma_bar;
  __shared__ uint64_t out_bar;    // completion of the output contraction (B beta) U, waited on by warps 2, 3 only
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vs = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int v0 = vs * KNV;
  const uint8_t* unit0 = ws + ((size_t)b * n_chunks * H + head) * U_BYTES;   // unit of chunk c: + c * H * U_BYTES
  const int slot = slots ? slots[b] : b;
  float* st = state + ((size_t)slot * H + head) * KD * KD + (size_t)tid * KD + v0;  // row k = tid

  if (tid == 0) {
    for (int i = 0; i < S_NSTAGE; i++) tc::mbar_init(&full_bar[i], 1);
    tc::mbar_init(&mma_bar, 1);
    tc::mbar_init(&out_bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 128);
  // zero halves of the [0 ; B beta] operands
  for (int i = tid; i < 8192 / 16; i += 128) {
    for (int st_i = 0; st_i < S_NSTAGE; st_i++) reinterpret_cast<uint4*>(smem + st_i * S_STAGE + S_BB)[i] = make_uint4(0, 0, 0, 0);
  }
  // state slice: thread = k row, 32 fp32 values in registers; fp16 copy as the B operand
  float S[KNV];
#pragma unroll
  for (int u = 0; u < KNV / 4; u++) {
    const float4 v = *reinterpret_cast<const float4*>(st + u * 4);
    S[4 * u] = v.x; S[4 * u + 1] = v.y; S[4 * u + 2] = v.z; S[4 * u + 3] = v.w;
  }
  // B operand, MN-major: off(k, n) = (n/8)*2048 + (k/8)*128 + (k%8)*16 + (n%8)*2
  uint8_t* sS_row = smem + P2_S + (tid >> 3) * 128 + (tid & 7) * 16;
#pragma unroll
  for (int u = 0; u < 4; u++) {
    uint4 p;
    p.x = pack_h2(S[8 * u], S[8 * u + 1]); p.y = pack_h2(S[8 * u + 2], S[8 * u + 3]);
    p.z = pack_h2(S[8 * u + 4], S[8 * u + 5]); p.w = pack_h2(S[8 * u + 6], S[8 * u + 7]);
    *reinterpret_cast<uint4*>(sS_row + u * 2048) = p;
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  // D1 alternates between two column ranges by chunk parity: the output rows of chunk c are read while the first
  // contraction of chunk c + 1 fills the other range
  const uint32_t d2 = tmem + 32;

  auto issue_loads = [&](int chunk) {
    uint8_t* stg = smem + (chunk % S_NSTAGE) * S_STAGE;
    const uint8_t* u = unit0 + (size_t)chunk * H * U_BYTES;
    uint64_t* bar = &full_bar[chunk % S_NSTAGE];
    tc::mbar_arrive_expect_tx(bar, S_TX);
    tc::bulk_g2s(stg + S_WQ, u + U_WQ, 32768, bar);
    tc::bulk_g2s(stg + S_BB + 8192, u + U_BB, 8192, bar);
    tc::bulk_g2s(stg + S_KT, u + U_KT, 16384, bar);
    tc::bulk_g2s(stg + S_UL, u + U_UL + vs * (KC * KNV * 2), 4096, bar);
    tc::bulk_g2s(stg + S_DEC, u + U_DEC, 512, bar);
  };
  if (tid == 0) {
    for (int c = 0; c < S_NSTAGE && c < n_chunks; c++) issue_loads(c);
  }

  const uint32_t idesc = tc::make_idesc(128, KNV, tc::FMT_F16, tc::FMT_F16, false, true);
  const uint32_t s_addr = tc::smem_u32(smem + P2_S), u_addr = tc::smem_u32(smem + P2_U);
  // The contractions are issued by the whole of warp 0 with one elected lane (descriptors stay warp-uniform for the
  // compiler: ~41 instead of ~47 cycles per M128 N32 product, see tc05.cuh).  Every wait of this kernel is executed
  // by all lanes, so warp 0 stays converged from one contraction to the next.
  const bool issue_warp = tc::warp_index_uniform() == 0;
  const uint32_t leader = issue_warp ? tc::elect_one() : 0u;
  uint32_t mma_parity = 0, out_parity = 0;

  // output rows of chunk c (TMEM lanes 64-127 of that chunk's D1 range = tokens), warps 2 and 3
  auto emit_outputs = [&](int c, bool valid) {
    const int tok = c * KC + (tid - 64);
    uint32_t r[32];
    tc::tmem_ld32(tmem + ((c & 1) ? 64u : 0u) + ((uint32_t)(warp * 32) << 16), r);
    tc::tmem_ld_wait();
    if (tok < seqlen && valid) {
      const size_t oi = (((size_t)b * seqlen + tok) * H + head) * KD + v0;
      uint4* o = reinterpret_cast<uint4*>(out + oi);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float a = __uint_as_float(r[8 * u + 2 * e]) * scale, c2 = __uint_as_float(r[8 * u + 2 * e + 1]) * scale;
          const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rz(a));
          const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rz(c2));
          w[e] = lo | (hi << 16);
        }
        o[u] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (out_f32) {
        float4* of = reinterpret_cast<float4*>(out_f32 + oi);
#pragma unroll
        for (int u = 0; u < 8; u++)
          of[u] = make_float4(__uint_as_float(r[4 * u]) * scale, __uint_as_float(r[4 * u + 1]) * scale,
                              __uint_as_float(r[4 * u + 2]) * scale, __uint_as_float(r[4 * u + 3]) * scale);
      }
    }
  };
  bool prev_ok = true;                                      // warps 2, 3: the previous chunk's waits all succeeded

  for (int chunk = 0; chunk < n_chunks; chunk++) {
    const int sidx = chunk % S_NSTAGE;
    uint8_t* stg = smem + sidx * S_STAGE;
    const uint32_t stg_addr = tc::smem_u32(stg);
    const uint32_t d1 = tmem + ((chunk & 1) ? 64u : 0u);
    KS_TRACE(0, chunk);
    bool ok = tc::mbar_wait(&full_bar[sidx], (chunk / S_NSTAGE) & 1, &abort_flag, 2);
    KS_TRACE(1, chunk);
    // ---- [W ; Q+] S0 -> D1 (128 x 32) ----
    if (issue_warp) {
#pragma unroll
      for (int kk = 0; kk < KD / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_WQ + kk * 2 * LBO, LBO, SBO_K128);
        const uint64_t bd = tc::make_sdesc(s_addr + kk * 2 * 128, 128, 2048);
        tc::mma_f16_if(leader, d1, ad, bd, idesc, kk > 0);
      }
      tc::mma_commit_if(leader, &mma_bar);
    }
    // the previous chunk's output rows leave while this chunk's first contraction runs (off the chain)
    if (warp >= 2 && chunk > 0) emit_outputs(chunk - 1, prev_ok);
    ok = tc::mbar_wait(&mma_bar, mma_parity, &abort_flag, 3) && ok;
    mma_parity ^= 1;
    tc::fence_after_sync();
    KS_TRACE(2, chunk);
    // ---- U = Uloc - W S0 (token rows = TMEM lanes 0-63) ----
    if (warp < 2) {
      const int t = tid;
      uint32_t r[32];
      tc::tmem_ld32(d1 + ((uint32_t)(warp * 32) << 16), r);
      tc::tmem_ld_wait();
      const uint4* ul = reinterpret_cast<const uint4*>(stg + S_UL + t * (KNV * 2));
      uint8_t* urow = smem + P2_U + (t >> 3) * 128 + (t & 7) * 16;  // off(k=t, n) = (n/8)*1024 + ...
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const uint4 lv = ul[u];
        const __half2* lh = reinterpret_cast<const __half2*>(&lv);
        float uu[8];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float2 f = __half22float2(lh[e]);
          uu[2 * e] = f.x - __uint_as_float(r[8 * u + 2 * e]);
          uu[2 * e + 1] = f.y - __uint_as_float(r[8 * u + 2 * e + 1]);
        }
        uint4 p;
        p.x = pack_h2(uu[0], uu[1]); p.y = pack_h2(uu[2], uu[3]); p.z = pack_h2(uu[4], uu[5]); p.w = pack_h2(uu[6], uu[7]);
        *reinterpret_cast<uint4*>(urow + u * 1024) = p;
      }
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    KS_TRACE(3, chunk);
    // ---- D2 = Kt^T U (state path, committed first) ;  D1 rows 64-127 += (B beta) U (outputs, own barrier) ----
    if (issue_warp) {
#pragma unroll
      for (int kk = 0; kk < KC / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_KT + kk * 2 * LBO, LBO, SBO_K64);
        const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
        tc::mma_f16_if(leader, d2, ad, bd, idesc, kk > 0);
      }
      tc::mma_commit_if(leader, &mma_bar);
#pragma unroll
      for (int kk = 0; kk < KC / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_BB + kk * 2 * LBO, LBO, SBO_K64);
        const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
        tc::mma_f16_if(leader, d1, ad, bd, idesc, true);
      }
      tc::mma_commit_if(leader, &out_bar);
    }
    ok = tc::mbar_wait(&mma_bar, mma_parity, &abort_flag, 4) && ok;
    mma_parity ^= 1;
    tc::fence_after_sync();
    KS_TRACE(4, chunk);
    // ---- state: S <- S e^{G_last} + Kt^T U (lane = k row), refresh the fp16 operand copy.  The output
    //      contraction is still running: only the state is on the chunk-to-chunk chain. ----
    {
      uint32_t r[32];
      tc::tmem_ld32(d2 + ((uint32_t)(warp * 32) << 16), r);
      tc::tmem_ld_wait();
      const float dec = reinterpret_cast<const float*>(stg + S_DEC)[tid];
#pragma unroll
      for (int j = 0; j < KNV; j++) S[j] = fmaf(S[j], dec, __uint_as_float(r[j]));
#pragma unroll
      for (int u = 0; u < 4; u++) {
        uint4 p;
        p.x = pack_h2(S[8 * u], S[8 * u + 1]); p.y = pack_h2(S[8 * u + 2], S[8 * u + 3]);
        p.z = pack_h2(S[8 * u + 4], S[8 * u + 5]); p.w = pack_h2(S[8 * u + 6], S[8 * u + 7]);
        *reinterpret_cast<uint4*>(sS_row + u * 2048) = p;
      }
    }
    KS_TRACE(5, chunk);
    // ---- warps 2, 3 make sure the output contraction is complete before the block barrier (the stage and the U
    //      tile it reads are rewritten after it); the rows themselves are read in the next iteration ----
    if (warp >= 2) {
      ok = tc::mbar_wait(&out_bar, out_parity, &abort_flag, 5) && ok;
      prev_ok = ok;
    }
    out_parity ^= 1;
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    KS_TRACE(6, chunk);
    // The refill is issued by a thread of warp 3, not by thread 0: the five copy instructions take about 400 cycles
    // to issue, which the MMA-issuing thread would add to the per-chunk chain (measured: 1.95 -> 1.87 ms at 32K
    // tokens).  Issuing them while the next contraction runs instead was slower (the barrier polls queue behind them).
    if (tid == 96 && chunk + S_NSTAGE < n_chunks) issue_loads(chunk + S_NSTAGE);
  }
  if (warp >= 2 && n_chunks > 0) emit_outputs(n_chunks - 1, prev_ok);
  if (!abort_flag) {
#pragma unroll
    for (int u = 0; u < KNV / 4; u++)
      *reinterpret_cast<float4*>(st + u * 4) = make_float4(S[4 * u], S[4 * u + 1], S[4 * u + 2], S[4 * u + 3]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 128);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}


// =================================================================================================
// fused form: preparation and scan in ONE persistent launch
//
// One CTA of 512 threads per SM.  The first n_slots CTAs are chain slots: each walks the chunks of one (batch, head)
// chain - or, when the call has more than 48 chains, of n_jobs / n_slots chains one after the other (the state is
// swapped at the chain boundary; ring, flags and barrier parities go by the slot's running chunk number) - with the
// whole 128-column state of the head, sixteen warps = four TMEM lane quarters x four 32-column blocks.  Every other CTA
// hosts two preparation workers of 256 threads (its two halves, each with its own shared memory, TMEM columns and
// named barrier), which take the units round robin in the order the slots need them.  A unit travels through a ring
// of KR chunk slots per chain slot in global memory - a few tens of MB that stay in L2 - instead of a per-chunk workspace in HBM:
//   ready[slot][v % KR] = v + 1 once the unit of that chunk is complete (release store after the worker's writes),
//   consumed[job]     = number of chunks whose unit has landed in the chain CTA's shared memory (the slot of chunk c
//                       may be rewritten once consumed > c).
// A worker that finds its slot still occupied, and a chain CTA that finds its unit not yet written, poll with a
// bound (about a second); on expiry they record HK_ERR_TIMEOUT, raise the launch-wide abort word and finish without
// waiting again.  All CTAs must be resident at once: the launch is cooperative and sized to the SM count.
// =================================================================================================
constexpr int KR = 16;                                    // ring slots (chunks) per chain
constexpr int F_NSTAGE = 2;                               // the ring protocol of the chain CTA is written for two stages
constexpr uint32_t F_WQ = 0;                              // 32768
constexpr uint32_t F_BB = 32768;                          // 16384: rows 0-63 zero (never overwritten), rows 64-127 = B beta
constexpr uint32_t F_KT = 49152;                          // 16384
constexpr uint32_t F_UL = 65536;                          // 16384: Uloc as [4 column blocks][64 tokens][32]
constexpr uint32_t F_DEC = 81920;                         // 512
constexpr uint32_t F_STAGE = 82432;
constexpr uint32_t F_S = F_NSTAGE * F_STAGE;              // fp16 B operand: state [128 k][128 v], MN-major, 32 KB
constexpr uint32_t F_U = F_S + 32768;                     // fp16 B operand: U [64 tokens][128 v], MN-major, 16 KB
constexpr uint32_t F_O = F_U + 16384;                     // bf16 output rows of one chunk: two swizzled 8 KB boxes for the tiled
                                                          // stores, or plain [64 tokens][256 B] rows when the kernel stores itself
constexpr uint32_t F_OPITCH = 256;
constexpr uint32_t F_SMEM_SCAN = F_O + KC * F_OPITCH + 1024;   // + slack to start the tiles at a 1 KB boundary
static_assert(F_O % 1024 == 0 && KC * F_OPITCH >= 16384, "the output tile holds two 8 KB swizzled boxes");
constexpr uint32_t F_SMEM = F_SMEM_SCAN > 2 * P1_SMEM ? F_SMEM_SCAN : 2 * P1_SMEM;
static_assert(U_KT + 16384 == U_UL && U_UL + 16384 == U_DEC && F_KT + 16384 == F_UL && F_UL + 16384 == F_DEC,
              "Kt^T, Uloc and the decay row travel as one copy");
constexpr int F_FLAG_INTS = 16;                           // [0] launch-wide abort word; the flag arrays follow

template <bool GATED>
__global__ __launch_bounds__(512, 1) void kda_fused_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ g, const void* __restrict__ beta_in,
    uint8_t* __restrict__ ring, int* __restrict__ flags, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
    float* __restrict__ out_f32, int seqlen, int H, int n_chunks, int n_jobs, int n_slots, const int* __restrict__ slots,
    float scale, int* __restrict__ status, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
    float lower_bound, const __grid_constant__ CUtensorMap tmap_out, int use_tma_out) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[F_NSTAGE];
  // chain: one barrier per contraction group, each completing once per chunk (parity = chunk & 1); the output warps
  // never wait for the first one, which a barrier shared by both groups would not allow (a skipped phase aliases)
  __shared__ uint64_t mma_bar;       // chain: [W;Q+] S0;       preparation worker 0: its product
  __shared__ uint64_t mma2_bar;      // chain: Kt^T U (state path)
  __shared__ uint64_t out_bar;       // chain: (B beta) U;      preparation worker 1: its product
  __shared__ uint64_t u_bar;         // chain: the 256 token-row threads have written U (count 256)
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
#ifdef HK_DIAG
  if (tid == 0 && blockIdx.x == 1) hk_kda_trace[32 + 11] = clock64();
#endif
  int* g_abort = flags;
  // A chain CTA ("slot") walks n_jobs / n_slots chains one after the other: its running chunk number v counts through
  // all of them (chain v / n_chunks of the slot, chunk v % n_chunks), and ring, flags and barrier parities go by v.
  int* ready = flags + F_FLAG_INTS;                        // [n_slots][KR]
  int* consumed = ready + (size_t)n_slots * KR;            // [n_slots]
  const int n_virtual = (n_jobs / n_slots) * n_chunks;     // chunks a slot walks

  if (tid == 0) {
    for (int i = 0; i < F_NSTAGE; i++) tc::mbar_init(&full_bar[i], 1);
    tc::mbar_init(&mma_bar, 1);
    tc::mbar_init(&mma2_bar, 1);
    tc::mbar_init(&out_bar, 1);
    tc::mbar_init(&u_bar, 256);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  uint8_t* const smem_base = smem;

  if ((int)blockIdx.x >= n_slots) {
    // =========================== two preparation workers ===========================
    const int sub = warp >> 3;
#ifdef HK_DIAG_ONE_WORKER
    const int worker = (int)blockIdx.x - n_slots, n_workers = (int)gridDim.x - n_slots;
#else
    const int worker = ((int)blockIdx.x - n_slots) * 2 + sub, n_workers = ((int)gridDim.x - n_slots) * 2;
#endif
    const long long n_units = (long long)n_chunks * n_jobs;
    PrepCtx ctx{smem + sub * P1_SMEM, sub ? &out_bar : &mma_bar, 0u, &abort_flag, tmem + sub * 256, tid & 255, 1 + sub, false,
                nullptr, 0, 0, g_abort};
#ifdef HK_DIAG
    ctx.trace = false;
#endif
    int it = 0;
#ifdef HK_DIAG_ONE_WORKER
    if (sub == 1) goto prep_done;                          // diagnostic: stage times of a worker that has its SM alone
#endif
    for (long long u = worker; u < n_units; u += n_workers, it++) {
      // units in the order the slots need them: running chunk v of every slot, then v + 1, ...
      const int v = (int)(u / n_slots), slot = (int)(u % n_slots);
      const int chunk = v % n_chunks, job = slot + n_slots * (v / n_chunks);
      const int b = job / H, head = job % H;
#ifdef HK_DIAG
      ctx.trace = (worker == 7 && it == 20);
#endif
      // the slot of this chunk must have been drained by the chain CTA (it held chunk - KR): thread 0 asks now and
      // looks at the answer just before the worker's first write to the unit (prep_unit calls slot_wait there)
      ctx.slot_flag = consumed + slot;
      ctx.slot_want = v >= KR ? v - KR + 1 : 0;
      ctx.slot_seen = (ctx.tid == 0 && ctx.slot_want > 0) ? ld_relaxed_gpu(ctx.slot_flag) : 0;
      uint8_t* unit = ring + ((size_t)(v % KR) * n_slots + slot) * U_BYTES;
      const long long pu = u + n_workers;
      int pf_head = 0, pf_chunk = -1;
      if (pu < n_units) {
        const int pv = (int)(pu / n_slots), pjob = (int)(pu % n_slots) + n_slots * (pv / n_chunks);
        if (pjob / H == b) { pf_chunk = pv % n_chunks; pf_head = pjob % H; }
      }
      ctx.bar_parity = it & 1;
      KT_TRACE(14);
      prep_unit<GATED, true>(ctx, qkv, g, beta_in, unit, seqlen, H, head, chunk, b, pf_head, pf_chunk, dt_bias, a_log, lower_bound);
      // publish: prep_unit ends with the worker's barrier, so every thread's writes of this unit precede this
      // release store (which is cumulative over them)
      if (ctx.tid == 0) st_release_gpu(ready + (size_t)slot * KR + (v % KR), v + 1);
      KT_TRACE(15);
      KT_FLUSH();
    }
#ifdef HK_DIAG_ONE_WORKER
  prep_done:;
#endif
  } else {
    // =========================== one (batch, head) chain ===========================
    // the chain CTA's tiles start at a 1 KB boundary (the output tile is written in the 128-byte-swizzle pattern,
    // which is a function of the shared-memory address)
    uint8_t* const smem = smem_base + ((1024u - (tc::smem_u32(smem_base) & 1023u)) & 1023u);
    const int cslot = blockIdx.x;                           // this CTA's chain slot
    const int lq = warp & 3, cb = warp >> 2;               // TMEM lane quarter, 32-column block
    const int rowi = lq * 32 + (tid & 31);                       // k row of the state / token row of W S0 / output row - 64
    const int v0 = cb * KNV;
    // chain number `ci` of this slot: (batch, head) = job cslot + n_slots * ci; its state rows for this thread
    auto chain_state = [&](int ci) -> float* {
      const int job = cslot + n_slots * ci, jb = job / H, jh = job % H;
      const int sl = slots ? slots[jb] : jb;
      return state + ((size_t)sl * H + jh) * KD * KD + (size_t)rowi * KD + v0;
    };
    float* st = chain_state(0);
    const int* my_ready = ready + (size_t)cslot * KR;

    for (int i = tid; i < 8192 / 16; i += 512)
      for (int s_i = 0; s_i < F_NSTAGE; s_i++) reinterpret_cast<uint4*>(smem + s_i * F_STAGE + F_BB)[i] = make_uint4(0, 0, 0, 0);
    float S[KNV];
#pragma unroll
    for (int u = 0; u < KNV / 4; u++) {
      const float4 v = *reinterpret_cast<const float4*>(st + u * 4);
      S[4 * u] = v.x; S[4 * u + 1] = v.y; S[4 * u + 2] = v.z; S[4 * u + 3] = v.w;
    }
    // B operand, MN-major, N = 128: off(k, n) = (n/8)*2048 + (k/8)*128 + (k%8)*16 + (n%8)*2
    uint8_t* sS_row = smem + F_S + (4 * cb) * 2048 + (rowi >> 3) * 128 + (rowi & 7) * 16;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      uint4 p;
      p.x = pack_h2(S[8 * u], S[8 * u + 1]); p.y = pack_h2(S[8 * u + 2], S[8 * u + 3]);
      p.z = pack_h2(S[8 * u + 4], S[8 * u + 5]); p.w = pack_h2(S[8 * u + 6], S[8 * u + 7]);
      *reinterpret_cast<uint4*>(sS_row + u * 2048) = p;
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t d2 = tmem + 256;                        // D1 alternates between columns 0-127 and 128-255

    // the producer thread (a lane of the last warp, which is never on the token-row path) owns the ring protocol
    const bool producer = tid == 480;
    int issued = 0;                                        // producer only: chunks whose copies have been issued
    auto issue_loads = [&](int chunk) {
      uint8_t* stg = smem + (chunk % F_NSTAGE) * F_STAGE;
      const uint8_t* u = ring + ((size_t)(chunk % KR) * n_slots + cslot) * U_BYTES;
      uint64_t* bar = &full_bar[chunk % F_NSTAGE];
      fence_proxy_async_all();
      tc::mbar_arrive_expect_tx(bar, U_BYTES);
      tc::bulk_g2s(stg + F_WQ, u + U_WQ, 32768, bar);
      tc::bulk_g2s(stg + F_BB + 8192, u + U_BB, 8192, bar);
      tc::bulk_g2s(stg + F_KT, u + U_KT, 16384 + 16384 + 512, bar);
    };
    if (producer) {
      for (; issued < F_NSTAGE && issued < n_virtual; issued++) {
        poll_flag_ge(my_ready + (issued % KR), issued + 1, &abort_flag, g_abort, 21);
        issue_loads(issued);
      }
    }

    const uint32_t idesc = tc::make_idesc(128, KD, tc::FMT_F16, tc::FMT_F16, false, true);
    const uint32_t s_addr = tc::smem_u32(smem + F_S), u_addr = tc::smem_u32(smem + F_U);
    // two issuing warps: warp 0 the contractions on the chain ([W;Q+] S0 and Kt^T U), warp 2 (an output warp) the
    // output contraction (B beta) U, so that warp 0 does not spend its issue time before its share of the state update
    const int warp_u = tc::warp_index_uniform();
    const bool issue_warp = warp_u == 0, out_issue_warp = warp_u == 2;
    const uint32_t leader = (issue_warp || out_issue_warp) ? tc::elect_one() : 0u;

    // Output rows of chunk c: TMEM lanes 64-127 of that chunk's D1 range = tokens, lane quarters 2 and 3 (eight warps =
    // two token halves x four column blocks).  A thread holds 32 columns of one token; stored directly, a warp-wide
    // 16-byte store would touch 32 different rows (32 L1 requests per instruction, over a thousand per chunk on this
    // one SM).  The bf16 rows are therefore assembled in shared memory (272-byte pitch: conflict-free both ways) and
    // written out with every warp instruction covering two whole 256-byte rows.  The eight warps meet at a named
    // barrier of their own; the block barriers of the chain separate one chunk's reads from the next chunk's writes.
    // With a tensor map over the output the rows leave as TWO tiled TMA stores per chunk (64 tokens x 64 channels each,
    // 128-byte-swizzle boxes; rows past the end of the sequence are clipped by the copy engine): the tile is written
    // conflict-free (16-byte piece p of row r at p ^ (r % 8)) and one thread hands it over.
    auto emit_outputs = [&](int vc, bool valid) {          // vc: running chunk number of the slot
      const int c = vc % n_chunks, ejob = cslot + n_slots * (vc / n_chunks), b = ejob / H, head = ejob % H;
      const int trow = rowi - 64;
      uint32_t r[32];
      tc::tmem_ld32(tmem + ((vc & 1) ? 128u : 0u) + (uint32_t)v0 + ((uint32_t)(lq * 32) << 16), r);
      tc::tmem_ld_wait();
      const bool issuer = warp == 2 && (tid & 31) == 0;
      if (use_tma_out) {
        if (issuer) tc::bulk_wait_read<0>();               // the previous chunk's tile has been read by the copy engine
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      uint8_t* orow = use_tma_out ? smem + F_O + (cb >> 1) * 8192 + trow * 128 : smem + F_O + trow * F_OPITCH + cb * (KNV * 2);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float a = __uint_as_float(r[8 * u + 2 * e]) * scale, c2 = __uint_as_float(r[8 * u + 2 * e + 1]) * scale;
          const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rz(a));
          const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rz(c2));
          w[e] = lo | (hi << 16);
        }
        const int off = use_tma_out ? ((((cb & 1) * 4 + u) ^ (trow & 7)) << 4) : u * 16;
        *reinterpret_cast<uint4*>(orow + off) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (use_tma_out) {
        tc::fence_async_smem();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (issuer && valid) {
#pragma unroll
          for (int hb = 0; hb < 2; hb++)
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(&tmap_out),
                         "r"(hb * 64), "r"(head), "r"(c * KC), "r"(b), "r"(tc::smem_u32(smem + F_O + hb * 8192))
                         : "memory");
          tc::bulk_commit();
        }
      } else {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const int ot = (lq - 2) * 128 + cb * 32 + (tid & 31);   // 0..255 over the eight output warps
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int piece = ot + 256 * i, prow = piece >> 4, pc = piece & 15;
          const int ptok = c * KC + prow;
          if (ptok < seqlen && valid) {
            const uint4 v = *reinterpret_cast<const uint4*>(smem + F_O + prow * F_OPITCH + pc * 16);
            *reinterpret_cast<uint4*>(out + (((size_t)b * seqlen + ptok) * H + head) * KD + pc * 8) = v;
          }
        }
      }
      const int tok = c * KC + trow;
      if (out_f32 && tok < seqlen && valid) {
        float4* of = reinterpret_cast<float4*>(out_f32 + (((size_t)b * seqlen + tok) * H + head) * KD + v0);
#pragma unroll
        for (int u = 0; u < 8; u++)
          of[u] = make_float4(__uint_as_float(r[4 * u]) * scale, __uint_as_float(r[4 * u + 1]) * scale,
                              __uint_as_float(r[4 * u + 2]) * scale, __uint_as_float(r[4 * u + 3]) * scale);
      }
    };
    bool prev_ok = true;

    // `chunk` is the slot's RUNNING chunk number over all of its chains
    for (int chunk = 0; chunk < n_virtual; chunk++) {
      if (chunk > 0 && chunk % n_chunks == 0) {
        // the next chain of this slot: its state replaces the previous one (stored at the end of the last iteration)
        st = chain_state(chunk / n_chunks);
#pragma unroll
        for (int u = 0; u < KNV / 4; u++) {
          const float4 v = *reinterpret_cast<const float4*>(st + u * 4);
          S[4 * u] = v.x; S[4 * u + 1] = v.y; S[4 * u + 2] = v.z; S[4 * u + 3] = v.w;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          uint4 p;
          p.x = pack_h2(S[8 * u], S[8 * u + 1]); p.y = pack_h2(S[8 * u + 2], S[8 * u + 3]);
          p.z = pack_h2(S[8 * u + 4], S[8 * u + 5]); p.w = pack_h2(S[8 * u + 6], S[8 * u + 7]);
          *reinterpret_cast<uint4*>(sS_row + u * 2048) = p;
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();
      }
      const int sidx = chunk % F_NSTAGE;
      uint8_t* stg = smem + sidx * F_STAGE;
      const uint32_t stg_addr = tc::smem_u32(stg);
      const uint32_t d1 = tmem + ((chunk & 1) ? 128u : 0u);
      int next_flag = 0;
      if (producer && issued <= chunk) {                   // the earlier attempts found the unit not written yet
        poll_flag_ge(my_ready + (chunk % KR), chunk + 1, &abort_flag, g_abort, 22);
        issue_loads(chunk);
        issued = chunk + 1;
      }
      KS_TRACE(0, chunk);
      KS_TRACE_AT(8, chunk, 0);
      KS_TRACE_AT(9, chunk, 50);
      KS_TRACE_AT(10, chunk, 450);
      bool ok = tc::mbar_wait(&full_bar[sidx], (chunk / F_NSTAGE) & 1, &abort_flag, 2);
      KS_TRACE(1, chunk);
      // ---- [W ; Q+] S0 -> D1 (128 x 128) ----
      if (issue_warp) {
#pragma unroll
        for (int kk = 0; kk < KD / 16; kk++) {
          const uint64_t ad = tc::make_sdesc(stg_addr + F_WQ + kk * 2 * LBO, LBO, SBO_K128);
          const uint64_t bd = tc::make_sdesc(s_addr + kk * 2 * 128, 128, 2048);
          tc::mma_f16_if(leader, d1, ad, bd, idesc, kk > 0);
        }
        tc::mma_commit_if(leader, &mma_bar);
      }
      // the previous chunk's output rows leave while this chunk's first contraction runs (off the chain)
      const uint32_t cpar = chunk & 1;
      if (lq >= 2 && chunk > 0) emit_outputs(chunk - 1, prev_ok);
      if (lq < 2) {
        ok = tc::mbar_wait(&mma_bar, cpar, &abort_flag, 3) && ok;
        tc::fence_after_sync();
      }
      KS_TRACE(2, chunk);
      // ---- U = Uloc - W S0 (token rows = TMEM lanes 0-63) ----
      if (lq < 2) {
        const int t = rowi;
        uint32_t r[32];
        tc::tmem_ld32(d1 + (uint32_t)v0 + ((uint32_t)(lq * 32) << 16), r);
        tc::tmem_ld_wait();
        const uint4* ul = reinterpret_cast<const uint4*>(stg + F_UL + cb * (KC * KNV * 2) + t * (KNV * 2));
        uint8_t* urow = smem + F_U + (4 * cb) * 1024 + (t >> 3) * 128 + (t & 7) * 16;   // off(k=t, n) = (n/8)*1024 + ...
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const uint4 lv = ul[u];
          const __half2* lh = reinterpret_cast<const __half2*>(&lv);
          float uu[8];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float2 f = __half22float2(lh[e]);
            uu[2 * e] = f.x - __uint_as_float(r[8 * u + 2 * e]);
            uu[2 * e + 1] = f.y - __uint_as_float(r[8 * u + 2 * e + 1]);
          }
          uint4 p;
          p.x = pack_h2(uu[0], uu[1]); p.y = pack_h2(uu[2], uu[3]); p.z = pack_h2(uu[4], uu[5]); p.w = pack_h2(uu[6], uu[7]);
          *reinterpret_cast<uint4*>(urow + u * 1024) = p;
        }
      }
      // U is complete when all 256 token-row threads have arrived (after their proxy fence); the two issuing warps
      // wait for that, nobody else does
      if (lq < 2) {
        tc::fence_async_smem();
        tc::mbar_arrive(&u_bar);
      }
      KS_TRACE(3, chunk);
      // The ring protocol runs here, while the producer's warp has nothing to do until the state contraction is
      // complete.  None of it waits for this thread's earlier global stores (a release store or a fence would, and
      // the block barriers of the chain would then wait for the output rows to reach memory).
      if (producer) {
        // the unit of this chunk has landed in shared memory: its slot may be rewritten.  A relaxed store is enough:
        // the copy engine's reads are complete, nothing this thread wrote is handed over with the flag.
        st_relaxed_gpu(consumed + cslot, chunk + 1);
        // catch-up: the other stage is free while the next chunk's copies have not been issued
        if (issued == chunk + 1 && chunk + 1 < n_virtual && ld_acquire_gpu(my_ready + ((chunk + 1) % KR)) >= chunk + 2) {
          issue_loads(chunk + 1);
          issued = chunk + 2;
        }
        // sampled now, used when this chunk's stage is released at the end of the iteration
        if (issued == chunk + 2 && chunk + 2 < n_virtual) next_flag = ld_acquire_gpu(my_ready + ((chunk + 2) % KR));
      }
      // ---- D2 = Kt^T U (state path, warp 0) ;  D1 rows 64-127 += (B beta) U (outputs, warp 2, own barrier) ----
      if (issue_warp) {
        ok = tc::mbar_wait(&u_bar, cpar, &abort_flag, 6) && ok;
        tc::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < KC / 16; kk++) {
          const uint64_t ad = tc::make_sdesc(stg_addr + F_KT + kk * 2 * LBO, LBO, SBO_K64);
          const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
          tc::mma_f16_if(leader, d2, ad, bd, idesc, kk > 0);
        }
        tc::mma_commit_if(leader, &mma2_bar);
      }
      if (out_issue_warp) {
        ok = tc::mbar_wait(&u_bar, cpar, &abort_flag, 7) && ok;
        tc::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < KC / 16; kk++) {
          const uint64_t ad = tc::make_sdesc(stg_addr + F_BB + kk * 2 * LBO, LBO, SBO_K64);
          const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
          tc::mma_f16_if(leader, d1, ad, bd, idesc, true);
        }
        tc::mma_commit_if(leader, &out_bar);
      }
      ok = tc::mbar_wait(&mma2_bar, cpar, &abort_flag, 4) && ok;
      tc::fence_after_sync();
      KS_TRACE(4, chunk);
      // ---- state: S <- S e^{G_last} + Kt^T U (lane = k row), refresh the fp16 operand copy ----
      {
        uint32_t r[32];
        tc::tmem_ld32(d2 + (uint32_t)v0 + ((uint32_t)(lq * 32) << 16), r);
        tc::tmem_ld_wait();
        const float dec = reinterpret_cast<const float*>(stg + F_DEC)[rowi];
#pragma unroll
        for (int j = 0; j < KNV; j++) S[j] = fmaf(S[j], dec, __uint_as_float(r[j]));
#pragma unroll
        for (int u = 0; u < 4; u++) {
          uint4 p;
          p.x = pack_h2(S[8 * u], S[8 * u + 1]); p.y = pack_h2(S[8 * u + 2], S[8 * u + 3]);
          p.z = pack_h2(S[8 * u + 4], S[8 * u + 5]); p.w = pack_h2(S[8 * u + 6], S[8 * u + 7]);
          *reinterpret_cast<uint4*>(sS_row + u * 2048) = p;
        }
      }
      if (chunk % n_chunks == n_chunks - 1 && !abort_flag) {
        // last chunk of a chain: its final state goes back to memory
#pragma unroll
        for (int u = 0; u < KNV / 4; u++)
          *reinterpret_cast<float4*>(st + u * 4) = make_float4(S[4 * u], S[4 * u + 1], S[4 * u + 2], S[4 * u + 3]);
      }
      KS_TRACE(5, chunk);
      // the output contraction must be complete before the block barrier: the stage and the U tile it reads are
      // rewritten after it; the rows themselves are read in the next iteration
      if (lq >= 2) {
        ok = tc::mbar_wait(&out_bar, cpar, &abort_flag, 5) && ok;
        prev_ok = ok;
      }
      tc::fence_async_smem();
      tc::fence_before_sync();
      __syncthreads();
      tc::fence_after_sync();
      KS_TRACE(6, chunk);
      // refill of this stage, if the unit two chunks ahead was already complete when its flag was sampled
      if (producer && issued == chunk + 2 && chunk + 2 < n_virtual && next_flag >= chunk + 3) {
        issue_loads(chunk + 2);
        issued = chunk + 3;
      }
    }
    if (lq >= 2 && n_virtual > 0) {
      emit_outputs(n_virtual - 1, prev_ok);
      if (use_tma_out && warp == 2 && (tid & 31) == 0) tc::bulk_wait_all<0>();
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

}  // namespace hk

#ifdef HK_DIAG
extern "C" __attribute__((visibility("default"))) int hk_debug_kda_trace(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, hk::hk_kda_trace, sizeof(long long) * 128) == cudaSuccess ? 0 : 3;
}
#endif

namespace hk {
namespace {
// The fused launch serves calls with few (batch, head) chains: every chain occupies one SM, the rest prepare.
// hk_kda_chunked_set_form(1) keeps the two-kernel form for every call (cross-check of the two forms in the tests).
int g_chunked_form = 0;
// Number of chain CTAs ("slots") of the fused launch for n_jobs (batch, head) chains, 0 = use the two-kernel form.  Up to
// 48 chains get a slot each; more chains share slots (a slot walks its chains one after the other), which needs a slot
// count that divides n_jobs: the largest divisor in [16, 48] that leaves at least 64 SMs to the preparation.
int fused_slots(long long n_jobs) {
  if (g_chunked_form != 0 || n_jobs <= 0) return 0;
  const int room = sm_count() - 64;
  for (int d = 48; d >= 1; d--) {
    if (d > room || n_jobs % d != 0) continue;
    if (d == n_jobs || d >= 16) return d;
    break;
  }
  return 0;
}
size_t fused_flag_bytes(int n_slots) {
  return (((size_t)F_FLAG_INTS + (size_t)n_slots * (KR + 1)) * sizeof(int) + 255) / 256 * 256;
}
}  // namespace
}  // namespace hk

HK_API int hk_kda_dispatch_is_chunked(int seqlen, int num_k_heads, int num_v_heads, int k_head_dim, int v_head_dim,
                                      int history_stride, int channelwise, int history) {
  return (channelwise && !history && seqlen >= hk::KC && k_head_dim == hk::KD && v_head_dim == hk::KD &&
          num_k_heads == num_v_heads && history_stride == 1)
             ? 1
             : 0;
}

HK_API int hk_kda_chunked_set_form(int form) {
  if (form != 0 && form != 1) return HK_ERR_INVALID;
  hk::g_chunked_form = form;
  return HK_OK;
}

HK_API size_t hk_kda_chunked_workspace_bytes(int bsz, int seqlen, int num_heads) {
  if (bsz <= 0 || seqlen <= 0 || num_heads <= 0) return 0;
  const long long n_jobs = (long long)bsz * num_heads;
  if (const int n_slots = hk::fused_slots(n_jobs))
    return hk::fused_flag_bytes(n_slots) + (size_t)hk::KR * n_slots * hk::U_BYTES;
  const size_t n_chunks = ((size_t)seqlen + hk::KC - 1) / hk::KC;
  return (size_t)bsz * num_heads * n_chunks * hk::U_BYTES;
}

namespace hk {
namespace {
int chunked_prefill_launch(const void* mixed_qkv, const float* g_or_f, const void* beta_or_b, const float* dt_bias,
                           const float* a_log, float lower_bound, bool gated, float* state, void* out,
                           float* out_f32, int bsz, int seqlen, int num_heads, const int* slots,
                           void* workspace, size_t workspace_bytes, void* stream) {
  HK_REQUIRE(mixed_qkv && g_or_f && beta_or_b && state && out && workspace);
  HK_REQUIRE(!gated || (dt_bias && a_log && aligned(dt_bias, 16) && aligned(beta_or_b, 4)));
  HK_REQUIRE(bsz > 0 && seqlen > 0 && num_heads > 0);
  HK_REQUIRE(bsz <= 65535 && (seqlen + KC - 1) / KC <= 65535);   // grid limits
  HK_REQUIRE(aligned(mixed_qkv, 16) && aligned(g_or_f, 16) && aligned(state, 16) && aligned(out, 16) &&
             aligned(workspace, 256) && (!out_f32 || aligned(out_f32, 16)));
  if (workspace_bytes < hk_kda_chunked_workspace_bytes(bsz, seqlen, num_heads)) return HK_ERR_WORKSPACE;
  const int n_chunks = (seqlen + KC - 1) / KC;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(kda_chunk_prep_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P1_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(kda_chunk_prep_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P1_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(kda_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(kda_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(kda_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  cudaStream_t s = as_stream(stream);
  int* st = device_status_ptr();
  if (const int n_slots = fused_slots((long long)bsz * num_heads)) {
    // one cooperative launch: chain slots on the first n_slots CTAs, preparation workers on all others
    const int n_jobs = bsz * num_heads;
    const size_t flag_bytes = fused_flag_bytes(n_slots);
    if (cudaMemsetAsync(workspace, 0, flag_bytes, s) != cudaSuccess) return HK_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(512);
    cfg.dynamicSmemBytes = F_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const __nv_bfloat16* a_qkv = (const __nv_bfloat16*)mixed_qkv;
    uint8_t* a_ring = (uint8_t*)workspace + flag_bytes;
    int* a_flags = (int*)workspace;
    __nv_bfloat16* a_out = (__nv_bfloat16*)out;
    const float a_scale = 1.0f / sqrtf((float)KD);
    // tensor map over the output [bsz][seqlen][H][128] bf16 for the chain CTAs' tiled stores: box = 64 channels x 1 head x
    // 64 tokens x 1 sequence, 128-byte swizzle; without the encoder the kernel stores the rows itself
    alignas(64) CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    int use_tma_out = 0;
    {
      typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
      static EncodeFn encode = nullptr;
      static bool looked_up = false;
      if (!looked_up) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
          encode = (EncodeFn)fn;
        looked_up = true;
      }
      if (encode) {
        const cuuint64_t dims[4] = {(cuuint64_t)KD, (cuuint64_t)num_heads, (cuuint64_t)seqlen, (cuuint64_t)bsz};
        const cuuint64_t strides[3] = {(cuuint64_t)KD * 2, (cuuint64_t)num_heads * KD * 2, (cuuint64_t)seqlen * num_heads * KD * 2};
        const cuuint32_t box[4] = {64, 1, (cuuint32_t)KC, 1};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
          use_tma_out = 1;
      }
    }
    const float* a_dt = gated ? dt_bias : nullptr;
    const float* a_al = gated ? a_log : nullptr;
    const float a_lb = gated ? lower_bound : 0.f;
    cudaError_t e = gated
        ? cudaLaunchKernelEx(&cfg, kda_fused_kernel<true>, a_qkv, g_or_f, beta_or_b, a_ring, a_flags, state, a_out, out_f32,
                             seqlen, num_heads, n_chunks, n_jobs, n_slots, slots, a_scale, st, a_dt, a_al, a_lb, tmap, use_tma_out)
        : cudaLaunchKernelEx(&cfg, kda_fused_kernel<false>, a_qkv, g_or_f, beta_or_b, a_ring, a_flags, state, a_out, out_f32,
                             seqlen, num_heads, n_chunks, n_jobs, n_slots, slots, a_scale, st, a_dt, a_al, a_lb, tmap, use_tma_out);
    return e == cudaSuccess ? HK_OK : HK_ERR_CUDA;
  }
  const dim3 grid(num_heads, n_chunks, bsz);
  if (gated)
    kda_chunk_prep_kernel<true><<<grid, 256, P1_SMEM, s>>>((const __nv_bfloat16*)mixed_qkv, g_or_f, beta_or_b,
                                                         (uint8_t*)workspace, seqlen, num_heads, n_chunks,
                                                         2 * sm_count(), st, dt_bias, a_log, lower_bound);
  else
    kda_chunk_prep_kernel<false><<<grid, 256, P1_SMEM, s>>>((const __nv_bfloat16*)mixed_qkv, g_or_f, beta_or_b,
                                                          (uint8_t*)workspace, seqlen, num_heads, n_chunks,
                                                          2 * sm_count(), st, nullptr, nullptr, 0.f);
  HK_LAUNCH_CHECK();
  kda_chunk_scan_kernel<<<dim3(KVS, num_heads, bsz), 128, P2_SMEM, s>>>(
      (const uint8_t*)workspace, state, (__nv_bfloat16*)out, out_f32, seqlen, num_heads, n_chunks,
      slots, 1.0f / sqrtf((float)KD), st);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
}  // namespace
}  // namespace hk

HK_API int hk_kda_chunked_prefill(const void* mixed_qkv, const float* g, const void* beta,
                                  float* state, void* out, float* out_f32, int bsz, int seqlen,
                                  int num_heads, const int* slots, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  return hk::chunked_prefill_launch(mixed_qkv, g, beta, nullptr, nullptr, 0.f, false, state, out, out_f32, bsz,
                                    seqlen, num_heads, slots, workspace, workspace_bytes, stream);
}

HK_API int hk_kda_chunked_prefill_gated(const void* mixed_qkv, const float* f, const float* b,
                                        const float* dt_bias, const float* a_log, float lower_bound,
                                        float* state, void* out, float* out_f32, int bsz, int seqlen,
                                        int num_heads, const int* slots, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  return hk::chunked_prefill_launch(mixed_qkv, f, b, dt_bias, a_log, lower_bound, true, state, out, out_f32, bsz,
                                    seqlen, num_heads, slots, workspace, workspace_bytes, stream);
}
