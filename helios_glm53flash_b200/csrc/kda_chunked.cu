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
// bulk copies (double buffered) and issues three tcgen05 contractions with TMEM accumulators:
// [W;Q+] S0 (M128 N32 K128), [0;B beta] U (accumulated onto the Q+ S0 rows) and Kt^T U (M128 N32 K64).
#include <cuda_pipeline_primitives.h>

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

// =================================================================================================
// kernel 1: per-chunk preparation
// =================================================================================================
constexpr int P1_LD = 132;                               // padded fp32 row (conflict-free fragments)
constexpr int P1_LDA = 68;                               // padded row of the 64x64 matrices
constexpr uint32_t P1_G = 0;                             // f32 [64][132] cumulative log decay
constexpr uint32_t P1_K = P1_G + KC * P1_LD * 4;         // f32 [64][132] k^
constexpr uint32_t P1_LK = P1_K + KC * P1_LD * 4;        // tf32 [64][132] k^ e^{G_t - P_blk}
constexpr uint32_t P1_LQ = P1_LK + KC * P1_LD * 4;       // tf32 [64][132] q^ e^{G_t - P_blk}
constexpr uint32_t P1_A = P1_LQ + KC * P1_LD * 4;        // f32 [64][68]  A_ts beta_s (strictly lower)
constexpr uint32_t P1_B = P1_A + KC * P1_LDA * 4;        // f32 [64][68]  B_ts beta_s (lower incl.)
constexpr uint32_t P1_T = P1_B + KC * P1_LDA * 4;        // fp16 A operand [128 rows][64], 16 KB
constexpr uint32_t P1_KV = P1_T + 16384;                 // fp16 B operand [64 tokens][256], 32 KB
constexpr uint32_t P1_P = P1_KV + 32768;                 // f32 [4][128] G before each 16-token block
constexpr uint32_t P1_EP = P1_P + 2048;                  // f32 [4][128] exp of the above
constexpr uint32_t P1_BETA = P1_EP + 2048;               // f32 [64]
constexpr uint32_t P1_SMEM = P1_BETA + 256;

__global__ __launch_bounds__(256, 1) void kda_chunk_prep_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ g,
    const __nv_bfloat16* __restrict__ beta, uint8_t* __restrict__ ws, int seqlen, int H,
    int n_chunks, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  float* sG = reinterpret_cast<float*>(smem + P1_G);
  float* sK = reinterpret_cast<float*>(smem + P1_K);
  float* sLk = reinterpret_cast<float*>(smem + P1_LK);
  float* sLq = reinterpret_cast<float*>(smem + P1_LQ);
  float* sA = reinterpret_cast<float*>(smem + P1_A);
  float* sB = reinterpret_cast<float*>(smem + P1_B);
  uint8_t* sT = smem + P1_T;
  uint8_t* sKV = smem + P1_KV;
  float* sP = reinterpret_cast<float*>(smem + P1_P);
  float* sEP = reinterpret_cast<float*>(smem + P1_EP);
  float* sBeta = reinterpret_cast<float*>(smem + P1_BETA);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int t0 = chunk * KC;
  const int n_valid = min(KC, seqlen - t0);
  const size_t row = (size_t)3 * H * KD;
  const __nv_bfloat16* tok0 = qkv + ((size_t)b * seqlen + t0) * row;
  const float* g0 = g + (((size_t)b * seqlen + t0) * H + head) * KD;
  uint8_t* unit = ws + (((size_t)b * H + head) * n_chunks + chunk) * U_BYTES;

  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 256);

  // ---- stage 1: load a token per warp-iteration; lane owns channels 4*lane .. 4*lane+3 ----
  for (int t = warp; t < KC; t += 8) {
    float kf[4] = {0.f, 0.f, 0.f, 0.f}, qf[4] = {0.f, 0.f, 0.f, 0.f}, vf[4] = {0.f, 0.f, 0.f, 0.f};
    float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < n_valid) {
      const __nv_bfloat16* tk = tok0 + (size_t)t * row;
      const uint2 qr = *reinterpret_cast<const uint2*>(tk + (size_t)head * KD + lane * 4);
      const uint2 kr = *reinterpret_cast<const uint2*>(tk + (size_t)(H + head) * KD + lane * 4);
      const uint2 vr = *reinterpret_cast<const uint2*>(tk + (size_t)(2 * H + head) * KD + lane * 4);
      qf[0] = bf16lo(qr.x); qf[1] = bf16hi(qr.x); qf[2] = bf16lo(qr.y); qf[3] = bf16hi(qr.y);
      kf[0] = bf16lo(kr.x); kf[1] = bf16hi(kr.x); kf[2] = bf16lo(kr.y); kf[3] = bf16hi(kr.y);
      vf[0] = bf16lo(vr.x); vf[1] = bf16hi(vr.x); vf[2] = bf16lo(vr.y); vf[3] = bf16hi(vr.y);
      gv = *reinterpret_cast<const float4*>(g0 + (size_t)t * H * KD + lane * 4);
    }
    const float sq = warp_sum(qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3]);
    const float sk = warp_sum(kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3]);
    const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
    *reinterpret_cast<float4*>(sK + t * P1_LD + lane * 4) = make_float4(kf[0] * rk, kf[1] * rk, kf[2] * rk, kf[3] * rk);
    *reinterpret_cast<float4*>(sLq + t * P1_LD + lane * 4) = make_float4(qf[0] * rq, qf[1] * rq, qf[2] * rq, qf[3] * rq);
    *reinterpret_cast<float4*>(sG + t * P1_LD + lane * 4) = gv;
    // V -> B operand columns 128..255 (MN-major: off = (n/8)*1024 + (t/8)*128 + (t%8)*16 + (n%8)*2)
    const int n = KD + lane * 4;
    uint2 pv;
    pv.x = pack_h2(vf[0], vf[1]);
    pv.y = pack_h2(vf[2], vf[3]);
    *reinterpret_cast<uint2*>(sKV + (n >> 3) * 1024 + (t >> 3) * 128 + (t & 7) * 16 + (n & 7) * 2) = pv;
  }
  if (tid < KC) sBeta[tid] = tid < n_valid ? __bfloat162float(beta[((size_t)b * seqlen + t0 + tid) * H + head]) : 0.f;
  for (int i = tid; i < KC * P1_LDA; i += 256) {
    sA[i] = 0.f;
    sB[i] = 0.f;
  }
  // rows 64..127 of the T operand are never produced: keep them zero so the unused TMEM lanes stay finite
  for (int i = tid; i < 8192 / 16; i += 256) reinterpret_cast<uint4*>(sT + 8192)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  // ---- stage 2: inclusive cumulative log decay per channel; block bases P and e^P; chunk decay ----
  if (tid < KD) {
    float acc = 0.f;
#pragma unroll 4
    for (int t = 0; t < KC; t++) {
      if ((t & 15) == 0) {
        sP[(t >> 4) * KD + tid] = acc;
        sEP[(t >> 4) * KD + tid] = __expf(acc);
      }
      acc += sG[t * P1_LD + tid];
      sG[t * P1_LD + tid] = acc;
    }
    reinterpret_cast<float*>(unit + U_DEC)[tid] = __expf(acc);
  }
  __syncthreads();

  // ---- stage 3: left operands (tf32) with the exponent re-based to the start of the row's block;
  //      K+ into the B operand, Q+ and Kt^T straight to the workspace ----
  for (int i = tid; i < KC * (KD / 8); i += 256) {
    const int t = i >> 4, cc = i & 15, c0 = cc * 8, blk = t >> 4;
    float kp[8], qp[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int c = c0 + u;
      const float f = __expf(sG[t * P1_LD + c] - sP[blk * KD + c]);
      const float lk = sK[t * P1_LD + c] * f, lq = sLq[t * P1_LD + c] * f;
      sLk[t * P1_LD + c] = __uint_as_float(f2tf32(lk));
      sLq[t * P1_LD + c] = __uint_as_float(f2tf32(lq));
      const float ep = sEP[blk * KD + c];
      kp[u] = lk * ep;
      qp[u] = lq * ep;
    }
    uint4 pk, pq;
    pk.x = pack_h2(kp[0], kp[1]); pk.y = pack_h2(kp[2], kp[3]); pk.z = pack_h2(kp[4], kp[5]); pk.w = pack_h2(kp[6], kp[7]);
    pq.x = pack_h2(qp[0], qp[1]); pq.y = pack_h2(qp[2], qp[3]); pq.z = pack_h2(qp[4], qp[5]); pq.w = pack_h2(qp[6], qp[7]);
    *reinterpret_cast<uint4*>(sKV + cc * 1024 + (t >> 3) * 128 + (t & 7) * 16) = pk;
    *reinterpret_cast<uint4*>(unit + U_WQ + ((64 + t) >> 3) * SBO_K128 + cc * LBO + (t & 7) * 16) = pq;
  }
  for (int i = tid; i < KD * (KC / 8); i += 256) {
    const int c = i & 127, tg = i >> 7;
    const float glast = sG[(KC - 1) * P1_LD + c];
    float kt[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int t = tg * 8 + u;
      kt[u] = sBeta[t] * sK[t * P1_LD + c] * __expf(glast - sG[t * P1_LD + c]);
    }
    uint4 p;
    p.x = pack_h2(kt[0], kt[1]); p.y = pack_h2(kt[2], kt[3]); p.z = pack_h2(kt[4], kt[5]); p.w = pack_h2(kt[6], kt[7]);
    *reinterpret_cast<uint4*>(unit + U_KT + (c >> 3) * SBO_K64 + tg * LBO + (c & 7) * 16) = p;
  }
  __syncthreads();

  // ---- stage 4: A and B on the warp-level tensor cores (TF32), one (row block, column block) pair
  //      of 16x16 per warp-iteration; right operand k^_s e^{P_rowblk - G_s} is formed on the fly ----
  {
    const int gq = lane >> 2, tig = lane & 3;
    for (int pair = warp; pair < 10; pair += 8) {
      // pairs ordered by decreasing work locality: (3,3)(3,2)(3,1)(3,0)(2,2)(2,1)(2,0)(1,1)(1,0)(0,0)
      int ib, jb;
      if (pair < 4) { ib = 3; jb = 3 - pair; }
      else if (pair < 7) { ib = 2; jb = 6 - pair; }
      else if (pair < 9) { ib = 1; jb = 8 - pair; }
      else { ib = 0; jb = 0; }
      float acc[2][2][4];
#pragma unroll
      for (int x = 0; x < 2; x++)
#pragma unroll
        for (int y = 0; y < 2; y++)
#pragma unroll
          for (int z = 0; z < 4; z++) acc[x][y][z] = 0.f;
      const float* lk0 = sLk + (ib * 16 + gq) * P1_LD;
      const float* lq0 = sLq + (ib * 16 + gq) * P1_LD;
      const float* pb = sP + ib * KD;
#pragma unroll 2
      for (int ks = 0; ks < KD / 8; ks++) {
        const int c = ks * 8 + tig;
        uint32_t ak[4], aq[4];
        ak[0] = __float_as_uint(lk0[c]); ak[1] = __float_as_uint(lk0[8 * P1_LD + c]);
        ak[2] = __float_as_uint(lk0[c + 4]); ak[3] = __float_as_uint(lk0[8 * P1_LD + c + 4]);
        aq[0] = __float_as_uint(lq0[c]); aq[1] = __float_as_uint(lq0[8 * P1_LD + c]);
        aq[2] = __float_as_uint(lq0[c + 4]); aq[3] = __float_as_uint(lq0[8 * P1_LD + c + 4]);
        const float p0 = pb[c], p1 = pb[c + 4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const int s = jb * 16 + nt * 8 + gq;
          const uint32_t b0 = f2tf32(sK[s * P1_LD + c] * __expf(p0 - sG[s * P1_LD + c]));
          const uint32_t b1 = f2tf32(sK[s * P1_LD + c + 4] * __expf(p1 - sG[s * P1_LD + c + 4]));
          mma_tf32(acc[0][nt], ak, b0, b1);
          mma_tf32(acc[1][nt], aq, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int z = 0; z < 4; z++) {
          const int t = ib * 16 + gq + ((z & 2) ? 8 : 0);
          const int s = jb * 16 + nt * 8 + tig * 2 + (z & 1);
          const float bs = sBeta[s];
          if (s < t) sA[t * P1_LDA + s] = acc[0][nt][z] * bs;
          if (s <= t) sB[t * P1_LDA + s] = acc[1][nt][z] * bs;
        }
    }
  }
  __syncthreads();

  // ---- stage 5: warps 0-1 invert (I + A beta) by forward substitution, one column per thread, fp32;
  //      the other warps ship B beta to the workspace meanwhile ----
  if (tid < KC) {
    const int j = tid;
    float x[KC];
#pragma unroll
    for (int t = 0; t < KC; t++) {
      float a0 = (t == j) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float4* nrow = reinterpret_cast<const float4*>(sA + t * P1_LDA);
#pragma unroll
      for (int s4 = 0; s4 < (t + 3) / 4; s4++) {
        const float4 nv = nrow[s4];
        if (s4 * 4 + 0 < t) a0 = fmaf(-nv.x, x[s4 * 4 + 0], a0);
        if (s4 * 4 + 1 < t) a1 = fmaf(-nv.y, x[s4 * 4 + 1], a1);
        if (s4 * 4 + 2 < t) a2 = fmaf(-nv.z, x[s4 * 4 + 2], a2);
        if (s4 * 4 + 3 < t) a3 = fmaf(-nv.w, x[s4 * 4 + 3], a3);
      }
      x[t] = (a0 + a1) + (a2 + a3);
    }
    // T[t][j] into the A operand (K-major, K = 64): off = (t/8)*1024 + (j/8)*128 + (t%8)*16 + (j%8)*2
    __half* tcol = reinterpret_cast<__half*>(sT + (j >> 3) * LBO + (j & 7) * 2);
#pragma unroll
    for (int t = 0; t < KC; t++) tcol[((t >> 3) * SBO_K64 + (t & 7) * 16) / 2] = __float2half_rn(x[t]);
  } else {
    for (int i = tid - KC; i < KC * (KC / 8); i += 256 - KC) {
      const int t = i >> 3, sc = i & 7;
      const float4 v0 = *reinterpret_cast<const float4*>(sB + t * P1_LDA + sc * 8);
      const float4 v1 = *reinterpret_cast<const float4*>(sB + t * P1_LDA + sc * 8 + 4);
      uint4 p;
      p.x = pack_h2(v0.x, v0.y); p.y = pack_h2(v0.z, v0.w); p.z = pack_h2(v1.x, v1.y); p.w = pack_h2(v1.z, v1.w);
      *reinterpret_cast<uint4*>(unit + U_BB + (t >> 3) * SBO_K64 + sc * LBO + (t & 7) * 16) = p;
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();

  // ---- stage 6: [W | Uloc] = T [K+ | V] : tcgen05 M128 N256 K64, fp16 in, fp32 TMEM accumulators ----
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const uint32_t idesc = tc::make_idesc(128, 256, tc::FMT_F16, tc::FMT_F16, false, true);
    const uint32_t a_addr = tc::smem_u32(sT), b_addr = tc::smem_u32(sKV);
#pragma unroll
    for (int kk = 0; kk < KC / 16; kk++) {
      const uint64_t ad = tc::make_sdesc(a_addr + kk * 2 * LBO, LBO, SBO_K64);
      const uint64_t bd = tc::make_sdesc(b_addr + kk * 2 * 128, 128, 1024);
      tc::mma_f16(tmem, ad, bd, idesc, kk > 0);
    }
    tc::mma_commit(&bar);
  }
  const bool ok = tc::mbar_wait(&bar, 0, &abort_flag, 1);
  tc::fence_after_sync();
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
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 256);
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
constexpr uint32_t P2_S = 2 * S_STAGE;    // fp16 B operand: state slice [128 k][32], MN-major, 8 KB
constexpr uint32_t P2_U = P2_S + 8192;    // fp16 B operand: U [64 tokens][32], MN-major, 4 KB
constexpr uint32_t P2_SMEM = P2_U + 4096;

__global__ __launch_bounds__(128, 1) void kda_chunk_scan_kernel(
    const uint8_t* __restrict__ ws, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
    float* __restrict__ out_f32, int seqlen, int H, int n_chunks, const int* __restrict__ slots,
    float scale, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[2];
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vs = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int v0 = vs * KNV;
  const uint8_t* unit0 = ws + (((size_t)b * H + head) * n_chunks) * U_BYTES;
  const int slot = slots ? slots[b] : b;
  float* st = state + ((size_t)slot * H + head) * KD * KD + (size_t)tid * KD + v0;  // row k = tid

  if (tid == 0) {
    tc::mbar_init(&full_bar[0], 1);
    tc::mbar_init(&full_bar[1], 1);
    tc::mbar_init(&mma_bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 64);
  // zero halves of the [0 ; B beta] operands
  for (int i = tid; i < 8192 / 16; i += 128) {
    reinterpret_cast<uint4*>(smem + S_BB)[i] = make_uint4(0, 0, 0, 0);
    reinterpret_cast<uint4*>(smem + S_STAGE + S_BB)[i] = make_uint4(0, 0, 0, 0);
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
  const uint32_t d1 = tmem, d2 = tmem + 32;

  auto issue_loads = [&](int chunk) {
    uint8_t* stg = smem + (chunk & 1) * S_STAGE;
    const uint8_t* u = unit0 + (size_t)chunk * U_BYTES;
    uint64_t* bar = &full_bar[chunk & 1];
    tc::mbar_arrive_expect_tx(bar, S_TX);
    tc::bulk_g2s(stg + S_WQ, u + U_WQ, 32768, bar);
    tc::bulk_g2s(stg + S_BB + 8192, u + U_BB, 8192, bar);
    tc::bulk_g2s(stg + S_KT, u + U_KT, 16384, bar);
    tc::bulk_g2s(stg + S_UL, u + U_UL + vs * (KC * KNV * 2), 4096, bar);
    tc::bulk_g2s(stg + S_DEC, u + U_DEC, 512, bar);
  };
  if (tid == 0) {
    issue_loads(0);
    if (n_chunks > 1) issue_loads(1);
  }

  const uint32_t idesc = tc::make_idesc(128, KNV, tc::FMT_F16, tc::FMT_F16, false, true);
  const uint32_t s_addr = tc::smem_u32(smem + P2_S), u_addr = tc::smem_u32(smem + P2_U);
  uint32_t mma_parity = 0;

  for (int chunk = 0; chunk < n_chunks; chunk++) {
    const int sidx = chunk & 1;
    uint8_t* stg = smem + sidx * S_STAGE;
    const uint32_t stg_addr = tc::smem_u32(stg);
    bool ok = tc::mbar_wait(&full_bar[sidx], (chunk >> 1) & 1, &abort_flag, 2);
    // ---- [W ; Q+] S0 -> D1 (128 x 32) ----
    if (tid == 0) {
#pragma unroll
      for (int kk = 0; kk < KD / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_WQ + kk * 2 * LBO, LBO, SBO_K128);
        const uint64_t bd = tc::make_sdesc(s_addr + kk * 2 * 128, 128, 2048);
        tc::mma_f16(d1, ad, bd, idesc, kk > 0);
      }
      tc::mma_commit(&mma_bar);
    }
    ok = tc::mbar_wait(&mma_bar, mma_parity, &abort_flag, 3) && ok;
    mma_parity ^= 1;
    tc::fence_after_sync();
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
    // ---- D1 rows 64-127 += (B beta) U ;  D2 = Kt^T U ----
    if (tid == 0) {
#pragma unroll
      for (int kk = 0; kk < KC / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_BB + kk * 2 * LBO, LBO, SBO_K64);
        const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
        tc::mma_f16(d1, ad, bd, idesc, true);
      }
#pragma unroll
      for (int kk = 0; kk < KC / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(stg_addr + S_KT + kk * 2 * LBO, LBO, SBO_K64);
        const uint64_t bd = tc::make_sdesc(u_addr + kk * 2 * 128, 128, 1024);
        tc::mma_f16(d2, ad, bd, idesc, kk > 0);
      }
      tc::mma_commit(&mma_bar);
    }
    ok = tc::mbar_wait(&mma_bar, mma_parity, &abort_flag, 4) && ok;
    mma_parity ^= 1;
    tc::fence_after_sync();
    // ---- outputs (TMEM lanes 64-127 = tokens) ----
    if (warp >= 2) {
      const int t = tid - 64;
      const int tok = chunk * KC + t;
      uint32_t r[32];
      tc::tmem_ld32(d1 + ((uint32_t)(warp * 32) << 16), r);
      tc::tmem_ld_wait();
      if (tok < seqlen && ok) {
        const size_t oi = (((size_t)b * seqlen + tok) * H + head) * KD + v0;
        uint4* o = reinterpret_cast<uint4*>(out + oi);
#pragma unroll
        for (int u = 0; u < 4; u++) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float a = __uint_as_float(r[8 * u + 2 * e]) * scale, c = __uint_as_float(r[8 * u + 2 * e + 1]) * scale;
            const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rz(a));
            const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rz(c));
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
    }
    // ---- state: S <- S e^{G_last} + Kt^T U (lane = k row), refresh the fp16 operand copy ----
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
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    if (tid == 0 && chunk + 2 < n_chunks) issue_loads(chunk + 2);
  }
  if (!abort_flag) {
#pragma unroll
    for (int u = 0; u < KNV / 4; u++)
      *reinterpret_cast<float4*>(st + u * 4) = make_float4(S[4 * u], S[4 * u + 1], S[4 * u + 2], S[4 * u + 3]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 64);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

}  // namespace hk

HK_API size_t hk_kda_chunked_workspace_bytes(int bsz, int seqlen, int num_heads) {
  if (bsz <= 0 || seqlen <= 0 || num_heads <= 0) return 0;
  const size_t n_chunks = ((size_t)seqlen + hk::KC - 1) / hk::KC;
  return (size_t)bsz * num_heads * n_chunks * hk::U_BYTES;
}

HK_API int hk_kda_chunked_prefill(const void* mixed_qkv, const float* g, const void* beta,
                                  float* state, void* out, float* out_f32, int bsz, int seqlen,
                                  int num_heads, const int* slots, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  using namespace hk;
  HK_REQUIRE(mixed_qkv && g && beta && state && out && workspace);
  HK_REQUIRE(bsz > 0 && seqlen > 0 && num_heads > 0);
  HK_REQUIRE(aligned(mixed_qkv, 8) && aligned(g, 16) && aligned(state, 16) && aligned(out, 16) &&
             aligned(workspace, 256) && (!out_f32 || aligned(out_f32, 16)));
  if (workspace_bytes < hk_kda_chunked_workspace_bytes(bsz, seqlen, num_heads)) return HK_ERR_WORKSPACE;
  const int n_chunks = (seqlen + KC - 1) / KC;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(kda_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P1_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(kda_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  cudaStream_t s = as_stream(stream);
  int* st = device_status_ptr();
  kda_chunk_prep_kernel<<<dim3(n_chunks, num_heads, bsz), 256, P1_SMEM, s>>>(
      (const __nv_bfloat16*)mixed_qkv, g, (const __nv_bfloat16*)beta, (uint8_t*)workspace, seqlen,
      num_heads, n_chunks, st);
  HK_LAUNCH_CHECK();
  kda_chunk_scan_kernel<<<dim3(KVS, num_heads, bsz), 128, P2_SMEM, s>>>(
      (const uint8_t*)workspace, state, (__nv_bfloat16*)out, out_f32, seqlen, num_heads, n_chunks,
      slots, 1.0f / sqrtf((float)KD), st);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
