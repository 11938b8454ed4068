// Absorbed MLA flash attention over the 512-wide fp16 latent cache on the 5th-generation tensor
// cores: dense causal ranges and gathered (sparse) rows, decode and prefill rows, final output or
// split-KV partials.  One kernel serves helios::attn::mla_sparse_decode and
// helios::attn::mla_dense_prefill (reference: src/cuda/attn/attn.cu:394-699, scalar kernels, one
// block per (row, head) or head pair).
//
// Work item = (query row, key split) -> one CTA; all 64 heads of the row share every latent row that
// is staged, so the cache is read once per row (the reference re-reads it per head pair).
// Per tile of 64 keys (64 KB, cp.async, double buffered, invalid slots zero-filled):
//   S  [64 heads x 64 keys]  = Q  K^T   tcgen05 M64  N64 K512: Q and the tile both K-major
//   softmax: heads are TMEM lanes, keys are columns -> max / exp2 / sum run inside one thread; the
//            running reference max only moves when a tile exceeds it by 2^8 (lazy rescale of O)
//   O^T[512 ch x 64 heads] += V^T P^T   4 x tcgen05 M128 N64 K64: the SAME tile read MN-major as A
//            (the latent row is both key and value), P written K-major by the head threads
// The no-swizzle core-matrix layout makes the two views of the tile coincide: 8 keys x 16 bytes of
// channels per core matrix, channel chunks 128 B apart, key groups 8 KB apart.
// HBM-bound by design: 1 KB per key for 128 K flops (128 flop/B), accumulators never leave TMEM.
#include <cuda_pipeline_primitives.h>

#include "mla_args.cuh"
#include "tc05.cuh"

namespace hk {

constexpr int FT_KEYS = 64;                       // keys per tile
constexpr int FT_HEADS = 64;
constexpr uint32_t FT_CS = 128;                   // channel-chunk stride inside a tile
constexpr uint32_t FT_KS = 64 * 128;              // key-group stride (64 channel chunks)
constexpr uint32_t FT_TILE = FT_KEYS * LATENT * 2;   // 65536
constexpr uint32_t FQ_LBO = 128, FQ_SBO = 64 * 128;  // Q operand [64 heads][512] K-major
constexpr uint32_t FP_LBO = 128, FP_SBO = 8 * 128;   // P operand [64 heads][64 keys] K-major
constexpr uint32_t FS_Q = 0;                      // 65536
constexpr uint32_t FS_K = 65536;                  // 2 x 65536
constexpr uint32_t FS_P = FS_K + 2 * FT_TILE;     // 8192
constexpr uint32_t FS_MISC = FS_P + 8192;         // alpha[64] f32, m[64], l[64], masks
constexpr uint32_t FS_SMEM = FS_MISC + 1024;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;         // log2 units: P stays below 2^8, fine for fp16

__global__ __launch_bounds__(128, 1) void mla_flash_tc_kernel(MlaArgs a, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem + FS_Q;
  uint8_t* sP = smem + FS_P;
  float* s_alpha = reinterpret_cast<float*>(smem + FS_MISC);
  float* s_m = s_alpha + 64;
  float* s_l = s_m + 64;
  unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(s_l + 64);  // [2]
  int* s_flag = reinterpret_cast<int*>(s_mask + 2);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sp = blockIdx.x, r = blockIdx.y;
  const bool sparse = a.raw_idx != nullptr;
  int n;
  int64_t base = 0;
  if (sparse) n = a.kidx;
  else {
    n = a.kv_len ? a.kv_len[r] : a.pos_start + r + 1;
    base = a.kv_base ? a.kv_base[r] : 0;
  }
  // split boundaries on tile granularity
  const int tiles_total = (n + FT_KEYS - 1) / FT_KEYS;
  const int tiles_per = (tiles_total + a.n_split - 1) / a.n_split;
  const int k0 = min(n, sp * tiles_per * FT_KEYS), k1 = min(n, (sp + 1) * tiles_per * FT_KEYS);
  const int n_tiles = (k1 - k0 + FT_KEYS - 1) / FT_KEYS;

  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
    *s_flag = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);

  // ---- Q: 64 heads x 64 chunks of 16 B, K-major operand; octet = 8 heads of one chunk ----
  {
    const __half* q = a.q_lat + (size_t)r * FT_HEADS * LATENT;
    for (int it = warp; it < 8 * 16; it += 4) {      // 8 head groups x 16 chunk quads
      const int hg = it >> 4, ch = (it & 15) * 4 + (lane >> 3), h = hg * 8 + (lane & 7);
      __pipeline_memcpy_async(sQ + hg * FQ_SBO + ch * FQ_LBO + (lane & 7) * 16, q + (size_t)h * LATENT + ch * 8, 16);
    }
  }
  // key tile loader: 8 key groups x 16 chunk quads per tile
  auto load_tile = [&](int tile, int buf) {
    uint8_t* dst0 = smem + FS_K + buf * FT_TILE;
    const int p0 = k0 + tile * FT_KEYS;
    for (int it = warp; it < 8 * 16; it += 4) {
      const int kg = it >> 4, ch = (it & 15) * 4 + (lane >> 3), key = kg * 8 + (lane & 7);
      const int p = p0 + key;
      int64_t tok = -1;
      if (p < k1) tok = sparse ? (int64_t)a.raw_idx[(size_t)r * a.kidx + p] : base + p;
      uint8_t* dst = dst0 + kg * FT_KS + ch * FT_CS + (lane & 7) * 16;
      if (tok >= 0) __pipeline_memcpy_async(dst, a.ckv + (size_t)tok * LATENT + ch * 8, 16);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    if (warp == 0) {
      // validity of the 64 key slots of this tile
      unsigned long long m = 0;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int p = p0 + half * 32 + lane;
        bool v = p < k1;
        if (v && sparse) v = a.raw_idx[(size_t)r * a.kidx + p] >= 0;
        m |= (unsigned long long)__ballot_sync(0xffffffffu, v) << (32 * half);
      }
      if (lane == 0) s_mask[buf] = m;
    }
  };
  if (n_tiles > 0) load_tile(0, 0);
  __pipeline_commit();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 64;   // S: 64 columns; O^T: 4 x 64 columns
  const uint32_t q_addr = tc::smem_u32(sQ), p_addr = tc::smem_u32(sP);
  const uint32_t idesc_s = tc::make_idesc(64, FT_KEYS, tc::FMT_F16, tc::FMT_F16, false, false);
  const uint32_t idesc_o = tc::make_idesc(128, FT_HEADS, tc::FMT_F16, tc::FMT_F16, true, false);
  const float sc2 = a.scale * LOG2E;
  const int head = warp * 16 + (lane & 15);   // rows of an M=64 accumulator sit in lanes 0-15 of each quarter
  const bool head_thread = lane < 16;
  float m_ref = -INFINITY, l_run = 0.f;
  uint32_t parity = 0;
  bool ok = true;

  for (int tile = 0; tile < n_tiles; tile++) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) load_tile(tile + 1, buf ^ 1);
    __pipeline_commit();
    __pipeline_wait_prior(1);
    tc::fence_async_smem();
    __syncthreads();
    const uint32_t k_addr = tc::smem_u32(smem + FS_K + buf * FT_TILE);
    // ---- S = Q K^T ----
    if (tid == 0) {
#pragma unroll 4
      for (int kk = 0; kk < LATENT / 16; kk++) {
        const uint64_t ad = tc::make_sdesc(q_addr + kk * 2 * FQ_LBO, FQ_LBO, FQ_SBO);
        const uint64_t bd = tc::make_sdesc(k_addr + kk * 2 * FT_CS, FT_CS, FT_KS);
        tc::mma_f16(tS, ad, bd, idesc_s, kk > 0);
      }
      tc::mma_commit(&bar);
    }
    ok = tc::mbar_wait(&bar, parity, &abort_flag, 1) && ok;
    parity ^= 1;
    tc::fence_after_sync();
    // ---- softmax of this tile: one thread per head ----
    {
      uint32_t s0[32], s1[32];
      tc::tmem_ld32(tS + ((uint32_t)(warp * 32) << 16), s0);
      tc::tmem_ld32(tS + ((uint32_t)(warp * 32) << 16) + 32, s1);
      tc::tmem_ld_wait();
      const unsigned long long mask = s_mask[buf];
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const float v0 = ((mask >> j) & 1ull) ? __uint_as_float(s0[j]) * sc2 : -INFINITY;
        const float v1 = ((mask >> (32 + j)) & 1ull) ? __uint_as_float(s1[j]) * sc2 : -INFINITY;
        s0[j] = __float_as_uint(v0);
        s1[j] = __float_as_uint(v1);
        tmax = fmaxf(tmax, fmaxf(v0, v1));
      }
      float alpha = 1.f;
      if (tmax > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && tmax > -INFINITY)) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - tmax);
        m_ref = tmax;
        l_run *= alpha;
        if (head_thread && tile > 0) *s_flag = 1;
      }
      if (head_thread) s_alpha[head] = alpha;
      float lsum = 0.f;
      uint8_t* prow = sP + (head >> 3) * FP_SBO + (head & 7) * 16;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        float p[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const int j = c * 8 + e;
          const float sv = __uint_as_float(j < 32 ? s0[j] : s1[j - 32]);
          p[e] = (m_ref == -INFINITY) ? 0.f : exp2f(sv - m_ref);
          lsum += p[e];
        }
        if (head_thread) {
          __half2 h0 = __floats2half2_rn(p[0], p[1]), h1 = __floats2half2_rn(p[2], p[3]);
          __half2 h2 = __floats2half2_rn(p[4], p[5]), h3 = __floats2half2_rn(p[6], p[7]);
          uint4 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
          *reinterpret_cast<uint4*>(prow + c * FP_LBO) = pk;
        }
      }
      l_run += lsum;
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    // ---- rare: a head's reference max moved, rescale the O^T accumulators (columns = heads) ----
    if (*s_flag) {
#pragma unroll 1
      for (int mt = 0; mt < 4; mt++) {
#pragma unroll 1
        for (int c0 = 0; c0 < FT_HEADS; c0 += 32) {
          uint32_t o[32];
          const uint32_t addr = tO + mt * 64 + c0 + ((uint32_t)(warp * 32) << 16);
          tc::tmem_ld32(addr, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * s_alpha[c0 + j]);
          tc::tmem_st32(addr, o);
        }
      }
      tc::tmem_st_wait();
      tc::fence_before_sync();
      __syncthreads();
      tc::fence_after_sync();
      if (tid == 0) *s_flag = 0;
    }
    // ---- O^T += V^T P^T ----
    if (tid == 0) {
#pragma unroll
      for (int mt = 0; mt < 4; mt++)
#pragma unroll
        for (int kk = 0; kk < FT_KEYS / 16; kk++) {
          const uint64_t ad = tc::make_sdesc(k_addr + mt * 16 * FT_CS + kk * 2 * FT_KS, FT_KS, FT_CS);
          const uint64_t bd = tc::make_sdesc(p_addr + kk * 2 * FP_LBO, FP_LBO, FP_SBO);
          tc::mma_f16(tO + mt * 64, ad, bd, idesc_o, tile > 0 || kk > 0);
        }
      tc::mma_commit(&bar);
    }
    ok = tc::mbar_wait(&bar, parity, &abort_flag, 2) && ok;
    parity ^= 1;
    tc::fence_after_sync();
  }
  __pipeline_wait_prior(0);

  // ---- epilogue ----
  if (head_thread) {
    s_m[head] = m_ref;
    s_l[head] = l_run;
  }
  __syncthreads();
  const size_t rows = (size_t)a.m * FT_HEADS;
  const size_t rh0 = (size_t)r * FT_HEADS;
  if (ok) {
#pragma unroll 1
    for (int mt = 0; mt < 4; mt++) {
      const int ch = mt * 128 + tid;   // TMEM lane = channel inside the M tile
#pragma unroll 1
      for (int c0 = 0; c0 < FT_HEADS; c0 += 32) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tc::tmem_ld32(tO + mt * 64 + c0 + ((uint32_t)(warp * 32) << 16), o);
          tc::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) o[j] = 0u;
        }
        if (a.out) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float l = s_l[c0 + j];
            const float v = l > 0.f ? __uint_as_float(o[j]) / l : 0.f;
            a.out[(rh0 + c0 + j) * LATENT + ch] = __float2half_rn(v);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++)
            a.part_acc[((size_t)sp * rows + rh0 + c0 + j) * LATENT + ch] = s_l[c0 + j] > 0.f ? __uint_as_float(o[j]) : 0.f;
        }
      }
    }
    if (!a.out && tid < FT_HEADS) {
      const float mr = s_m[tid];
      a.part_m[(size_t)sp * rows + rh0 + tid] = (mr == -INFINITY || !(s_l[tid] > 0.f)) ? -INFINITY : mr / LOG2E;
      a.part_l[(size_t)sp * rows + rh0 + tid] = s_l[tid];
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

int mla_flash_tc_auto_splits(int m, int n_keys) {
  // about one CTA per SM, at least two 64-key tiles per split, splits of equal tile counts
  const int sms = sm_count();
  const int tiles = (n_keys + FT_KEYS - 1) / FT_KEYS;
  int want = (sms + m - 1) / m;
  if (want > 256) want = 256;
  if (want < 1) want = 1;
  int tiles_per = (tiles + want - 1) / want;
  if (tiles_per < 2) tiles_per = 2;
  int n_split = (tiles + tiles_per - 1) / tiles_per;
  return n_split < 1 ? 1 : n_split;
}

int mla_flash_tc_launch(const MlaArgs& a, cudaStream_t s) {
  if (a.n_heads != FT_HEADS) return HK_ERR_UNSUPPORTED;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(mla_flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FS_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  dim3 grid(a.n_split, a.m);
  mla_flash_tc_kernel<<<grid, 128, FS_SMEM, s>>>(a, device_status_ptr());
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

}  // namespace hk
