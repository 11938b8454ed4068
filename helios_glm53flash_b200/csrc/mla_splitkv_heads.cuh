// Split-KV MLA decode across the GPUs of one node, combine sharded by heads.
//
// Every rank attends its slice of the latent cache for all 64 heads (flash kernel, local splits over the
// SMs).  What follows the flash kernel is three small kernels per step and rank:
//   merge + signal   the local splits of every (row, head) are merged into ONE (m, l, acc) set in this rank's
//                    exchange region; the last CTA to finish (atomic ticket) stores the step's epoch into slot
//                    `rank` of every rank's "partial ready" flags (system-scope release stores over NVLink);
//   combine by heads rank g owns heads [g*64/G, (g+1)*64/G): it waits (bounded) for all G ready flags, reads
//                    ONLY its heads from the G partial sets (plain peer loads, all in flight at once), normalises
//                    and stores the fp16 rows into EVERY rank's output buffer in its region (peer stores); the
//                    last CTA then publishes "output slice written" to every rank;
//   gather           waits (bounded) for the G "slice written" flags and copies the region's output buffer to
//                    the caller's tensor; its last CTA advances the device-side step counter.
// Per rank and step m*64/G*(G*2056) B are read and m*64*1024 B written across NVLink, whatever G is (the
// all-read-all form reads G times as much).  The reference has no multi-GPU path; the merge arithmetic is its
// in-kernel warp merge (src/cuda/attn/attn.cu:462-481).
//
// Exchange sets and output buffers are double buffered by step parity.  A wait that expires makes the whole grid
// skip its writes (one decision per grid, taken through a word in the region), sets HK_ERR_TIMEOUT in the device
// status word and lets the step finish; after a timeout the group has to be re-synchronised on the host
// (hk_splitkv_region_reset on every rank between two host barriers) before the next step.
//
// Only plain loads and stores touch peer memory: no TMA, no multicast.
// Included at the end of mla_attend.cu (one translation unit with the combine helpers of mla_simt.cuh).
#pragma once

namespace hk {

namespace {

constexpr int SK_MAX_RANKS = 32;
// region header (ints): [0] step counter, [1] merge ticket, [2] combine ticket, [3] gather ticket,
// [4] combine decision, [5] gather decision; [64..96) partial-ready flags; [128..160) slice-written flags
constexpr int SK_STEP = 0, SK_T_MERGE = 1, SK_T_COMB = 2, SK_T_GATHER = 3, SK_D_COMB = 4, SK_D_GATHER = 5;
constexpr int SK_F_READY = 64, SK_F_DONE = 128;
constexpr size_t SK_HEADER = 1024;

struct SkLayout {
  size_t set_bytes, off_set[2], off_out[2], total, off_l, off_acc;
};
__host__ __device__ inline size_t sk_up(size_t v) { return (v + 255) / 256 * 256; }
__host__ __device__ inline SkLayout sk_layout(int64_t rows) {
  SkLayout L;
  const size_t ml = sk_up((size_t)rows * 4);
  L.off_l = ml;
  L.off_acc = 2 * ml;
  L.set_bytes = 2 * ml + (size_t)rows * LATENT * 4;
  L.off_set[0] = SK_HEADER;
  L.off_set[1] = SK_HEADER + L.set_bytes;
  L.off_out[0] = SK_HEADER + 2 * L.set_bytes;
  L.off_out[1] = L.off_out[0] + sk_up((size_t)rows * LATENT * 2);
  L.total = L.off_out[1] + sk_up((size_t)rows * LATENT * 2);
  return L;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One decision per grid: every CTA's thread 0 calls this; the first to see all `n` flags at `epoch` (or to run out
// of time) records +epoch (or -epoch) in *decision with a compare-and-swap and everybody follows that record.
__device__ bool sk_wait_all(const int* flags, int n, int epoch, int* decision, long long max_wait_cycles,
                            int* status) {
  const long long t0 = clock64();
  for (;;) {
    const int d = ld_volatile(decision);
    if (d == epoch) return true;
    if (d == -epoch) return false;
    bool all = true;
    for (int s = 0; s < n; s++)
      if (ld_acquire_sys(flags + s) < epoch) { all = false; break; }
    if (all) {
      atomicCAS(decision, d, epoch);
    } else if (clock64() - t0 > max_wait_cycles) {
      if (atomicCAS(decision, d, -epoch) == d && status) atomicExch(status, HK_ERR_TIMEOUT);
    } else {
      __nanosleep(100);
    }
  }
}

// merge of this rank's local splits into its exchange set of the step's parity, then the ready signal
__global__ __launch_bounds__(LSE_THREADS) void sk_merge_signal_kernel(
    const float* __restrict__ part_m, const float* __restrict__ part_l, const float* __restrict__ part_acc,
    int n_split, int64_t rows, uint8_t* const* __restrict__ regions, int n_ranks, int my_rank, int do_store) {
  uint8_t* mine = regions[my_rank];
  int* hdr = reinterpret_cast<int*>(mine);
  const int epoch = ld_volatile(hdr + SK_STEP) + 1;
  const SkLayout L = sk_layout(rows);
  uint8_t* set = mine + L.off_set[epoch & 1];
  const int64_t r = blockIdx.x;
  float gm, gl;
  float4 o;
  lse_reduce_row<false, LSE_GROUPS>(part_m, part_l, part_acc, nullptr, nullptr, nullptr, n_split, rows, r, gm, gl, o);
  if (threadIdx.x < 128)
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(set + L.off_acc) + (size_t)r * LATENT + threadIdx.x * 4) = o;
  if (threadIdx.x == 0) {
    reinterpret_cast<float*>(set)[r] = gm;
    reinterpret_cast<float*>(set + L.off_l)[r] = gl;
  }
  // the block barrier orders every thread's writes before thread 0's fence, which is cumulative over them
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int ticket = atomicAdd(hdr + SK_T_MERGE, 1);
    if (ticket == (int)rows - 1) {
      hdr[SK_T_MERGE] = 0;
      __threadfence_system();
      if (do_store)
        for (int s = 0; s < n_ranks; s++)
          st_release_sys(reinterpret_cast<int*>(regions[s]) + SK_F_READY + my_rank, epoch);
    }
  }
}

// grid = m * heads_per_rank CTAs of 128 threads: (row, head) pairs of THIS rank's head range
__global__ __launch_bounds__(128) void sk_combine_heads_kernel(
    uint8_t* const* __restrict__ regions, int n_ranks, int my_rank, int n_heads, int64_t rows,
    long long max_wait_cycles, int* __restrict__ status) {
  __shared__ int go;
  uint8_t* mine = regions[my_rank];
  int* hdr = reinterpret_cast<int*>(mine);
  const int epoch = ld_volatile(hdr + SK_STEP) + 1;
  const int par = epoch & 1;
  if (threadIdx.x == 0) go = sk_wait_all(hdr + SK_F_READY, n_ranks, epoch, hdr + SK_D_COMB, max_wait_cycles, status) ? 1 : 0;
  __syncthreads();
  const SkLayout L = sk_layout(rows);
  if (go) {
    const int hpr = n_heads / n_ranks;
    const int64_t r = (int64_t)(blockIdx.x / hpr) * n_heads + my_rank * hpr + blockIdx.x % hpr;
    const int t = threadIdx.x;
    float gm = -INFINITY, gl = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    // batches of 8 ranks: every load of a batch is issued before the first one is used (one NVLink round trip)
    for (int s0 = 0; s0 < n_ranks; s0 += 8) {
      float ms[8], ls[8];
      float4 as[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int s = s0 + u;
        if (s < n_ranks) {
          const uint8_t* set = regions[s] + L.off_set[par];
          ms[u] = __ldcv(reinterpret_cast<const float*>(set) + r);
          ls[u] = __ldcv(reinterpret_cast<const float*>(set + L.off_l) + r);
          as[u] = __ldcv(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(set + L.off_acc) + (size_t)r * LATENT) + t);
        } else {
          ms[u] = -INFINITY; ls[u] = 0.f; as[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float bm = gm;
#pragma unroll
      for (int u = 0; u < 8; u++) bm = fmaxf(bm, ms[u]);
      if (bm != -INFINITY) {
        const float resc = gm == -INFINITY ? 0.f : __expf(gm - bm);
        gl *= resc; o.x *= resc; o.y *= resc; o.z *= resc; o.w *= resc;
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const float w = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - bm);
          gl = fmaf(w, ls[u], gl);
          o.x = fmaf(w, as[u].x, o.x); o.y = fmaf(w, as[u].y, o.y); o.z = fmaf(w, as[u].z, o.z); o.w = fmaf(w, as[u].w, o.w);
        }
        gm = bm;
      }
    }
    const float inv = gl > 0.f ? 1.f / gl : 0.f;
    __half2 h0 = __floats2half2_rn(o.x * inv, o.y * inv);
    __half2 h1 = __floats2half2_rn(o.z * inv, o.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    for (int d = 0; d < n_ranks; d++)
      *reinterpret_cast<uint2*>(regions[d] + L.off_out[par] + ((size_t)r * LATENT + t * 4) * 2) = pk;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int ticket = atomicAdd(hdr + SK_T_COMB, 1);
    if (ticket == (int)gridDim.x - 1) {
      hdr[SK_T_COMB] = 0;
      __threadfence_system();
      if (go)
        for (int s = 0; s < n_ranks; s++)
          st_release_sys(reinterpret_cast<int*>(regions[s]) + SK_F_DONE + my_rank, epoch);
    }
  }
}

// copies this rank's output buffer of the step to the caller's tensor once every rank has written its slice
__global__ __launch_bounds__(128) void sk_gather_kernel(uint8_t* __restrict__ mine, int n_ranks, int64_t rows,
                                                        __half* __restrict__ out, long long max_wait_cycles,
                                                        int* __restrict__ status) {
  __shared__ int go;
  int* hdr = reinterpret_cast<int*>(mine);
  const int epoch = ld_volatile(hdr + SK_STEP) + 1;
  if (threadIdx.x == 0) go = sk_wait_all(hdr + SK_F_DONE, n_ranks, epoch, hdr + SK_D_GATHER, max_wait_cycles, status) ? 1 : 0;
  __syncthreads();
  if (go) {
    const SkLayout L = sk_layout(rows);
    const uint4* src = reinterpret_cast<const uint4*>(mine + L.off_out[epoch & 1]);
    uint4* dst = reinterpret_cast<uint4*>(out);
    const size_t n16 = (size_t)rows * LATENT * 2 / 16;
    for (size_t i = (size_t)blockIdx.x * 128 + threadIdx.x; i < n16; i += (size_t)gridDim.x * 128) dst[i] = __ldcv(src + i);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(hdr + SK_T_GATHER, 1);
    if (ticket == (int)gridDim.x - 1) {
      hdr[SK_T_GATHER] = 0;
      __threadfence();
      hdr[SK_STEP] = epoch;                               // every CTA of this step has read the counter
    }
  }
}

}  // namespace
}  // namespace hk

HK_API size_t hk_splitkv_region_bytes(int m, int n_heads) {
  if (m <= 0 || n_heads <= 0) return 0;
  return hk::sk_layout((int64_t)m * n_heads).total;
}

HK_API int hk_splitkv_region_reset(void* region, int m, int n_heads, void* stream) {
  using namespace hk;
  HK_REQUIRE(region && m > 0 && n_heads > 0);
  return cudaMemsetAsync(region, 0, SK_HEADER, as_stream(stream)) == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

HK_API int hk_mla_splitkv_heads_step(const void* q_lat, const void* ckv_shard, const int64_t* kv_base, const int* kv_len,
                                     int m, int n_heads, float scale, int n_split, int n_keys_hint, void* workspace,
                                     size_t workspace_bytes, void* const* region_ptrs, int n_ranks, int my_rank,
                                     void* my_region, void* out_f16, int max_wait_ms, int signal, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv_shard && region_ptrs && my_region && out_f16 && workspace);
  HK_REQUIRE(m > 0 && n_heads == 64 && n_ranks >= 1 && n_ranks <= SK_MAX_RANKS && n_heads % n_ranks == 0);
  HK_REQUIRE(my_rank >= 0 && my_rank < n_ranks && max_wait_ms > 0 && max_wait_ms <= 10000);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv_shard, 16) && aligned(my_region, 256) && aligned(workspace, 256) &&
             aligned(out_f16, 16));
  if (n_split <= 0) n_split = mla_flash_tc_auto_splits(m, n_keys_hint > 0 ? n_keys_hint : 4096);
  if (n_split > LSE_MAX_SPLITS) return HK_ERR_UNSUPPORTED;
  const int64_t rows = (int64_t)m * n_heads;
  const size_t ml = (((size_t)n_split * rows * sizeof(float)) + 255) / 256 * 256;
  const size_t need = 2 * ml + (size_t)n_split * rows * LATENT * sizeof(float);
  if (workspace_bytes < need) return HK_ERR_WORKSPACE;
  char* ws = (char*)workspace;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv_shard;
  a.kv_base = kv_base; a.kv_len = kv_len; a.pos_start = 0;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  a.n_split = n_split;
  a.part_m = (float*)ws; a.part_l = (float*)(ws + ml); a.part_acc = (float*)(ws + 2 * ml);
  cudaStream_t s = as_stream(stream);
  const int st = mla_flash_tc_launch(a, s);
  if (st != HK_OK) return st;
  const long long cycles = (long long)max_wait_ms * 2000000LL;   // ~2 GHz
  uint8_t* const* regions = (uint8_t* const*)region_ptrs;
  sk_merge_signal_kernel<<<(unsigned)rows, LSE_THREADS, 0, s>>>(a.part_m, a.part_l, a.part_acc, n_split, rows, regions, n_ranks,
                                                                my_rank, signal);
  HK_LAUNCH_CHECK();
  sk_combine_heads_kernel<<<(unsigned)(m * (n_heads / n_ranks)), 128, 0, s>>>(regions, n_ranks, my_rank, n_heads, rows, cycles,
                                                                              device_status_ptr());
  HK_LAUNCH_CHECK();
  const unsigned gather_ctas = (unsigned)((rows * LATENT * 2 / 16 + 127) / 128);
  sk_gather_kernel<<<gather_ctas < 512 ? gather_ctas : 512, 128, 0, s>>>((uint8_t*)my_region, n_ranks, rows, (__half*)out_f16, cycles,
                                                                         device_status_ptr());
  HK_LAUNCH_CHECK();
  return HK_OK;
}
