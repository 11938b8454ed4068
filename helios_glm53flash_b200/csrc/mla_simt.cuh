// CUDA-core flash attention over the latent cache: the cross-check / odd-shape path of the MLA
// entry points (any head count divisible by 4, any key count), and the split-KV combine kernels.
// fp32 products and accumulation throughout (the reference's scalar kernels use fp16 products,
// src/cuda/attn/attn.cu:517-533).
#pragma once
#include "hk_common.cuh"
#include "mla_args.cuh"

namespace hk {

constexpr int SIMT_HG = 4;  // heads per CTA



// grid (n_heads/4, n_split, m), 256 threads.  Warp w walks keys k0+w, k0+w+8, ...; lane owns 16
// channels; the 8 warps are merged through shared memory at the end.
__global__ __launch_bounds__(256) void mla_simt_kernel(MlaArgs a) {
  extern __shared__ float smem[];
  float* w_acc = smem;                           // [8][4][512]
  float* w_m = smem + 8 * SIMT_HG * LATENT;      // [8][4]
  float* w_l = w_m + 8 * SIMT_HG;                // [8][4]
  const int hg = blockIdx.x, sp = blockIdx.y, r = blockIdx.z;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int h0 = hg * SIMT_HG;
  const bool sparse = a.raw_idx != nullptr;
  int n;
  int64_t base = 0;
  if (sparse) n = a.kidx;
  else {
    n = a.kv_len ? a.kv_len[r] : a.pos_start + r + 1;
    base = a.kv_base ? a.kv_base[r] : 0;
    if (a.ckv_rows > 0) n = (int)max((int64_t)0, min((int64_t)n, a.ckv_rows - base));
  }
  const int per = (n + a.n_split - 1) / a.n_split;
  const int k0 = sp * per, k1 = min(n, k0 + per);

  float qf[SIMT_HG][16];
#pragma unroll
  for (int h = 0; h < SIMT_HG; h++) {
    const __half* q = a.q_lat + ((size_t)r * a.n_heads + h0 + h) * LATENT + lane * 16;
    uint4 u0 = *reinterpret_cast<const uint4*>(q), u1 = *reinterpret_cast<const uint4*>(q + 8);
    const __half2* p0 = reinterpret_cast<const __half2*>(&u0);
    const __half2* p1 = reinterpret_cast<const __half2*>(&u1);
#pragma unroll
    for (int u = 0; u < 4; u++) {
      float2 f0 = __half22float2(p0[u]), f1 = __half22float2(p1[u]);
      qf[h][2 * u] = f0.x * a.scale; qf[h][2 * u + 1] = f0.y * a.scale;
      qf[h][8 + 2 * u] = f1.x * a.scale; qf[h][8 + 2 * u + 1] = f1.y * a.scale;
    }
  }
  float m_i[SIMT_HG], l_i[SIMT_HG], acc[SIMT_HG][16];
#pragma unroll
  for (int h = 0; h < SIMT_HG; h++) {
    m_i[h] = -INFINITY;
    l_i[h] = 0.f;
#pragma unroll
    for (int u = 0; u < 16; u++) acc[h][u] = 0.f;
  }
  for (int i = k0 + wid; i < k1; i += 8) {
    int64_t tok = sparse ? (int64_t)a.raw_idx[(size_t)r * a.kidx + i] : base + i;
    if (tok < 0 || (a.ckv_rows > 0 && tok >= a.ckv_rows)) continue;  // warp-uniform
    const __half* crow = a.ckv + (size_t)tok * LATENT + lane * 16;
    uint4 u0 = *reinterpret_cast<const uint4*>(crow), u1 = *reinterpret_cast<const uint4*>(crow + 8);
    const __half2* p0 = reinterpret_cast<const __half2*>(&u0);
    const __half2* p1 = reinterpret_cast<const __half2*>(&u1);
    float kf[16];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      float2 f0 = __half22float2(p0[u]), f1 = __half22float2(p1[u]);
      kf[2 * u] = f0.x; kf[2 * u + 1] = f0.y; kf[8 + 2 * u] = f1.x; kf[8 + 2 * u + 1] = f1.y;
    }
#pragma unroll
    for (int h = 0; h < SIMT_HG; h++) {
      float d = 0.f;
#pragma unroll
      for (int u = 0; u < 16; u++) d = fmaf(qf[h][u], kf[u], d);
      d = warp_sum(d);
      if (d > m_i[h]) {
        const float sc = __expf(m_i[h] - d);
#pragma unroll
        for (int u = 0; u < 16; u++) acc[h][u] *= sc;
        l_i[h] *= sc;
        m_i[h] = d;
      }
      const float p = __expf(d - m_i[h]);
      l_i[h] += p;
#pragma unroll
      for (int u = 0; u < 16; u++) acc[h][u] = fmaf(p, kf[u], acc[h][u]);
    }
  }
#pragma unroll
  for (int h = 0; h < SIMT_HG; h++) {
    if (lane == 0) {
      w_m[wid * SIMT_HG + h] = m_i[h];
      w_l[wid * SIMT_HG + h] = l_i[h];
    }
#pragma unroll
    for (int u = 0; u < 16; u++) w_acc[(wid * SIMT_HG + h) * LATENT + lane * 16 + u] = acc[h][u];
  }
  __syncthreads();
  const size_t rows = (size_t)a.m * a.n_heads;
  for (int idx = threadIdx.x; idx < SIMT_HG * LATENT; idx += 256) {
    const int h = idx / LATENT, ch = idx % LATENT;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; w++) gm = fmaxf(gm, w_m[w * SIMT_HG + h]);
    float gl = 0.f, o = 0.f;
    if (gm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 8; w++) {
        const float mw = w_m[w * SIMT_HG + h];
        const float sc = mw == -INFINITY ? 0.f : __expf(mw - gm);
        gl += sc * w_l[w * SIMT_HG + h];
        o += sc * w_acc[(w * SIMT_HG + h) * LATENT + ch];
      }
    }
    const size_t rh = (size_t)r * a.n_heads + h0 + h;
    if (a.out) {
      a.out[rh * LATENT + ch] = __float2half_rn(gl > 0.f ? o / gl : 0.f);
    } else {
      a.part_acc[((size_t)sp * rows + rh) * LATENT + ch] = o;
      if (ch == 0) {
        a.part_m[(size_t)sp * rows + rh] = gm;
        a.part_l[(size_t)sp * rows + rh] = gl;
      }
    }
  }
}

constexpr size_t MLA_SIMT_SMEM = (size_t)(8 * SIMT_HG * LATENT + 2 * 8 * SIMT_HG) * sizeof(float);

// ---- split-KV log-sum-exp combine: one CTA (128 threads x 4 channels) per (row, head) ----
// gm = max m_s; gl = sum e^{m_s-gm} l_s; o = sum e^{m_s-gm} acc_s / gl; m_s = -inf weighs 0; all
// -inf (or gl = 0) gives zeros (reference in-kernel merge: src/cuda/attn/attn.cu:462-481).
// One CTA of 1024 threads per (row, head).  The split weights e^{m_s-gm} are computed once into shared
// memory (splits strided over the threads); the accumulators are then summed by eight thread groups
// (splits strided over the groups), thread = one float4 of the 512 channels, independent loads in flight.
constexpr int LSE_MAX_SPLITS = 1024;
constexpr int LSE_GROUPS = 8;
constexpr int LSE_THREADS = 128 * LSE_GROUPS;
// Few splits over many rows (batched decode): two thread groups per row instead of eight, so that every row's CTA
// is resident at once (256 threads: 8 CTAs per SM) and a thread keeps up to 12 independent loads in flight.
constexpr int LSE_GROUPS_FEW = 2;
constexpr int LSE_FEW_SPLITS = 24;

// LANES float4 lanes per thread group = the channels [cpart * 4 LANES, (cpart + 1) * 4 LANES) of the row; PRE =
// accumulator pieces per thread requested ahead of the weights.
template <bool PTRS, int GROUPS, int LANES = 128, int PRE = 24 / GROUPS>
__device__ __forceinline__ void lse_reduce_row(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                               const float* __restrict__ part_acc, const float* const* __restrict__ ptrs_m,
                                               const float* const* __restrict__ ptrs_l,
                                               const float* const* __restrict__ ptrs_acc, int n_split, int64_t rows,
                                               int64_t r, float& gm_out, float& gl_out, float4& o_out, int cpart = 0) {
  constexpr int THREADS = LANES * GROUPS;
  __shared__ float s_w[LSE_MAX_SPLITS];
  __shared__ float s_red[THREADS / 32];
  __shared__ float4 s_o[GROUPS - 1][LANES];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int cq = t % LANES, sg = t / LANES;
  auto load_acc = [&](int s) -> float4 {
    const float* pa = PTRS ? ptrs_acc[s] : part_acc + (size_t)s * rows * LATENT;
    const float4* ap = reinterpret_cast<const float4*>(pa + (size_t)r * LATENT) + cpart * LANES + cq;
    // peer memory: cache-volatile.  Local partials: L2 loads (ld.global.cg), never the non-coherent read-only path:
    // as a programmatic dependent this kernel's lifetime overlaps the grid that writes the partials.
    return PTRS ? __ldcv(ap) : __ldcg(ap);
  };
  auto load_ml = [&](const float* base) -> float { return PTRS ? __ldcv(base + r) : __ldcg(base + r); };
  // All loads that do not depend on the weights go out first: this thread's first PRE accumulator pieces
  // and the (m, l) pair of split t.  The weight phases below then run while they are in flight (one memory
  // round trip on the critical path instead of three).
  float4 pre[PRE];
#pragma unroll
  for (int u = 0; u < PRE; u++) {
    const int s = sg + u * GROUPS;
    pre[u] = s < n_split ? load_acc(s) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m_first = -INFINITY, l_first = 0.f;
  if (t < n_split) {
    m_first = load_ml(PTRS ? ptrs_m[t] : part_m + (size_t)t * rows);
    l_first = load_ml(PTRS ? ptrs_l[t] : part_l + (size_t)t * rows);
  }
  float mloc = -INFINITY;
  for (int s = t; s < n_split; s += THREADS) {
    const float m = s == t ? m_first : load_ml(PTRS ? ptrs_m[s] : part_m + (size_t)s * rows);
    s_w[s] = m;
    mloc = fmaxf(mloc, m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
  if (lane == 0) s_red[warp] = mloc;
  __syncthreads();
  float gm = s_red[0];
#pragma unroll
  for (int w = 1; w < THREADS / 32; w++) gm = fmaxf(gm, s_red[w]);
  __syncthreads();
  float lloc = 0.f;
  for (int s = t; s < n_split; s += THREADS) {
    const float m = s_w[s];
    const float w = (m == -INFINITY) ? 0.f : __expf(m - gm);
    s_w[s] = w;
    lloc += w * (s == t ? l_first : load_ml(PTRS ? ptrs_l[s] : part_l + (size_t)s * rows));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
  if (lane == 0) s_red[warp] = lloc;
  __syncthreads();
  float gl = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; w++) gl += s_red[w];
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  // same summation order as a plain loop over s = sg, sg + GROUPS, ...
#pragma unroll
  for (int u = 0; u < PRE; u++) {
    const int s = sg + u * GROUPS;
    if (s < n_split) {
      const float w = s_w[s];
      o.x = fmaf(w, pre[u].x, o.x); o.y = fmaf(w, pre[u].y, o.y); o.z = fmaf(w, pre[u].z, o.z); o.w = fmaf(w, pre[u].w, o.w);
    }
  }
#pragma unroll 4
  for (int s = sg + PRE * GROUPS; s < n_split; s += GROUPS) {
    const float4 a = load_acc(s);
    const float w = s_w[s];
    o.x = fmaf(w, a.x, o.x); o.y = fmaf(w, a.y, o.y); o.z = fmaf(w, a.z, o.z); o.w = fmaf(w, a.w, o.w);
  }
  if (sg > 0) s_o[sg - 1][cq] = o;
  __syncthreads();
  if (sg == 0) {
#pragma unroll
    for (int gi = 0; gi < GROUPS - 1; gi++) {
      const float4 p = s_o[gi][cq];
      o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
    }
  }
  gm_out = gm; gl_out = gl; o_out = o;      // o is complete in threads 0..LANES-1
}

template <bool PTRS, int GROUPS>
__global__ __launch_bounds__(128 * GROUPS) void lse_combine_kernel(
    const float* __restrict__ part_m, const float* __restrict__ part_l,
    const float* __restrict__ part_acc, const float* const* __restrict__ ptrs_m,
    const float* const* __restrict__ ptrs_l, const float* const* __restrict__ ptrs_acc,
    int n_split, int64_t rows, __half* __restrict__ out) {
  // when launched as a programmatic dependent of the kernel that writes the partials: wait until that grid has
  // completed and its writes are visible (a no-op after a plain launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t r = blockIdx.x;
  float gm, gl;
  float4 o;
  lse_reduce_row<PTRS, GROUPS>(part_m, part_l, part_acc, ptrs_m, ptrs_l, ptrs_acc, n_split, rows, r, gm, gl, o);
  if (threadIdx.x < 128) {
    const float inv = gl > 0.f ? 1.f / gl : 0.f;
    __half2 h0 = __floats2half2_rn(o.x * inv, o.y * inv);
    __half2 h1 = __floats2half2_rn(o.z * inv, o.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(out + (size_t)r * LATENT + threadIdx.x * 4) = pk;
  }
}

// The same for few rows (single-sequence decode: 64 (row, head) pairs): every row is shared by CSPLIT CTAs, each
// owning 512 / CSPLIT channels, with GROUPS groups of 32 float4 lanes over the splits, so that 64 rows still cover
// the machine and a thread has all of its loads in flight at once.  grid = (rows, CSPLIT).
constexpr int LSE_CSPLIT = 4;
template <int GROUPS>
__global__ __launch_bounds__(32 * GROUPS) void lse_combine_cs_kernel(
    const float* __restrict__ part_m, const float* __restrict__ part_l, const float* __restrict__ part_acc,
    int n_split, int64_t rows, __half* __restrict__ out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");   // see lse_combine_kernel
  constexpr int LANES = 128 / LSE_CSPLIT;
  const int64_t r = blockIdx.x;
  const int cpart = blockIdx.y;
  float gm, gl;
  float4 o;
  lse_reduce_row<false, GROUPS, LANES, 3>(part_m, part_l, part_acc, nullptr, nullptr, nullptr, n_split, rows, r,
                                                                gm, gl, o, cpart);
  if (threadIdx.x < LANES) {
    const float inv = gl > 0.f ? 1.f / gl : 0.f;
    __half2 h0 = __floats2half2_rn(o.x * inv, o.y * inv);
    __half2 h1 = __floats2half2_rn(o.z * inv, o.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(out + (size_t)r * LATENT + (cpart * LANES + threadIdx.x) * 4) = pk;
  }
}

// ---- merge of S partial sets into ONE partial set (still un-normalised): the per-GPU reduction before
// the cross-GPU exchange, so that only 2,056 B per (row, head) cross NVLink ----
// With a step counter (split-KV across GPUs, double-buffered exchange sets) the set of the step that is
// being computed, (*step_ctr + 1) & 1, is the one written.
__global__ __launch_bounds__(LSE_THREADS) void lse_merge_partials_kernel(
    const float* __restrict__ part_m, const float* __restrict__ part_l, const float* __restrict__ part_acc,
    int n_split, int64_t rows, float* __restrict__ out_m, float* __restrict__ out_l, float* __restrict__ out_acc,
    float* __restrict__ out_m1, float* __restrict__ out_l1, float* __restrict__ out_acc1,
    const int* __restrict__ step_ctr) {
  const int64_t r = blockIdx.x;
  float gm, gl;
  float4 o;
  lse_reduce_row<false, LSE_GROUPS>(part_m, part_l, part_acc, nullptr, nullptr, nullptr, n_split, rows, r, gm, gl, o);
  if (step_ctr && ((*step_ctr + 1) & 1)) {
    out_m = out_m1; out_l = out_l1; out_acc = out_acc1;
  }
  if (threadIdx.x < 128) *reinterpret_cast<float4*>(out_acc + (size_t)r * LATENT + threadIdx.x * 4) = o;
  if (threadIdx.x == 0) {
    out_m[r] = gm;
    out_l[r] = gl;
  }
}

// ---- split-KV across GPUs: peer signal + combine over peer-mapped partial buffers ----
// Rank g publishes "my partial of step `epoch` is complete" by storing `epoch` into slot g of every
// rank's flag array (its own included).  The stores are system-scope releases issued after a
// system-scope fence, in a kernel launched behind the partial kernel on the same stream.
__global__ void peer_signal_kernel(int* const* __restrict__ flag_ptrs, int n_ranks, int my_rank, int epoch) {
  const int s = threadIdx.x;
  if (s < n_ranks) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag_ptrs[s] + my_rank), "r"(epoch) : "memory");
  }
}

// The same with the step number kept on the device (so that a captured graph can be replayed): the
// step is *step_ctr + 1; the counter is advanced here, after the stores (or instead of them when
// do_store == 0: a rank that stays silent for one step, used by failure-injection tests).
__global__ void peer_signal_ctr_kernel(int* const* __restrict__ flag_ptrs, int n_ranks, int my_rank,
                                       int* __restrict__ step_ctr, int do_store) {
  const int s = threadIdx.x;
  const int epoch = *step_ctr + 1;
  __syncthreads();
  if (s < n_ranks && do_store) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag_ptrs[s] + my_rank), "r"(epoch) : "memory");
  }
  if (s == 0) *step_ctr = epoch;
}

// Combine that first waits (bounded) until every rank's flag in THIS GPU's flag array has reached
// `epoch`, then reads the S partial sets through their pointers (peer memory: plain cache-volatile
// loads over NVLink, nothing else).  On expiry the CTA writes nothing and reports a timeout.
__global__ __launch_bounds__(128) void lse_combine_peers_kernel(
    const float* const* __restrict__ ptrs_m, const float* const* __restrict__ ptrs_l,
    const float* const* __restrict__ ptrs_acc, int n_split, int64_t rows, __half* __restrict__ out,
    const int* __restrict__ flags, int epoch, long long max_wait_cycles, int* __restrict__ status,
    const int* __restrict__ step_ctr) {
  __shared__ int ready;
  if (step_ctr) {
    // device-side step number; the pointer tables hold both exchange sets, [parity][rank]
    epoch = *step_ctr;
    const int par = epoch & 1;
    ptrs_m += par * n_split; ptrs_l += par * n_split; ptrs_acc += par * n_split;
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (int s = 0; s < n_split; s++) {
      for (;;) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + s) : "memory");
        if (v >= epoch) break;
        if (clock64() - t0 > max_wait_cycles) { ok = 0; break; }
        __nanosleep(200);
      }
      if (!ok) break;
    }
    ready = ok;
    if (!ok && status) atomicExch(status, HK_ERR_TIMEOUT);
  }
  __syncthreads();
  if (!ready) return;
  const int64_t r = blockIdx.x;
  const int t = threadIdx.x;
  float gm = -INFINITY, gl = 0.f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  // batches of 8 partial sets: every load of a batch is issued before the first one is used, so a batch costs one
  // round trip over NVLink (a loop that uses each value as it arrives pays one round trip per set and pass)
  for (int s0 = 0; s0 < n_split; s0 += 8) {
    float ms[8], ls[8];
    float4 as[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int s = s0 + u;
      if (s < n_split) {
        ms[u] = __ldcv(ptrs_m[s] + r);
        ls[u] = __ldcv(ptrs_l[s] + r);
        as[u] = __ldcv(reinterpret_cast<const float4*>(ptrs_acc[s] + (size_t)r * LATENT + t * 4));
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
  *reinterpret_cast<uint2*>(out + (size_t)r * LATENT + t * 4) = pk;
}

}  // namespace hk
