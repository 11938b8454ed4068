// Pooled indexer key of one pool, one thread per channel (helios::attn::kpool_write, reference: src/cuda/attn/attn.cu:332-390).
// A pool key is produced by the call that writes the pool's LAST member; members written by earlier calls are read back
// from the ring, members of this call straight from the inputs (and copied into the ring for later calls).
#pragma once
#include "hk_common.cuh"

namespace hk {

// ik / ig: the call's new key and gate rows [n_new][128] (any address space); p = pool, c = channel
__device__ __forceinline__ void kpool_one(const __half* ik, const __half* ig, __half* __restrict__ ring, int raw_rows,
                                          __half* __restrict__ pk_nt, const float* __restrict__ ape, int pos_start, int n_new,
                                          int p, int c) {
  const int t0 = p * POOL;
  const int last = t0 + POOL - 1;
  const bool complete = last >= pos_start && last < pos_start + n_new;
  float kk[POOL], gg[POOL];
  float mx = -1e30f;
#pragma unroll
  for (int i = 0; i < POOL; i++) {
    const int pos = t0 + i, src = pos - pos_start;
    __half* r = ring + (size_t)(pos % raw_rows) * 256;
    __half hk_, hg_;
    if (src >= 0 && src < n_new) {
      hk_ = ik[(size_t)src * 128 + c];
      hg_ = ig[(size_t)src * 128 + c];
      r[c] = hk_;
      r[128 + c] = hg_;
    } else if (complete && src < 0) {
      hk_ = r[c];
      hg_ = r[128 + c];
    } else {
      hk_ = __float2half(0.f);
      hg_ = __float2half(0.f);
    }
    kk[i] = __half2float(hk_);
    gg[i] = __half2float(hg_) + ape[i * 128 + c];
    mx = fmaxf(mx, gg[i]);
  }
  if (!complete) return;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < POOL; i++) {
    gg[i] = __expf(gg[i] - mx);
    sum += gg[i];
  }
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < POOL; i++) o += (gg[i] / sum) * kk[i];
  o *= 0.25f;
  pk_nt[(size_t)p * 128 + c] = __float2half_rn(o);
}

}  // namespace hk
