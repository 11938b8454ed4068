// CPU oracle for the GLM-5.3-Flash trunk-attention hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, on the host and in plain multithreaded C++, the
// arithmetic of the reference's CUDA kernels for the path.  Only the test-suite, the smoke check
// and the benchmark's cpu_baseline / reference legs may load it; the product library never does.
//
// Parity pinning: the reference has no CPU implementation of this path and cannot run without a
// GPU, so the restatement is pinned two ways: (1) against the closed-form fp64 definitions that the
// reference's own parity test carries inline (src/cuda/attn/test/test_attn_parity.cpp), reproduced
// with its mt19937(7) fixtures; (2) against outputs of the reference's kernels themselves, run on a
// B200 from the reference's sources (oracle/ref_shim.cu) and committed as fixtures under
// tests/golden/.
//
// Each function cites the reference file:line it follows (paths relative to the reference tree).
// Storage types: bf16 and fp16 tensors travel as uint16_t bit patterns.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------------------
// number formats
// ---------------------------------------------------------------------------------------------
inline float bf16_to_f(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f_to_bf16_rn(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
inline uint16_t f_to_bf16_rz(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  return (uint16_t)(u >> 16);
}
inline float h_to_f(uint16_t h) {
  _Float16 x;
  std::memcpy(&x, &h, 2);
  return (float)x;
}
inline uint16_t f_to_h_rn(float f) {
  _Float16 x = (_Float16)f;  // IEEE round-to-nearest-even
  uint16_t h;
  std::memcpy(&h, &x, 2);
  return h;
}

// ---------------------------------------------------------------------------------------------
// threading
// ---------------------------------------------------------------------------------------------
int g_threads = 0;

int n_threads() {
  if (g_threads > 0) return g_threads;
  if (const char* e = std::getenv("HK_ORACLE_THREADS")) {
    int v = std::atoi(e);
    if (v > 0) return v;
  }
  unsigned hc = std::thread::hardware_concurrency();
  return hc ? (int)hc : 1;
}

// Dynamic work distribution: items are claimed one at a time from an atomic counter.
void parallel_for(int64_t n, const std::function<void(int64_t)>& fn) {
  int nt = (int)std::min<int64_t>(n_threads(), n);
  if (nt <= 1) {
    for (int64_t i = 0; i < n; i++) fn(i);
    return;
  }
  std::atomic<int64_t> next(0);
  std::vector<std::thread> pool;
  pool.reserve(nt);
  for (int t = 0; t < nt; t++)
    pool.emplace_back([&]() {
      for (;;) {
        int64_t i = next.fetch_add(1);
        if (i >= n) break;
        fn(i);
      }
    });
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

void orc_set_threads(int n) { g_threads = n; }
int orc_get_threads() { return n_threads(); }

// ---------------------------------------------------------------------------------------------
// A1  causal short convolution + SiLU, rolling window state
// follows src/cuda/aux/gdn.cu:896-951 (conv1d_update_kernel) and the launcher :972-1023
//   x      [bsz][dim][seqlen]  bf16 (channel-major)
//   state  [slots][dim][state_size] bf16, updated in place
//   w      [dim][K] bf16, bias [dim] bf16 or null
//   out    [bsz][seqlen][dim] bf16 (round to nearest)
// ---------------------------------------------------------------------------------------------
int orc_conv1d_update(const uint16_t* x, uint16_t* state, const int* slots, const uint16_t* w,
                      const uint16_t* bias, uint16_t* out, int bsz, int dim, int seqlen,
                      int state_size, int K, int activation, int history) {
  if (K > 16 || state_size < K) return 1;
  parallel_for((int64_t)bsz * dim, [&](int64_t bd) {
    int b = (int)(bd / dim), d = (int)(bd % dim);
    int slot = slots ? slots[b] : b;
    const uint16_t* x_d = x + ((size_t)b * dim + d) * seqlen;
    uint16_t* st = state + ((size_t)slot * dim + d) * state_size;
    float wk[16], old_state[16], win[16];
    for (int k = 0; k < K; k++) wk[k] = bf16_to_f(w[(size_t)d * K + k]);
    float bias_d = bias ? bf16_to_f(bias[d]) : 0.0f;
    for (int k = 0; k < K; k++) old_state[k] = bf16_to_f(st[k]);
    for (int k = 0; k < K - 1; k++) win[k] = old_state[k + 1];
    for (int s = 0; s < seqlen; s++) {
      win[K - 1] = bf16_to_f(x_d[s]);
      float acc = bias_d;
      for (int k = 0; k < K; k++) acc = std::fmaf(wk[k], win[k], acc);
      if (activation) acc *= 1.0f / (1.0f + std::exp(-acc));
      out[((size_t)b * seqlen + s) * dim + d] = f_to_bf16_rn(acc);
      for (int k = 0; k < K - 1; k++) win[k] = win[k + 1];
    }
    if (!history) {
      for (int k = 0; k < K; k++) {
        int src_t = seqlen + k;
        float v = (src_t < K) ? old_state[src_t] : bf16_to_f(x_d[src_t - K]);
        st[k] = f_to_bf16_rn(v);
      }
    } else {
      int total = K + seqlen;
      int write_size = state_size < total ? state_size : total;
      int dst_start = state_size - write_size, src_start = total - write_size;
      for (int j = 0; j < write_size; j++) {
        int src_t = src_start + j;
        float v = (src_t < K) ? old_state[src_t] : bf16_to_f(x_d[src_t - K]);
        st[dst_start + j] = f_to_bf16_rn(v);
      }
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A2/A3  gated delta rule recurrence (KDA when channelwise)
// follows src/cuda/aux/gdn.cu:614-748 (128-dim kernel) / :316-553 (generic) and the launcher
// :760-866.  Per token and head:
//   q^ = q * rsqrt(sum q^2 + 1e-6), k^ likewise                       (:639-669)
//   channelwise: d_c = exp(g_c); kv_j = sum_c k^_c d_c S[c][j]         (:671, :680-705)
//   head-wide  : kv_j = sum_c k^_c S[c][j];  v'_j = v_j - kv_j * exp(g)
//   S[c][j] <- S[c][j] * decay + k^_c * v'_j * beta                    (:727-729)
//   o_j = (sum_c q^_c S_new[c][j]) / sqrt(dk)  -> bf16 round toward zero (:741)
// The k-reduction is done as 4 sub-sums over dk/4 consecutive channels, added in order 0..3
// (:683-705).  acc64 != 0 switches the reductions to fp64 (error attribution only).
//   mixed_qkv [bsz][seqlen][2*Hk*dk + Hv*dv] bf16 = q(Hk*dk) | k(Hk*dk) | v(Hv*dv)
//   g  [bsz][seqlen][Hv][dk] f32 (channelwise) or [bsz][seqlen][Hv]
//   beta [bsz][seqlen][Hv] bf16
//   state [slots][history_stride][Hv][dk][dv] f32, updated in place
//   out [bsz][seqlen][Hv][dv] bf16;  out_f32 (optional) same shape, value before rounding
// ---------------------------------------------------------------------------------------------
int orc_kda_recurrent(const uint16_t* mixed_qkv, const float* g, const uint16_t* beta, float* state,
                      uint16_t* out, float* out_f32, int bsz, int seqlen, int Hk, int Hv, int dk,
                      int dv, int history_stride, const int* slots, int channelwise, int history,
                      int acc64) {
  if (Hv % Hk != 0 || dk % 4 != 0) return 1;
  const int group = Hv / Hk;
  const size_t head_state = (size_t)dk * dv;
  const size_t state_size = (size_t)Hv * head_state;
  const size_t slot_size = (size_t)history_stride * state_size;
  const size_t row = (size_t)2 * Hk * dk + (size_t)Hv * dv;
  const float scale = 1.0f / std::sqrt((float)dk);
  const int sub = dk / 4;
  parallel_for((int64_t)bsz * Hv, [&](int64_t bh) {
    int b = (int)(bh / Hv), head = (int)(bh % Hv), k_head = head / group;
    int slot = slots ? slots[b] : b;
    float* slot_state = state + (size_t)slot * slot_size;
    std::vector<float> qn(dk), kn(dk), dec(dk), cur(head_state);
    std::memcpy(cur.data(), slot_state + head * head_state, head_state * sizeof(float));
    for (int s = 0; s < seqlen; s++) {
      const uint16_t* tok = mixed_qkv + ((size_t)b * seqlen + s) * row;
      const uint16_t* gq = tok + (size_t)k_head * dk;
      const uint16_t* gk = tok + (size_t)(Hk + k_head) * dk;
      const uint16_t* gv = tok + (size_t)2 * Hk * dk + (size_t)head * dv;
      const float* gg = g + ((size_t)b * seqlen + s) * Hv * (channelwise ? dk : 1) +
                        (size_t)head * (channelwise ? dk : 1);
      float sumq = 0.f, sumk = 0.f;
      for (int c = 0; c < dk; c++) {
        float q = bf16_to_f(gq[c]), k = bf16_to_f(gk[c]);
        sumq += q * q;
        sumk += k * k;
      }
      float rq = 1.0f / std::sqrt(sumq + 1e-6f), rk = 1.0f / std::sqrt(sumk + 1e-6f);
      for (int c = 0; c < dk; c++) {
        qn[c] = bf16_to_f(gq[c]) * rq;
        kn[c] = bf16_to_f(gk[c]) * rk;
        dec[c] = channelwise ? std::exp(gg[c]) : 1.0f;
      }
      float g_h = channelwise ? 1.0f : std::exp(gg[0]);
      float beta_h = bf16_to_f(beta[((size_t)b * seqlen + s) * Hv + head]);
      for (int j = 0; j < dv; j++) {
        float kv;
        if (acc64) {
          double a = 0;
          for (int c = 0; c < dk; c++) a += (double)kn[c] * dec[c] * cur[(size_t)c * dv + j];
          kv = (float)a;
        } else {
          kv = 0.f;
          for (int part = 0; part < 4; part++) {
            float sum = 0.f;
            for (int c = part * sub; c < (part + 1) * sub; c++)
              sum = sum + kn[c] * dec[c] * cur[(size_t)c * dv + j];
            kv = kv + sum;
          }
        }
        float v = bf16_to_f(gv[j]) - kv * g_h;
        float o;
        if (acc64) {
          double a = 0;
          for (int c = 0; c < dk; c++) {
            float st = cur[(size_t)c * dv + j];
            st = st * (channelwise ? dec[c] : g_h) + kn[c] * v * beta_h;
            cur[(size_t)c * dv + j] = st;
            a += (double)qn[c] * st;
          }
          o = (float)a;
        } else {
          o = 0.f;
          for (int part = 0; part < 4; part++) {
            float sum = 0.f;
            for (int c = part * sub; c < (part + 1) * sub; c++) {
              float st = cur[(size_t)c * dv + j];
              st = st * (channelwise ? dec[c] : g_h) + kn[c] * v * beta_h;
              cur[(size_t)c * dv + j] = st;
              sum = sum + qn[c] * st;
            }
            o = o + sum;
          }
        }
        size_t oi = (((size_t)b * seqlen + s) * Hv + head) * dv + j;
        out[oi] = f_to_bf16_rz(o * scale);
        if (out_f32) out_f32[oi] = o * scale;
      }
      if (history) {
        // step s writes history slot s+1; the last step writes the final slot 0 (:623-632)
        bool last = (s == seqlen - 1);
        float* dst = (last ? slot_state : slot_state + (size_t)(s + 1) * state_size) +
                     head * head_state;
        std::memcpy(dst, cur.data(), head_state * sizeof(float));
      }
    }
    if (!history)
      std::memcpy(slot_state + head * head_state, cur.data(), head_state * sizeof(float));
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A4  pooled indexer keys: ring write + softmax-weighted pooling of 4 consecutive tokens
// follows src/cuda/attn/attn.cu:332-382
//   idx_k, idx_g [n_new][128] f16; ring [raw_rows][256] f16; pool_k_nt [npools][128] f16;
//   ape [4][128] f32.  A pool is finalised by the call that writes its last member.
// ---------------------------------------------------------------------------------------------
int orc_kpool_write(const uint16_t* idx_k, const uint16_t* idx_g, uint16_t* ring, int raw_rows,
                    uint16_t* pool_k_nt, const float* ape, int pos_start, int n_new) {
  const int POOL = 4;
  int blocks = (pos_start + n_new + POOL - 1) / POOL;
  // pass 1: ring rows (all pools), pass 2: pool keys; the kernel's blocks may run in any order, and
  // its preconditions (ring larger than a call) make the result order-independent.
  for (int p = 0; p < blocks; p++)
    for (int j = 0; j < POOL; j++) {
      int pos = p * POOL + j, src = pos - pos_start;
      if (src >= 0 && src < n_new) {
        uint16_t* r = ring + (size_t)(pos % raw_rows) * 256;
        std::memcpy(r, idx_k + (size_t)src * 128, 256);
        std::memcpy(r + 128, idx_g + (size_t)src * 128, 256);
      }
    }
  for (int p = 0; p < blocks; p++) {
    int t0 = p * POOL, last = t0 + POOL - 1;
    if (last < pos_start || last >= pos_start + n_new) continue;
    for (int c = 0; c < 128; c++) {
      float gk[4], kk[4], mx = -1e30f;
      for (int i = 0; i < POOL; i++) {
        const uint16_t* r = ring + (size_t)((t0 + i) % raw_rows) * 256;
        kk[i] = h_to_f(r[c]);
        gk[i] = h_to_f(r[128 + c]) + ape[i * 128 + c];
        mx = std::max(mx, gk[i]);
      }
      float sum = 0.f;
      for (int i = 0; i < POOL; i++) {
        gk[i] = std::exp(gk[i] - mx);
        sum += gk[i];
      }
      float o = 0.f;
      for (int i = 0; i < POOL; i++) o += (gk[i] / sum) * kk[i];
      o *= 0.25f;
      pool_k_nt[(size_t)p * 128 + c] = f_to_h_rn(o);
    }
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A5  indexer scores
// follows src/cuda/attn/attn.cu:134-158 (scalar form) with the fp32 accumulation of :182-258
//   S[r][p] = 32^-1/2 * sum_h w[r][h] * relu(128^-1/2 * q[r][h] . pk[p]);  -inf if 4p+3 > q_pos[r]
//   key_is_bf16 selects bf16 storage for q / pool keys / w (the benchmark config); scores are f16.
//   acc64 != 0: fp64 accumulation (the inline definition of test_attn_parity.cpp:224-236).
// ---------------------------------------------------------------------------------------------
int orc_indexer_score(const uint16_t* q_idx, const uint16_t* pool_k_nt, const uint16_t* w,
                      const int* q_pos, uint16_t* scores, float* scores_f32, int m, int npools,
                      int n_heads, int key_is_bf16, int acc64) {
  auto ld = [&](uint16_t v) { return key_is_bf16 ? bf16_to_f(v) : h_to_f(v); };
  const uint16_t NEG_INF = 0xfc00;
  parallel_for((int64_t)m, [&](int64_t r) {
    std::vector<float> qf((size_t)n_heads * 128), wf(n_heads);
    for (int i = 0; i < n_heads * 128; i++) qf[i] = ld(q_idx[(size_t)r * n_heads * 128 + i]);
    for (int h = 0; h < n_heads; h++) wf[h] = ld(w[(size_t)r * n_heads + h]);
    int pos = q_pos[r];
    for (int p = 0; p < npools; p++) {
      size_t oi = (size_t)r * npools + p;
      if (p * 4 + 3 > pos) {
        scores[oi] = NEG_INF;
        if (scores_f32) scores_f32[oi] = -INFINITY;
        continue;
      }
      float kf[128];
      for (int d = 0; d < 128; d++) kf[d] = ld(pool_k_nt[(size_t)p * 128 + d]);
      float res;
      if (acc64) {
        double tot = 0;
        for (int h = 0; h < n_heads; h++) {
          double dot = 0;
          for (int d = 0; d < 128; d++) dot += (double)kf[d] * qf[(size_t)h * 128 + d];
          dot /= std::sqrt(128.0);
          if (dot > 0) tot += (double)wf[h] * dot;
        }
        res = (float)(tot / std::sqrt((double)n_heads));
      } else {
        float tot = 0.f;
        for (int h = 0; h < n_heads; h++) {
          float dot = 0.f;
          for (int d = 0; d < 128; d++) dot += kf[d] * qf[(size_t)h * 128 + d];
          dot *= 0.08838834764f;
          if (dot > 0.f) tot += wf[h] * dot;
        }
        res = tot * (1.0f / std::sqrt((float)n_heads));
      }
      scores[oi] = f_to_h_rn(res);
      if (scores_f32) scores_f32[oi] = res;
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A6  exact top-k over f16 scores, reference tie order
// follows src/cuda/aux/dsa_topk.cu:21-24 (order-preserving key), :134-144 (fewer than k finite),
// :179-267 (emission: every entry above the k-th value in ascending index order, then ties with
// the k-th value in ascending index order until k entries; -1 padding to k_pad)
// ---------------------------------------------------------------------------------------------
static inline uint16_t topk_key(uint16_t u) {
  return (u & 0x8000) ? (uint16_t)~u : (uint16_t)(u | 0x8000);
}

int orc_dsa_topk(const uint16_t* scores, int s_stride, int* indices, int R, int T, int k, int k_pad) {
  if (k > k_pad) return 1;
  const uint16_t KEY_NEG_INF = 0x03ff;
  parallel_for((int64_t)R, [&](int64_t r) {
    const uint16_t* row = scores + (size_t)r * s_stride;
    int* o = indices + (size_t)r * k_pad;
    std::vector<int> hist(65536, 0);
    int finite = 0;
    for (int i = 0; i < T; i++) {
      uint16_t key = topk_key(row[i]);
      if (key > KEY_NEG_INF) {
        hist[key]++;
        finite++;
      }
    }
    int emitted = 0;
    if (finite < k) {
      for (int i = 0; i < T; i++)
        if (topk_key(row[i]) > KEY_NEG_INF) o[emitted++] = i;
    } else if (k > 0) {
      int above = 0, thresh = 65535;
      for (; thresh > KEY_NEG_INF; thresh--) {
        if (above + hist[thresh] >= k) break;
        above += hist[thresh];
      }
      int n_eq_take = k - above;
      for (int i = 0; i < T; i++) {
        uint16_t key = topk_key(row[i]);
        if (key > KEY_NEG_INF && key > thresh) o[emitted++] = i;
      }
      int taken = 0;
      for (int i = 0; i < T && taken < n_eq_take; i++)
        if (topk_key(row[i]) == thresh) {
          o[emitted++] = i;
          taken++;
        }
    }
    for (int j = emitted; j < k_pad; j++) o[j] = -1;
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A7  pool index -> token index expansion (no de-duplication of the tail)
// follows src/cuda/attn/attn.cu:307-322 (per-row) and :284-298 (shared cur_pos when q_pos == null)
// ---------------------------------------------------------------------------------------------
int orc_pool_expand(const int* pool_idx, const int* q_pos, int* raw_idx, int m, int cur_pos,
                    int n_sel) {
  const int POOL = 4;
  const int row_len = n_sel * POOL + POOL;
  for (int r = 0; r < m; r++) {
    int cur = q_pos ? q_pos[r] : cur_pos;
    int* row = raw_idx + (size_t)r * row_len;
    for (int i = 0; i < n_sel; i++) {
      int pi = pool_idx[(size_t)r * n_sel + i];
      for (int j = 0; j < POOL; j++) {
        int tok = pi >= 0 ? pi * POOL + j : -1;
        row[i * POOL + j] = (tok >= 0 && tok <= cur) ? tok : -1;
      }
    }
    for (int i = 0; i < POOL; i++) {
      int tail = cur - (POOL - 1 - i);
      row[n_sel * POOL + i] = tail >= 0 ? tail : -1;
    }
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A8/A9  absorbed MLA attention over the latent cache (gathered rows or a dense causal range)
// follows src/cuda/attn/attn.cu:394-482 (sparse) and :621-692 (dense); softmax exactly as the
// reference test's inline fp64 definition (test_attn_parity.cpp:294-311, :322-338).
//   q_lat [m][n_heads][512] f16, ckv [Tmax][512] f16, out [m][n_heads][512] f16 (rn)
//   sparse: raw_idx [m][kidx] (-1 = skip, duplicates counted twice)
//   dense : raw_idx == null, row r attends ckv[base_r .. base_r + len_r) where
//           len_r = kv_len[r] (if given) else pos_start + r + 1, base_r = kv_base[r] (or 0)
//   part_m / part_l / part_acc (optional): un-normalised partial in the split-KV format
//           (m = running max of scaled scores, l = sum exp(s-m), acc[512] = sum exp(s-m) * row)
// ---------------------------------------------------------------------------------------------
int orc_mla_attend(const uint16_t* q_lat, const uint16_t* ckv, const int* raw_idx, int kidx,
                   const int64_t* kv_base, const int* kv_len, int pos_start, uint16_t* out,
                   float* out_f32, float* part_m, float* part_l, float* part_acc, int m,
                   int n_heads, float scale) {
  const int D = 512;
  parallel_for((int64_t)m * n_heads, [&](int64_t rh) {
    int r = (int)(rh / n_heads);
    const uint16_t* q = q_lat + (size_t)rh * D;
    float qf[D];
    for (int c = 0; c < D; c++) qf[c] = h_to_f(q[c]);
    int n;
    int64_t base = 0;
    if (raw_idx) n = kidx;
    else {
      n = kv_len ? kv_len[r] : pos_start + r + 1;
      base = kv_base ? kv_base[r] : 0;
    }
    std::vector<double> sc(n);
    double mx = -INFINITY;
    for (int i = 0; i < n; i++) {
      int64_t t = raw_idx ? raw_idx[(size_t)r * kidx + i] : base + i;
      if (t < 0) {
        sc[i] = -INFINITY;
        continue;
      }
      const uint16_t* kr = ckv + (size_t)t * D;
      double d = 0;
      for (int c = 0; c < D; c++) d += (double)qf[c] * h_to_f(kr[c]);
      sc[i] = d * (double)scale;
      mx = std::max(mx, sc[i]);
    }
    double l = 0;
    std::vector<double> acc(D, 0.0);
    for (int i = 0; i < n; i++) {
      if (sc[i] == -INFINITY) continue;
      int64_t t = raw_idx ? raw_idx[(size_t)r * kidx + i] : base + i;
      const uint16_t* kr = ckv + (size_t)t * D;
      double p = std::exp(sc[i] - mx);
      l += p;
      for (int c = 0; c < D; c++) acc[c] += p * h_to_f(kr[c]);
    }
    if (part_m) {
      part_m[rh] = (float)mx;
      part_l[rh] = (float)l;
      for (int c = 0; c < D; c++) part_acc[(size_t)rh * D + c] = (float)acc[c];
    }
    for (int c = 0; c < D; c++) {
      float v = l > 0 ? (float)(acc[c] / l) : 0.f;  // all skipped -> zeros (attn.cu:585,596)
      if (out) out[(size_t)rh * D + c] = f_to_h_rn(v);
      if (out_f32) out_f32[(size_t)rh * D + c] = v;
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A10  split-KV log-sum-exp combine
// follows the in-kernel merge src/cuda/attn/attn.cu:462-481:
//   gm = max_s m_s;  gl = sum_s e^{m_s-gm} l_s;  o = sum_s e^{m_s-gm} acc_s / gl
//   m_s = -inf contributes weight 0; every m_s = -inf (or gl = 0) gives zeros.
//   part_m, part_l [n_split][rows]; part_acc [n_split][rows][512]; out [rows][512] f16
// ---------------------------------------------------------------------------------------------
int orc_lse_combine(const float* part_m, const float* part_l, const float* part_acc, int n_split,
                    int64_t rows, uint16_t* out, float* out_f32) {
  const int D = 512;
  parallel_for(rows, [&](int64_t r) {
    double gm = -INFINITY;
    for (int s = 0; s < n_split; s++) gm = std::max(gm, (double)part_m[(size_t)s * rows + r]);
    double gl = 0;
    std::vector<double> o(D, 0.0);
    if (gm != -INFINITY) {
      for (int s = 0; s < n_split; s++) {
        double ms = part_m[(size_t)s * rows + r];
        double sc = ms == -INFINITY ? 0.0 : std::exp(ms - gm);
        gl += sc * part_l[(size_t)s * rows + r];
        const float* a = part_acc + ((size_t)s * rows + r) * D;
        for (int c = 0; c < D; c++) o[c] += sc * a[c];
      }
    }
    for (int c = 0; c < D; c++) {
      float v = gl > 0 ? (float)(o[c] / gl) : 0.f;
      if (out) out[(size_t)r * D + c] = f_to_h_rn(v);
      if (out_f32) out_f32[(size_t)r * D + c] = v;
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A11  absorbed projections (adjacent to the path)
// follows src/cuda/attn/attn.cu:12-34 (q_latent) and :69-84 (o_absorb)
//   q_lat[m,h,c] = sum_j q_nope[m,h,j] * kv_b[h*512+j][c]           (256 -> 512)
//   o[m,h,j]     = sum_c lat_out[m,h,c] * kv_b[h*512+256+j][c]      (512 -> 256)
// ---------------------------------------------------------------------------------------------
int orc_q_latent(const uint16_t* q_nope, const uint16_t* kv_b, uint16_t* q_lat, int m, int n_heads) {
  parallel_for((int64_t)m * n_heads, [&](int64_t rh) {
    int h = (int)(rh % n_heads);
    std::vector<double> acc(512, 0.0);
    for (int j = 0; j < 256; j++) {
      double qv = h_to_f(q_nope[(size_t)rh * 256 + j]);
      const uint16_t* wr = kv_b + ((size_t)h * 512 + j) * 512;
      for (int c = 0; c < 512; c++) acc[c] += qv * h_to_f(wr[c]);
    }
    for (int c = 0; c < 512; c++) q_lat[(size_t)rh * 512 + c] = f_to_h_rn((float)acc[c]);
  });
  return 0;
}

int orc_o_absorb(const uint16_t* lat_out, const uint16_t* kv_b, uint16_t* o, int m, int n_heads) {
  parallel_for((int64_t)m * n_heads, [&](int64_t rh) {
    int h = (int)(rh % n_heads);
    for (int j = 0; j < 256; j++) {
      const uint16_t* wr = kv_b + ((size_t)h * 512 + 256 + j) * 512;
      double acc = 0;
      for (int c = 0; c < 512; c++) acc += (double)h_to_f(lat_out[(size_t)rh * 512 + c]) * h_to_f(wr[c]);
      o[(size_t)rh * 256 + j] = f_to_h_rn((float)acc);
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// N2  KDA producers: transpose + cast and gate preparation
// follows src/engine/glue2.cu:318-344 (kda_transpose_cast_k) and :347-368 (kda_gate_k; the same
// arithmetic is in kda_prepare_k :370-396)
//   mixed[f][s] = bf16_rn(qkv[s][f]);  beta[s][h] = bf16_rn(sigmoid(b[s][h]))
//   g[s][h][d]  = lower_bound * sigmoid(exp(a_log[h]) * (f[s][h][d] + dt_bias[h][d]))
// exp here is the host's (the device uses its fast exponential): compare within a few ulp.
// ---------------------------------------------------------------------------------------------
int orc_kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                    const float* a_log, float lower_bound, uint16_t* mixed, uint16_t* beta, float* g,
                    int S, int F, int H, int Dk) {
  if (qkv && mixed) {
    parallel_for(F, [&](int64_t ff) {
      for (int s = 0; s < S; s++) mixed[(size_t)ff * S + s] = f_to_bf16_rn(qkv[(size_t)s * F + ff]);
    });
  }
  if (b && beta) {
    for (int64_t j = 0; j < (int64_t)S * H; j++) beta[j] = f_to_bf16_rn(1.0f / (1.0f + std::exp(-b[j])));
  }
  if (f && g) {
    parallel_for(S, [&](int64_t s) {
      for (int h = 0; h < H; h++) {
        const float decay = std::exp(a_log[h]);
        for (int d = 0; d < Dk; d++) {
          const size_t i = ((size_t)s * H + h) * Dk + d;
          g[i] = lower_bound * (1.0f / (1.0f + std::exp(-(decay * (f[i] + dt_bias[h * Dk + d])))));
        }
      }
    });
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// N3  gated RMS norm (the KDA output gate)
// follows src/cuda/aux/norm.cu:294-392 (gated_rms_norm_kernel) and the launcher :402-468
//   y = x * w * rsqrt(mean(x^2) + eps) * act(g)        (gate_first: act(g) multiplies x before the norm)
//   x bf16; w f32 or bf16, row r uses w[r % w_groups]; g f32 or bf16; y f16 (rn) or f32
//   act = SiLU (gate_act 0) or sigmoid (gate_act 1).  The sum of squares runs in fp64 here (the device
//   sums fp32 partials in lane order); products follow the device order x * w * rmf, then * act(g).
// ---------------------------------------------------------------------------------------------
int orc_gated_rms_norm(const uint16_t* x, const void* w, int w_bf16, void* y, int y_f32, const void* g,
                       int g_bf16, int64_t rows, int dim, float eps, float constant_bias, int w_groups,
                       int gate_first, int gate_act) {
  if (dim % 4 != 0 || w_groups < 1) return 1;
  parallel_for(rows, [&](int64_t r) {
    auto wv = [&](int c) {
      const size_t i = (size_t)(r % w_groups) * dim + c;
      return (w_bf16 ? bf16_to_f(((const uint16_t*)w)[i]) : ((const float*)w)[i]) + (constant_bias != 0.0f ? constant_bias : 0.0f);
    };
    auto gv = [&](int c) {
      const size_t i = (size_t)r * dim + c;
      const float v = g_bf16 ? bf16_to_f(((const uint16_t*)g)[i]) : ((const float*)g)[i];
      const float sg = 1.0f / (1.0f + std::exp(-v));
      return gate_act == 1 ? sg : v * sg;
    };
    double ss = 0.0;
    for (int c = 0; c < dim; c++) {
      float xv = bf16_to_f(x[(size_t)r * dim + c]);
      if (gate_first) xv *= gv(c);
      ss += (double)xv * xv;
    }
    const float rmf = 1.0f / std::sqrt((float)(ss / dim) + eps);
    for (int c = 0; c < dim; c++) {
      float xv = bf16_to_f(x[(size_t)r * dim + c]);
      if (gate_first) xv *= gv(c);
      float o = xv * wv(c) * rmf;
      if (!gate_first) o *= gv(c);
      if (y_f32) ((float*)y)[(size_t)r * dim + c] = o;
      else ((uint16_t*)y)[(size_t)r * dim + c] = f_to_h_rn(o);
    }
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// N4  producers of the latent cache and of the indexer keys
// orc_mla_cache_append follows src/cuda/aux/norm.cu:16-164 (rms_norm_kernel, float in / half weight /
// half out) and the copy into the cache at src/engine/runner.cpp:571-572:
//   ckv[pos + r][c] = f16_rn(kv_pre[r][c] * ln_w[c] * rsqrt(mean(kv_pre[r]^2) + eps)),  dim 512
// orc_layernorm_f16 follows src/engine/glue2.cu:420-447:
//   y = f16_rn((x - mean) * rsqrt(E[x^2] - mean^2 + eps) * w + b)
// Sums run in fp64 here (the device adds fp32 partials in lane order).
// ---------------------------------------------------------------------------------------------
int orc_mla_cache_append(const float* kv_pre, const uint16_t* ln_w, uint16_t* ckv, int64_t pos, int n, float eps) {
  parallel_for(n, [&](int64_t r) {
    const float* x = kv_pre + (size_t)r * 512;
    double ss = 0.0;
    for (int c = 0; c < 512; c++) ss += (double)x[c] * x[c];
    const float rmf = 1.0f / std::sqrt((float)(ss / 512.0) + eps);
    for (int c = 0; c < 512; c++) ckv[(size_t)(pos + r) * 512 + c] = f_to_h_rn(x[c] * h_to_f(ln_w[c]) * rmf);
  });
  return 0;
}

int orc_layernorm_f16(const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y, int rows, int dim,
                      float eps) {
  parallel_for(rows, [&](int64_t r) {
    const uint16_t* xr = x + (size_t)r * dim;
    double sum = 0.0, sq = 0.0;
    for (int i = 0; i < dim; i++) {
      const double v = h_to_f(xr[i]);
      sum += v;
      sq += v * v;
    }
    const float mean = (float)(sum / dim), var = (float)(sq / dim) - mean * mean;
    const float inv = 1.0f / std::sqrt(var + eps);
    for (int i = 0; i < dim; i++)
      y[(size_t)r * dim + i] = f_to_h_rn((h_to_f(xr[i]) - mean) * inv * h_to_f(w[i]) + h_to_f(b[i]));
  });
  return 0;
}

}  // extern "C"
