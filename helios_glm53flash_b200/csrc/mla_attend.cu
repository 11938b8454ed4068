// Host entry points of absorbed MLA over the latent cache (dense / sparse, final / partial) and of
// the split-KV log-sum-exp combine.  Replaces helios::attn::mla_sparse_decode and
// helios::attn::mla_dense_prefill (reference: src/cuda/attn/attn.cu:394-699) and restates the
// reference's in-kernel merge (:462-481) as a standalone combine.
//
// Dispatch: 64-head launches go to the tcgen05 flash kernel (mla_flash_tc.cu); every other head
// count (multiple of 4) and the HK_MLA_FORCE_SIMT debug switch go to the CUDA-core kernel.
#include <cstdlib>

#include "mla_simt.cuh"

namespace hk {

// implemented in mla_flash_tc.cu; returns HK_ERR_UNSUPPORTED when the shape is not covered
int mla_flash_tc_launch(const MlaArgs& a, cudaStream_t s);
int mla_flash_tc_auto_splits(int m, int n_keys);

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct PartialLayout {
  size_t off_l, off_acc, total;
};
static PartialLayout partial_layout(int n_split, int64_t rows) {
  PartialLayout p;
  size_t ml = align_up((size_t)n_split * rows * sizeof(float), 256);
  p.off_l = ml;
  p.off_acc = 2 * ml;
  p.total = p.off_acc + (size_t)n_split * rows * LATENT * sizeof(float);
  return p;
}

static bool force_simt() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("HK_MLA_FORCE_SIMT");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

static int simt_auto_splits(int m, int n_heads, int n_keys) {
  long ctas = (long)m * (n_heads / SIMT_HG);
  int want = (int)((2L * sm_count() + ctas - 1) / ctas);
  int cap = (n_keys + 63) / 64;
  int s = want < 1 ? 1 : want;
  if (s > cap) s = cap < 1 ? 1 : cap;
  if (s > 64) s = 64;
  return s;
}

static int launch_simt(const MlaArgs& a, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(mla_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)MLA_SIMT_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  dim3 grid(a.n_heads / SIMT_HG, a.n_split, a.m);
  mla_simt_kernel<<<grid, 256, MLA_SIMT_SMEM, s>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

// Launched with programmatic stream serialisation: the flash kernel releases its dependents at entry, so the
// combine's CTAs are placed while the partial kernel still runs and block in griddepcontrol.wait (first statement
// of lse_combine_kernel) until that grid has completed and its writes are visible; the launch latency of the
// second kernel disappears from every decode step.  Behind any other kernel the attribute only delays the start
// until that kernel has finished, as a plain launch would.
template <int GROUPS>
static int combine_launch(const float* pm, const float* pl, const float* pa, int n_split, int64_t rows, __half* out,
                          cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows);
  cfg.blockDim = dim3(128 * GROUPS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* const* none = nullptr;
  return cudaLaunchKernelEx(&cfg, lse_combine_kernel<false, GROUPS>, pm, pl, pa, none, none, none, n_split, rows, out) ==
                 cudaSuccess
             ? HK_OK
             : HK_ERR_CUDA;
}

template <int GROUPS>
static int combine_cs_launch(const float* pm, const float* pl, const float* pa, int n_split, int64_t rows, __half* out,
                             cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows, LSE_CSPLIT);
  cfg.blockDim = dim3(32 * GROUPS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, lse_combine_cs_kernel<GROUPS>, pm, pl, pa, n_split, rows, out) == cudaSuccess ? HK_OK
                                                                                                                 : HK_ERR_CUDA;
}

static int combine(const float* pm, const float* pl, const float* pa, int n_split, int64_t rows,
                   __half* out, cudaStream_t s) {
  if (n_split > LSE_MAX_SPLITS) return HK_ERR_UNSUPPORTED;
  // few rows and few splits (sparse decode of one sequence: 64 rows x 22 splits): channel-split form, four CTAs per
  // row (15.1 vs 16.1 us per layer for the sparse step).  With many splits (dense decode of one sequence, 137) the
  // same form with 32 thread groups measured slower than eight groups of 128 lanes (24.5 vs 23.5 us): not used.
  if (rows < 256 && n_split <= LSE_FEW_SPLITS) return combine_cs_launch<8>(pm, pl, pa, n_split, rows, out, s);
  if (n_split <= LSE_FEW_SPLITS && rows >= 256) return combine_launch<LSE_GROUPS_FEW>(pm, pl, pa, n_split, rows, out, s);
  return combine_launch<LSE_GROUPS>(pm, pl, pa, n_split, rows, out, s);
}

// common driver: final output, optionally through split partials in the workspace
static int attend(MlaArgs a, int n_keys_hint, int n_split, void* workspace, size_t workspace_bytes,
                  cudaStream_t s) {
  const bool tc = (a.n_heads == 64) && !force_simt();
  if (n_split <= 0)
    n_split = tc ? mla_flash_tc_auto_splits(a.m, n_keys_hint)
                 : simt_auto_splits(a.m, a.n_heads, n_keys_hint);
  const int64_t rows = (int64_t)a.m * a.n_heads;
  __half* final_out = a.out;
  a.n_split = n_split;
  if (n_split > 1) {
    PartialLayout pl = partial_layout(n_split, rows);
    if (!workspace || workspace_bytes < pl.total) return HK_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return HK_ERR_INVALID;
    char* ws = (char*)workspace;
    a.part_m = (float*)ws;
    a.part_l = (float*)(ws + pl.off_l);
    a.part_acc = (float*)(ws + pl.off_acc);
    a.out = nullptr;
  }
  int st = HK_ERR_UNSUPPORTED;
  if (tc) st = mla_flash_tc_launch(a, s);
  if (st == HK_ERR_UNSUPPORTED) st = launch_simt(a, s);
  if (st != HK_OK) return st;
  if (n_split > 1) return combine(a.part_m, a.part_l, a.part_acc, n_split, rows, final_out, s);
  return HK_OK;
}

}  // namespace hk

HK_API size_t hk_mla_partial_bytes(int n_split, int64_t rows) {
  if (n_split <= 0 || rows <= 0) return 0;
  return hk::partial_layout(n_split, rows).total;
}

HK_API int hk_mla_auto_splits(int m, int n_keys) {
  if (m <= 0 || n_keys <= 0) return 1;
  return hk::force_simt() ? hk::simt_auto_splits(m, 64, n_keys) : hk::mla_flash_tc_auto_splits(m, n_keys);
}

HK_API int hk_mla_sparse(const void* q_lat, const void* ckv, int64_t ckv_rows, const int* raw_idx, int kidx,
                         void* lat_out, int m, int n_heads, float scale, int n_split,
                         void* workspace, size_t workspace_bytes, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv && raw_idx && lat_out && ckv_rows >= 0);
  HK_REQUIRE(m >= 0 && kidx >= 0 && n_heads > 0 && n_heads % SIMT_HG == 0);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv, 16) && aligned(lat_out, 16));
  if (m == 0) return HK_OK;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv; a.ckv_rows = ckv_rows;
  a.raw_idx = raw_idx; a.kidx = kidx;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  a.out = (__half*)lat_out;
  return attend(a, kidx, n_split, workspace, workspace_bytes, as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// Sparse MLA decode for callers that cannot allocate device memory.
//
// Some hosts of this library own all of their device memory up front and have nothing to hand out
// at call time: the Helios engine carves every buffer out of one bump allocator at start-up and
// its launcher signatures carry no workspace pointer, and code running under a memory-pool policy
// or inside a region where the CUDA allocator must not be entered has the same problem.  For them
// the split-KV partials of this entry point live in a fixed array in the library's own device
// image: every GPU that loads the library holds these HK_STATIC_SCRATCH_BYTES (about 8 MiB) until
// the process exits, whether or not the function is ever called.
//
// In host code the array's name is only a handle, not a device address, so it must never be
// passed to a kernel; the address is obtained once per device with cudaGetSymbolAddress while that
// device is current.  The first call on a device does this set-up: make that first call outside
// any stream capture.  All calls on a device share the one array and it keeps whatever the last
// call left in it; nothing in it needs to start at zero because every launch rewrites every
// (m, l, acc) slot it later reads, but two calls that overlap on the GPU (different streams,
// no ordering between them) would overwrite each other's partials: order them.
// ---------------------------------------------------------------------------------------------
constexpr size_t HK_STATIC_MAX_SLOTS = 64;   // n_split * m must not exceed this
constexpr size_t HK_STATIC_SCRATCH_BYTES = 2 * ((HK_STATIC_MAX_SLOTS * 64 * sizeof(float) + 255) / 256 * 256) +
                                           HK_STATIC_MAX_SLOTS * 64 * hk::LATENT * sizeof(float);
static __device__ __align__(256) unsigned char hk_static_scratch[HK_STATIC_SCRATCH_BYTES];

static void* static_scratch_address(int* status) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *status = HK_ERR_CUDA;
    return nullptr;
  }
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, hk_static_scratch) != cudaSuccess || !p) {
      *status = HK_ERR_CUDA;
      return nullptr;
    }
    cached[dev] = p;
  }
  *status = HK_OK;
  return cached[dev];
}

HK_API size_t hk_mla_sparse_static_max_slots(void) { return HK_STATIC_MAX_SLOTS; }

HK_API int hk_mla_sparse_static(const void* q_lat, const void* ckv, const int* raw_idx, int kidx,
                                void* lat_out, int m, float scale, int n_split, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv && raw_idx && lat_out && m >= 0 && kidx >= 0);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv, 16) && aligned(lat_out, 16));
  if (m == 0) return HK_OK;
  if ((size_t)m > HK_STATIC_MAX_SLOTS) return HK_ERR_WORKSPACE;  // beyond the built-in scratch: use hk_mla_sparse
  if (n_split <= 0) {
    n_split = force_simt() ? simt_auto_splits(m, 64, kidx) : mla_flash_tc_auto_splits(m, kidx);
    const int cap = (int)(HK_STATIC_MAX_SLOTS / (size_t)m);
    if (n_split > cap) n_split = cap;
  }
  if ((size_t)n_split * (size_t)m > HK_STATIC_MAX_SLOTS) return HK_ERR_WORKSPACE;
  int st = HK_OK;
  void* scratch = static_scratch_address(&st);
  if (st != HK_OK) return st;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv;
  a.raw_idx = raw_idx; a.kidx = kidx;
  a.m = m; a.n_heads = 64; a.scale = scale;
  a.out = (__half*)lat_out;
  return attend(a, kidx, n_split, scratch, HK_STATIC_SCRATCH_BYTES, as_stream(stream));
}

HK_API int hk_mla_dense(const void* q_lat, const void* ckv, int64_t ckv_rows, const int64_t* kv_base,
                        const int* kv_len, int pos_start, void* lat_out, int m, int n_heads,
                        float scale, int n_split, void* workspace, size_t workspace_bytes,
                        void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv && lat_out && ckv_rows >= 0);
  HK_REQUIRE(m >= 0 && pos_start >= 0 && n_heads > 0 && n_heads % SIMT_HG == 0);
  // causal form (no per-row arrays): the last row attends rows 0 .. pos_start + m - 1, which must exist
  if (ckv_rows > 0 && !kv_base && !kv_len) HK_REQUIRE((int64_t)pos_start + m <= ckv_rows);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv, 16) && aligned(lat_out, 16));
  if (m == 0) return HK_OK;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv; a.ckv_rows = ckv_rows;
  a.kv_base = kv_base; a.kv_len = kv_len; a.pos_start = pos_start;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  a.out = (__half*)lat_out;
  // without host-visible lengths the split heuristic uses the longest causal row
  const int hint = kv_len ? (pos_start > 0 ? pos_start : 4096) : pos_start + m;
  return attend(a, hint, n_split, workspace, workspace_bytes, as_stream(stream));
}

HK_API int hk_mla_dense_partial(const void* q_lat, const void* ckv, const int64_t* kv_base,
                                const int* kv_len, int pos_start, float* part_m, float* part_l,
                                float* part_acc, int m, int n_heads, float scale, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv && part_m && part_l && part_acc);
  HK_REQUIRE(m >= 0 && n_heads > 0 && n_heads % SIMT_HG == 0);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv, 16) && aligned(part_acc, 16));
  if (m == 0) return HK_OK;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv;
  a.kv_base = kv_base; a.kv_len = kv_len; a.pos_start = pos_start;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  a.n_split = 1;
  a.part_m = part_m; a.part_l = part_l; a.part_acc = part_acc;
  int st = HK_ERR_UNSUPPORTED;
  if (n_heads == 64 && !force_simt()) st = mla_flash_tc_launch(a, as_stream(stream));
  if (st == HK_ERR_UNSUPPORTED) st = launch_simt(a, as_stream(stream));
  return st;
}

HK_API int hk_mla_dense_partial_ws(const void* q_lat, const void* ckv, const int64_t* kv_base,
                                   const int* kv_len, int pos_start, float* part_m, float* part_l,
                                   float* part_acc, int m, int n_heads, float scale, int n_split,
                                   int n_keys_hint, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv && part_m && part_l && part_acc);
  HK_REQUIRE(m >= 0 && n_heads > 0 && n_heads % SIMT_HG == 0);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv, 16) && aligned(part_acc, 16));
  if (m == 0) return HK_OK;
  const bool tc = (n_heads == 64) && !force_simt();
  if (n_split <= 0)
    n_split = tc ? mla_flash_tc_auto_splits(m, n_keys_hint > 0 ? n_keys_hint : 4096)
                 : simt_auto_splits(m, n_heads, n_keys_hint > 0 ? n_keys_hint : 4096);
  if (n_split == 1)
    return hk_mla_dense_partial(q_lat, ckv, kv_base, kv_len, pos_start, part_m, part_l, part_acc, m, n_heads, scale, stream);
  const int64_t rows = (int64_t)m * n_heads;
  PartialLayout pl = partial_layout(n_split, rows);
  if (!workspace || workspace_bytes < pl.total) return HK_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return HK_ERR_INVALID;
  char* ws = (char*)workspace;
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv;
  a.kv_base = kv_base; a.kv_len = kv_len; a.pos_start = pos_start;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  a.n_split = n_split;
  a.part_m = (float*)ws; a.part_l = (float*)(ws + pl.off_l); a.part_acc = (float*)(ws + pl.off_acc);
  cudaStream_t s = as_stream(stream);
  int st = HK_ERR_UNSUPPORTED;
  if (tc) st = mla_flash_tc_launch(a, s);
  if (st == HK_ERR_UNSUPPORTED) st = launch_simt(a, s);
  if (st != HK_OK) return st;
  if (n_split > LSE_MAX_SPLITS) return HK_ERR_UNSUPPORTED;
  lse_merge_partials_kernel<<<(unsigned)rows, LSE_THREADS, 0, s>>>(a.part_m, a.part_l, a.part_acc, n_split, rows,
                                                           part_m, part_l, part_acc, nullptr, nullptr, nullptr, nullptr);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_lse_combine(const float* part_m, const float* part_l, const float* part_acc,
                          int n_split, int64_t rows, void* out_f16, void* stream) {
  using namespace hk;
  HK_REQUIRE(part_m && part_l && part_acc && out_f16 && n_split >= 1 && rows >= 0);
  HK_REQUIRE(aligned(part_acc, 16) && aligned(out_f16, 8));
  if (rows == 0) return HK_OK;
  return combine(part_m, part_l, part_acc, n_split, rows, (__half*)out_f16, as_stream(stream));
}

HK_API int hk_lse_combine_ptrs(const float* const* ptrs_m, const float* const* ptrs_l,
                               const float* const* ptrs_acc, int n_split, int64_t rows,
                               void* out_f16, void* stream) {
  using namespace hk;
  HK_REQUIRE(ptrs_m && ptrs_l && ptrs_acc && out_f16 && n_split >= 1 && n_split <= LSE_MAX_SPLITS && rows >= 0);
  if (rows == 0) return HK_OK;
  lse_combine_kernel<true, LSE_GROUPS><<<(unsigned)rows, LSE_THREADS, 0, as_stream(stream)>>>(
      nullptr, nullptr, nullptr, ptrs_m, ptrs_l, ptrs_acc, n_split, rows, (__half*)out_f16);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_peer_signal(int* const* flag_ptrs, int n_ranks, int my_rank, int epoch, void* stream) {
  using namespace hk;
  HK_REQUIRE(flag_ptrs && n_ranks >= 1 && n_ranks <= 32 && my_rank >= 0 && my_rank < n_ranks);
  peer_signal_kernel<<<1, 32, 0, as_stream(stream)>>>(flag_ptrs, n_ranks, my_rank, epoch);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

HK_API int hk_lse_combine_peers(const float* const* ptrs_m, const float* const* ptrs_l,
                                const float* const* ptrs_acc, int n_split, int64_t rows, void* out_f16,
                                const int* local_flags, int epoch, int max_wait_ms, void* stream) {
  using namespace hk;
  HK_REQUIRE(ptrs_m && ptrs_l && ptrs_acc && out_f16 && local_flags && n_split >= 1 && n_split <= 32 && rows >= 0);
  HK_REQUIRE(max_wait_ms > 0 && max_wait_ms <= 10000);
  if (rows == 0) return HK_OK;
  const long long cycles = (long long)max_wait_ms * 2000000LL;   // ~2 GHz
  lse_combine_peers_kernel<<<(unsigned)rows, 128, 0, as_stream(stream)>>>(
      ptrs_m, ptrs_l, ptrs_acc, n_split, rows, (__half*)out_f16, local_flags, epoch, cycles,
      device_status_ptr(), nullptr);
  HK_LAUNCH_CHECK();
  return HK_OK;
}

// One split-KV decode step of one rank in ONE host call: local partial (local splits, merged), signal,
// bounded-wait combine over all ranks' partial sets.  The step number lives on the device (step_ctr,
// advanced by the signal kernel), so a captured graph of this call can be replayed: the exchange set
// written and read in step e is set e & 1, the flags carry e.
namespace hk {
// partial over this rank's slice (dense range or gathered rows), local splits merged into the exchange set of the
// step, signal, bounded-wait combine over all ranks' sets
static int splitkv_exchange(MlaArgs a, int n_split, int n_keys_hint, void* workspace, size_t workspace_bytes,
                            float* part_m0, float* part_l0, float* part_acc0, float* part_m1, float* part_l1, float* part_acc1,
                            int* const* flag_ptrs, const float* const* ptrs_m, const float* const* ptrs_l,
                            const float* const* ptrs_acc, int n_ranks, int my_rank, int* step_ctr, const int* local_flags,
                            void* out_f16, int max_wait_ms, int signal, cudaStream_t s) {
  const bool tc = (a.n_heads == 64) && !force_simt();
  if (n_split <= 0)
    n_split = tc ? mla_flash_tc_auto_splits(a.m, n_keys_hint > 0 ? n_keys_hint : 4096)
                 : simt_auto_splits(a.m, a.n_heads, n_keys_hint > 0 ? n_keys_hint : 4096);
  if (n_split > LSE_MAX_SPLITS) return HK_ERR_UNSUPPORTED;
  const int64_t rows = (int64_t)a.m * a.n_heads;
  PartialLayout pl = partial_layout(n_split, rows);
  if (workspace_bytes < pl.total) return HK_ERR_WORKSPACE;
  char* ws = (char*)workspace;
  a.n_split = n_split;
  a.part_m = (float*)ws; a.part_l = (float*)(ws + pl.off_l); a.part_acc = (float*)(ws + pl.off_acc);
  int st = HK_ERR_UNSUPPORTED;
  if (tc) st = mla_flash_tc_launch(a, s);
  if (st == HK_ERR_UNSUPPORTED) st = launch_simt(a, s);
  if (st != HK_OK) return st;
  lse_merge_partials_kernel<<<(unsigned)rows, LSE_THREADS, 0, s>>>(a.part_m, a.part_l, a.part_acc, n_split, rows, part_m0, part_l0,
                                                           part_acc0, part_m1, part_l1, part_acc1, step_ctr);
  HK_LAUNCH_CHECK();
  peer_signal_ctr_kernel<<<1, 32, 0, s>>>(flag_ptrs, n_ranks, my_rank, step_ctr, signal);
  HK_LAUNCH_CHECK();
  lse_combine_peers_kernel<<<(unsigned)rows, 128, 0, s>>>(ptrs_m, ptrs_l, ptrs_acc, n_ranks, rows, (__half*)out_f16, local_flags,
                                                          0, (long long)max_wait_ms * 2000000LL, device_status_ptr(), step_ctr);
  HK_LAUNCH_CHECK();
  return HK_OK;
}
}  // namespace hk

HK_API int hk_mla_splitkv_step(const void* q_lat, const void* ckv_shard, const int64_t* kv_base, const int* kv_len,
                               float* part_m0, float* part_l0, float* part_acc0, float* part_m1, float* part_l1,
                               float* part_acc1, int m, int n_heads, float scale, int n_split, int n_keys_hint,
                               void* workspace, size_t workspace_bytes, int* const* flag_ptrs,
                               const float* const* ptrs_m, const float* const* ptrs_l, const float* const* ptrs_acc,
                               int n_ranks, int my_rank, int* step_ctr, const int* local_flags, void* out_f16,
                               int max_wait_ms, int signal, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv_shard && part_m0 && part_l0 && part_acc0 && part_m1 && part_l1 && part_acc1);
  HK_REQUIRE(flag_ptrs && ptrs_m && ptrs_l && ptrs_acc && step_ctr && local_flags && out_f16 && workspace);
  HK_REQUIRE(m > 0 && n_heads > 0 && n_heads % SIMT_HG == 0 && n_ranks >= 1 && n_ranks <= 32 && my_rank >= 0 && my_rank < n_ranks);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv_shard, 16) && aligned(part_acc0, 16) && aligned(part_acc1, 16) && aligned(workspace, 256));
  HK_REQUIRE(max_wait_ms > 0 && max_wait_ms <= 10000);
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv_shard;
  a.kv_base = kv_base; a.kv_len = kv_len; a.pos_start = 0;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  return splitkv_exchange(a, n_split, n_keys_hint, workspace, workspace_bytes, part_m0, part_l0, part_acc0, part_m1, part_l1,
                          part_acc1, flag_ptrs, ptrs_m, ptrs_l, ptrs_acc, n_ranks, my_rank, step_ctr, local_flags, out_f16,
                          max_wait_ms, signal, as_stream(stream));
}

// The same step over GATHERED rows of this rank's slice (sparse split-KV): raw_local [m][kidx] holds row numbers
// relative to the slice, negative = not on this rank (skipped); a rank without any selected row contributes an
// empty partial (m = -inf, l = 0), which the combine weighs with zero.
HK_API int hk_mla_splitkv_sparse_step(const void* q_lat, const void* ckv_shard, int64_t ckv_rows, const int* raw_local, int kidx,
                                      float* part_m0, float* part_l0, float* part_acc0, float* part_m1, float* part_l1,
                                      float* part_acc1, int m, int n_heads, float scale, int n_split,
                                      void* workspace, size_t workspace_bytes, int* const* flag_ptrs,
                                      const float* const* ptrs_m, const float* const* ptrs_l, const float* const* ptrs_acc,
                                      int n_ranks, int my_rank, int* step_ctr, const int* local_flags, void* out_f16,
                                      int max_wait_ms, int signal, void* stream) {
  using namespace hk;
  HK_REQUIRE(q_lat && ckv_shard && raw_local && part_m0 && part_l0 && part_acc0 && part_m1 && part_l1 && part_acc1);
  HK_REQUIRE(flag_ptrs && ptrs_m && ptrs_l && ptrs_acc && step_ctr && local_flags && out_f16 && workspace);
  HK_REQUIRE(m > 0 && kidx >= 0 && ckv_rows >= 0 && n_heads > 0 && n_heads % SIMT_HG == 0);
  HK_REQUIRE(n_ranks >= 1 && n_ranks <= 32 && my_rank >= 0 && my_rank < n_ranks);
  HK_REQUIRE(aligned(q_lat, 16) && aligned(ckv_shard, 16) && aligned(part_acc0, 16) && aligned(part_acc1, 16) && aligned(workspace, 256));
  HK_REQUIRE(max_wait_ms > 0 && max_wait_ms <= 10000);
  MlaArgs a{};
  a.q_lat = (const __half*)q_lat; a.ckv = (const __half*)ckv_shard; a.ckv_rows = ckv_rows;
  a.raw_idx = raw_local; a.kidx = kidx;
  a.m = m; a.n_heads = n_heads; a.scale = scale;
  return splitkv_exchange(a, n_split, kidx, workspace, workspace_bytes, part_m0, part_l0, part_acc0, part_m1, part_l1,
                          part_acc1, flag_ptrs, ptrs_m, ptrs_l, ptrs_acc, n_ranks, my_rank, step_ctr, local_flags, out_f16,
                          max_wait_ms, signal, as_stream(stream));
}


#include "mla_splitkv_heads.cuh"
