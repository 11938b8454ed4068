/* helios_b200.h — C ABI of libhelios_b200.so
 *
 * sm_100a (B200) implementation of the GLM-5.3-Flash trunk-attention hot path of the Helios engine:
 * KDA (short conv, recurrent decode, chunked prefill), absorbed MLA over the 512-wide fp16 latent
 * cache (dense and sparse, decode and chunked prefill), the DSA indexer (pooled keys, scores,
 * top-k, expansion) and the split-KV log-sum-exp combine.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise;
 *   - bf16 / fp16 tensors are passed as void* (bit patterns of __nv_bfloat16 / __half);
 *   - `stream` is a cudaStream_t passed as void*; every call is asynchronous on that stream;
 *   - nothing is allocated, freed or synchronised behind the caller's back: scratch memory is
 *     caller-provided and sized by the *_workspace_bytes() queries;
 *   - every function returns an hk_status (0 = ok).  Argument errors are detected on the host
 *     before any launch.  The reference's launchers return void and abort() on precondition
 *     failure; the C++ shim (helios_b200_shim.hpp) keeps that behaviour on top of these codes.
 *
 * Each entry point names the reference interface it replaces (paths relative to the reference tree).
 */
#ifndef HELIOS_B200_H
#define HELIOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hk_status {
  HK_OK = 0,
  HK_ERR_INVALID = 1,      /* bad shape / null pointer / misaligned buffer                        */
  HK_ERR_UNSUPPORTED = 2,  /* valid request the library has no kernel for (e.g. head dim 96)      */
  HK_ERR_CUDA = 3,         /* the CUDA runtime reported an error at launch                        */
  HK_ERR_WORKSPACE = 4,    /* caller-provided workspace too small                                 */
  HK_ERR_TIMEOUT = 5       /* a bounded device-side wait expired (see hk_read_device_status)      */
} hk_status;

/* dtype tags for the entry points that accept either 16-bit float format */
enum { HK_F16 = 0, HK_BF16 = 1, HK_F32 = 2 };

const char* hk_status_string(int status);
int hk_abi_version(void);

/* ---------------------------------------------------------------------------------------------
 * (a) KDA
 * ------------------------------------------------------------------------------------------- */

/* Causal depthwise short convolution (+SiLU) with rolling window state.
 * Replaces helios::aux::cuda_causal_conv1d_update  (src/cuda/aux/gdn.cuh:67-83, gdn.cu:972-1023).
 *   x     [bsz][dim][seqlen] bf16 (channel-major)      state [slots][dim][state_size] bf16 (in place)
 *   w     [dim][K] bf16     bias [dim] bf16 or NULL    out   [bsz][seqlen][dim] bf16
 *   slots [bsz] or NULL (identity).  K <= 16, state_size >= K.                                  */
int hk_conv1d_update(const void* x, void* conv_state, const int* slots, const void* weight,
                     const void* bias, void* out, int bsz, int dim, int seqlen, int state_size,
                     int K, int activation, int history, void* stream);

/* Gated delta rule recurrence, token by token (decode, short sequences, history mode).
 * Replaces helios::aux::cuda_recurrent_gated_delta_rule (src/cuda/aux/gdn.cuh:47-65,
 * gdn.cu:760-866).  Same tensor layouts:
 *   mixed_qkv [bsz][seqlen][2*Hk*dk + Hv*dv] bf16 = q | k | v      g [bsz][seqlen][Hv][dk] f32
 *   (channelwise) or [bsz][seqlen][Hv]      beta [bsz][seqlen][Hv] bf16
 *   state [slots][history_stride][Hv][dk][dv] f32 (in place)   out [bsz][seqlen][Hv][dv] bf16 (rz)
 *   out_f32: optional (may be NULL) copy of the output before bf16 rounding, same shape.
 * Supported head dims: (dk,dv) = (128,128) and (64,64).                                          */
int hk_kda_recurrent(const void* mixed_qkv, const float* g, const void* beta, float* state,
                     void* out, float* out_f32, int bsz, int seqlen, int num_k_heads,
                     int num_v_heads, int k_head_dim, int v_head_dim, int history_stride,
                     const int* slots, int channelwise, int history, void* stream);

/* One KDA decode step with the short convolution inside: what the engine runs per decoded token as
 * cuda_causal_conv1d_update(seqlen 1, K = state_size = 4, SiLU) followed by cuda_recurrent_gated_delta_rule(seqlen 1,
 * channelwise) (src/engine/runner.cpp:443-471), in ONE launch and with the same bits.  Head dim 128, Hk == Hv.
 *   x [bsz][3*H*128] bf16 (the token's pre-conv q|k|v)   conv_state [slots][3*H*128][4] bf16 (in place)
 *   conv_weight [3*H*128][4] bf16   conv_bias [3*H*128] bf16 or NULL   g [bsz][H][128] f32   beta [bsz][H] bf16
 *   rec_state [slots][H][128][128] f32 (in place)   out [bsz][H][128] bf16 (rz)   out_f32 optional
 *   conv_out optional [bsz][3*H*128] bf16: the convolved q|k|v (what the two-kernel sequence leaves in between).
 *   tickets: bsz*H device ints, zero before the first call; every call leaves them zero (the slices of a head count
 *   themselves there to find out which one rolls the head's q / k window).  Calls that share `tickets` must not
 *   overlap on the GPU.                                                                                          */
int hk_kda_decode_step(const void* x, void* conv_state, const void* conv_weight, const void* conv_bias, const float* g,
                       const void* beta, float* rec_state, void* out, float* out_f32, void* conv_out, int bsz,
                       int num_heads, const int* slots, int* tickets, void* stream);

/* The whole KDA layer of ONE decoded token per sequence in one launch: cast of the projected row x32 [bsz][3*H*128] fp32
 * to bf16 (glue::kda_transpose_cast of one row), g = lower_bound * sigmoid(exp(a_log[h]) * (f + dt_bias)) and
 * beta = sigmoid(b) (glue::kda_gate; f [bsz][H][128] fp32, b [bsz][H] fp32), hk_kda_decode_step, and the gated RMS norm
 * of the output (hk_gated_rms_norm with w_groups 1, gate after the norm): y [bsz*H][128] of y_type (HK_F16 / HK_F32),
 * norm_w [128] of w_type (HK_F32 / HK_BF16), gate_out [bsz*H][128] of g_type (HK_F32 / HK_BF16).  `out` (bf16) and
 * out_f32 (optional) receive the recurrence output.  The reference's decode runs five launches here
 * (src/engine/runner.cpp:433-489); results are bit-identical to calling the five in turn.
 * tickets: 2 * bsz * H zeroed ints of caller memory, left zeroed; calls sharing them must not overlap on the GPU.   */
int hk_kda_decode_layer(const float* x32, void* conv_state, const void* conv_weight, const void* conv_bias, const float* f,
                        const float* b, const float* dt_bias, const float* a_log, float lower_bound, float* rec_state,
                        void* out, float* out_f32, const void* norm_w, int w_type, const void* gate_out, int g_type, void* y,
                        int y_type, float epsilon, float constant_bias, int gate_act, int bsz, int num_heads,
                        const int* slots, int* tickets, void* stream);

/* Chunked (64-token) KDA prefill on the tensor cores; numerically equivalent to
 * hk_kda_recurrent(channelwise=1, history=0) on the same arguments (the reference has no chunked
 * kernel: prefill calls the recurrence with seqlen = n, src/engine/runner.cpp:468-471).
 * Requires dk = dv = 128, Hk == Hv.  seqlen may be any positive length (a ragged tail shorter
 * than a chunk is processed by the same kernels).  `workspace` must hold at least
 * hk_kda_chunked_workspace_bytes(bsz, seqlen, num_heads) bytes, 256-byte aligned.
 * Two forms.  ONE persistent cooperative launch when the chains fit its chain CTAs (at most 48 chains: a chain per SM;
 * more chains when a number of chain CTAs in [16, 48] divides their count, e.g. 64 heads or 8 x 32: a chain CTA then
 * walks several chains one after the other); the other SMs prepare the chunks and hand them over through a ring of 16
 * chunk slots per chain CTA (workspace = chain CTAs * 16 * 74,240 B + flags, independent of seqlen; it stays in L2).
 * Other calls run as two kernels with one 74,240-byte workspace unit per (batch, head, chunk).
 * hk_kda_chunked_set_form(1) selects the two-kernel form for every later call and workspace query of this
 * process, hk_kda_chunked_set_form(0) the automatic choice (default).                              */
int hk_kda_chunked_set_form(int form);
/* The rule by which the launcher of the reference's name (helios::aux::cuda_recurrent_gated_delta_rule in the C++
 * layer, the Python wrapper of the same name) sends a call to the chunked kernels (1) or to hk_kda_recurrent (0).  */
int hk_kda_dispatch_is_chunked(int seqlen, int num_k_heads, int num_v_heads, int k_head_dim, int v_head_dim,
                               int history_stride, int channelwise, int history);
size_t hk_kda_chunked_workspace_bytes(int bsz, int seqlen, int num_heads);
int hk_kda_chunked_prefill(const void* mixed_qkv, const float* g, const void* beta, float* state,
                           void* out, float* out_f32, int bsz, int seqlen, int num_heads,
                           const int* slots, void* workspace, size_t workspace_bytes,
                           void* stream);

/* The same prefill with the gate preparation inside the first kernel: `f` [bsz][seqlen][H][128] f32 is the
 * raw gate projection and `b` [bsz][seqlen][H] f32 the raw beta logit;
 *   g = lower_bound * sigmoid(exp(a_log[h]) * (f + dt_bias[h][d])),  beta = bf16(sigmoid(b))
 * are formed on the fly, so the fp32 gate tensor of helios::glue::kda_gate (src/engine/glue2.cuh:62-63,
 * glue2.cu:347-368) is neither written nor read back.  Results equal hk_kda_gate followed by
 * hk_kda_chunked_prefill, bit for bit.  dt_bias [H][128] f32 (16-byte aligned), a_log [H] f32.      */
int hk_kda_chunked_prefill_gated(const void* mixed_qkv, const float* f, const float* b,
                                 const float* dt_bias, const float* a_log, float lower_bound,
                                 float* state, void* out, float* out_f32, int bsz, int seqlen,
                                 int num_heads, const int* slots, void* workspace,
                                 size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (a') producers and consumer either side of the KDA recurrence
 * ------------------------------------------------------------------------------------------- */

/* dst[f][s] = bf16(src[s][f]): token-major fp32 projection output -> channel-major conv input.
 * Replaces helios::glue::kda_transpose_cast (src/engine/glue2.cuh:61, glue2.cu:318-344).          */
int hk_kda_transpose_cast(void* dst_bf16, const float* src, int S, int F, void* stream);

/* beta[s][h] = bf16(sigmoid(b[s][h]));  g[s][h][d] = lower_bound * sigmoid(exp(a_log[h]) * (f[s][h][d] +
 * dt_bias[h][d])).  Replaces helios::glue::kda_gate (src/engine/glue2.cuh:62-63, glue2.cu:347-368). */
int hk_kda_gate(const float* b, const float* f, const float* dt_bias, const float* a_log,
                float lower_bound, void* beta_bf16, float* g, int S, int H, int Dk, void* stream);

/* Both of the above in one call.  Replaces helios::glue::kda_prepare (src/engine/glue2.cuh:64-67,
 * glue2.cu:370-404).                                                                              */
int hk_kda_prepare(const float* qkv, const float* b, const float* f, const float* dt_bias,
                   const float* a_log, float lower_bound, void* mixed_qkv_bf16, void* beta_bf16,
                   float* g, int S, int F, int H, int Dk, void* stream);

/* Cast + short convolution (window 4) in one pass over the TOKEN-major fp32 projection output, i.e.
 * hk_kda_transpose_cast followed by hk_conv1d_update(K = 4, state_size = 4, history = 0) without the
 * transposed intermediate; same bits.   x [bsz][seqlen][dim] f32 (16-byte aligned, dim % 4 == 0)
 * state [slots][dim][4] bf16 (in place)   w [dim][4] bf16   bias [dim] bf16 or NULL
 * out [bsz][seqlen][dim] bf16.                                                                    */
int hk_kda_cast_conv(const float* x, void* conv_state, const int* slots, const void* weight,
                     const void* bias, void* out, int bsz, int dim, int seqlen, int activation,
                     void* stream);

/* y = x * w * rsqrt(mean(x^2) + epsilon) * act(g) per row of `dim` channels (gate_first: the gate is
 * applied to x before the norm).  Replaces helios::aux::gated_rms_norm (src/cuda/aux/norm.cuh:71-87,
 * norm.cu:294-468).  x bf16; w_type HK_F32 / HK_BF16 ([w_groups][dim], row r uses w[r % w_groups]);
 * y_type HK_F16 / HK_F32; g_type HK_BF16 / HK_F32; gate_act 0 = SiLU, 1 = sigmoid; dim % 4 == 0.     */
int hk_gated_rms_norm(const void* x, const void* w, int w_type, void* y, int y_type, const void* g,
                      int g_type, long long rows, int dim, float epsilon, float constant_bias,
                      int w_groups, int gate_first, int gate_act, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (c) DSA indexer
 * ------------------------------------------------------------------------------------------- */

/* Ring write of k||gate rows and pooling of every 4-token group completed by this call.
 * Replaces helios::attn::kpool_write (src/cuda/attn/attn.cuh:74-87, attn.cu:332-390).          */
int hk_kpool_write(const void* idx_k, const void* idx_g, void* raw_ring, int raw_rows,
                   void* pool_k_nt, const float* ape, int pos_start, int n_new, void* stream);

/* scores[r][p] = n_heads^-1/2 * sum_h w[r][h] * relu(128^-1/2 * q[r][h] . pool_k[p]),
 * -inf where 4p+3 > q_pos[r].  Replaces helios::attn::indexer_score / indexer_score_mma
 * (src/cuda/attn/attn.cuh:44-55, attn.cu:182-273).  Tensor-core (tcgen05) kernel.
 *   q_idx [m][n_heads][128], pool_k_nt [npools][128], w [m][n_heads]: fp16 or bf16 (`dtype`);
 *   scores [m][score_stride] fp16.  n_heads must be 32.                                         */
int hk_indexer_score(const void* q_idx, const void* pool_k_nt, const void* w, const int* q_pos,
                     void* scores, int m, int npools, int score_stride, int n_heads, int dtype,
                     void* stream);

/* Scalar cross-check kernel reading the transposed [128][pk_stride] plane.
 * Replaces helios::attn::indexer_score_legacy (src/cuda/attn/attn.cu:134-158, :275-280).        */
int hk_indexer_score_legacy(const void* q_idx, const void* pool_k, const void* w, const int* q_pos,
                            void* scores, int m, int npools, int pk_stride, void* stream);

/* Exact top-k over fp16 score rows: every entry above the k-th value in ascending index order,
 * then ties with the k-th value in ascending index order, -1 padding up to k_pad; -inf is never
 * selected.  Replaces helios::aux::dsa_topk (src/cuda/aux/dsa_topk.cuh:15-27, dsa_topk.cu:668-732).
 * If t_ptr != NULL: T = t_seq > 0 ? t_ptr[row / t_seq] : t_ptr[0] (device override, as there).   */
int hk_dsa_topk(const void* scores, int s_stride, int* indices, int R, int T, int k, int k_pad,
                const int* t_ptr, int t_seq, void* stream);

/* hk_dsa_topk with hk_pool_expand folded into the output writes: indices [R][512] as hk_dsa_topk (k_pad = 512) AND
 * raw_idx [R][2052] as hk_pool_expand(indices, q_pos) would give, in one kernel.  after_scorer != 0: the kernel is
 * launched as a programmatic dependent of the kernel before it in the stream (use only directly behind
 * hk_indexer_score of at most 8 rows, which releases its dependents early).                                       */
int hk_dsa_topk_expand(const void* scores, int s_stride, int* indices, int* raw_idx, const int* q_pos, int R, int T,
                       int k, int after_scorer, void* stream);

/* Decode-step selection in one call: hk_indexer_score into `scores` (workspace, [m][score_stride] fp16), then
 * hk_dsa_topk_expand behind it.  Two launches where the reference's decode runs indexer_score, dsa_topk and
 * pool_expand_row (src/engine/runner.cpp:620-630).  Arguments as in those calls; k <= 512.                        */
int hk_indexer_select(const void* q_idx, const void* pool_k_nt, const void* w, const int* q_pos, void* scores,
                      int* indices, int* raw_idx, int m, int npools, int score_stride, int n_heads, int dtype, int k,
                      void* stream);

/* Pool index -> token index expansion plus the 4 tail tokens, clipped to the row's position.
 * Replaces helios::attn::pool_expand_row (q_pos != NULL) and helios::attn::pool_expand
 * (q_pos == NULL, cur_pos used for every row)  (src/cuda/attn/attn.cuh:57-72, attn.cu:284-327).
 *   pool_idx [m][n_sel], raw_idx [m][4*n_sel + 4]                                               */
int hk_pool_expand(const int* pool_idx, const int* q_pos, int* raw_idx, int m, int cur_pos,
                   int n_sel, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (b) absorbed MLA, (d) split-KV combine
 * ------------------------------------------------------------------------------------------- */

/* Partial format of a split: for every (row, head) a running max m, a sum l = sum exp(s - m) and an
 * un-normalised accumulator acc[512] = sum exp(s - m) * latent.  A workspace for n_split splits of
 * `rows` (row, head) pairs is laid out as  m[n_split][rows] f32 | l[n_split][rows] f32 |
 * acc[n_split][rows][512] f32, i.e. n_split * rows * 2056 bytes (+ alignment).                  */
size_t hk_mla_partial_bytes(int n_split, int64_t rows);

/* Number of KV splits the library would pick for a launch with `m` query rows attending `n_keys`
 * keys each (so that the grid covers the GPU); 1 means no workspace is needed.                  */
int hk_mla_auto_splits(int m, int n_keys);

/* Sparse (gathered) attention: row r attends ckv[raw_idx[r][i]] for every i < kidx with
 * raw_idx >= 0 (duplicates count twice; all skipped -> zeros).
 * Replaces helios::attn::mla_sparse_decode (src/cuda/attn/attn.cuh:89-99, attn.cu:394-617) with an
 * explicit softmax scale and head count (the reference pins 0.0625 and 64).
 *   q_lat [m][n_heads][512] f16, ckv [ckv_rows][512] f16, lat_out [m][n_heads][512] f16.
 * ckv_rows: rows the cache buffer holds; row numbers at or beyond it are treated as holes instead of being read
 * (0 = not told, as in the reference's signature: every non-negative row number is read).
 * n_split = 0 lets the library choose; workspace may be NULL when the choice is 1.             */
int hk_mla_sparse(const void* q_lat, const void* ckv, int64_t ckv_rows, const int* raw_idx, int kidx, void* lat_out,
                  int m, int n_heads, float scale, int n_split, void* workspace,
                  size_t workspace_bytes, void* stream);

/* Sparse MLA decode that allocates nothing and takes no workspace: the split partials live in a
 * fixed ~8 MiB array inside the library's device image (held by every GPU that loads the library
 * until exit).  For hosts that cannot call an allocator at this point - an engine that owns all
 * device memory through its own start-up arena and whose launcher signatures have no scratch
 * argument, or code that must not enter the CUDA allocator.  It has no counterpart in the reference.
 * Same arguments and result as hk_mla_sparse with n_heads = 64.  Limit: n_split * m <= 64
 * (hk_mla_sparse_static_max_slots()); larger requests return HK_ERR_WORKSPACE - use hk_mla_sparse
 * with caller memory instead.  n_split = 0 picks a split count that fits.  The first call on a
 * device looks the array's address up (make it outside stream capture); calls on one device share
 * the array, so calls that overlap on the GPU race.                                               */
size_t hk_mla_sparse_static_max_slots(void);
int hk_mla_sparse_static(const void* q_lat, const void* ckv, const int* raw_idx, int kidx,
                         void* lat_out, int m, float scale, int n_split, void* stream);

/* Dense causal attention: row r attends ckv[kv_base[r] .. kv_base[r] + kv_len[r]).
 * With kv_base == NULL and kv_len == NULL: base 0 and len = pos_start + r + 1, which is
 * helios::attn::mla_dense_prefill (src/cuda/attn/attn.cuh:101-108, attn.cu:621-699); qlen = 1 is
 * dense decode, and per-row base/len arrays give batched decode over concatenated caches.
 * ckv_rows: rows the cache buffer holds (0 = not told).  With it the causal form is checked on the host
 * (pos_start + m <= ckv_rows, else HK_ERR_INVALID), per-row ranges are cut at the end of the cache on the device, and
 * the copy engine's tensor map gets the real extent, so that nothing past the buffer is read.               */
int hk_mla_dense(const void* q_lat, const void* ckv, int64_t ckv_rows, const int64_t* kv_base, const int* kv_len,
                 int pos_start, void* lat_out, int m, int n_heads, float scale, int n_split,
                 void* workspace, size_t workspace_bytes, void* stream);

/* Same two, but writing un-normalised split partials only (no combine): the building block of
 * split-KV across GPUs.  part_* point at storage for ONE split: m[rows], l[rows], acc[rows][512]. */
int hk_mla_dense_partial(const void* q_lat, const void* ckv, const int64_t* kv_base,
                         const int* kv_len, int pos_start, float* part_m, float* part_l,
                         float* part_acc, int m, int n_heads, float scale, void* stream);

/* The same single partial set, computed with n_split splits over this GPU's SMs (workspace as for
 * hk_mla_dense: hk_mla_partial_bytes(n_split, m*n_heads)) and merged on the GPU, so that a rank of a
 * multi-GPU split-KV decode uses every SM yet exports only one (m, l, acc) set.  n_split = 0: the
 * library picks from n_keys_hint (keys per row on this GPU).                                     */
int hk_mla_dense_partial_ws(const void* q_lat, const void* ckv, const int64_t* kv_base,
                            const int* kv_len, int pos_start, float* part_m, float* part_l,
                            float* part_acc, int m, int n_heads, float scale, int n_split,
                            int n_keys_hint, void* workspace, size_t workspace_bytes, void* stream);

/* Log-sum-exp combine of n_split partials (layout above; the three arrays may live anywhere,
 * split stride = `rows` elements for m/l and rows*512 for acc).
 * Restates the in-kernel merge src/cuda/attn/attn.cu:462-481 as a standalone kernel.           */
int hk_lse_combine(const float* part_m, const float* part_l, const float* part_acc, int n_split,
                   int64_t rows, void* out_f16, void* stream);

/* Combine where split s lives at the s-th pointer of device arrays (e.g. peer-mapped buffers of
 * other GPUs, read with plain loads over NVLink).  ptrs_* are DEVICE arrays of n_split pointers. */
int hk_lse_combine_ptrs(const float* const* ptrs_m, const float* const* ptrs_l,
                        const float* const* ptrs_acc, int n_split, int64_t rows, void* out_f16,
                        void* stream);

/* Split-KV across GPUs (one process per GPU, partial buffers and flag arrays mapped into every
 * peer).  After its hk_mla_dense_partial, rank g calls hk_peer_signal: it stores `epoch` into slot g
 * of every rank's flag array (flag_ptrs: DEVICE array of n_ranks pointers to int[n_ranks]).
 * hk_lse_combine_peers then waits on THIS GPU's flag array until all n_split slots have reached
 * `epoch` - a bounded wait of at most max_wait_ms (1..10000); on expiry nothing is written and the
 * device status word reports HK_ERR_TIMEOUT - and combines the partial sets through their pointers
 * with plain loads over NVLink.  Epochs must increase from call to call; flags are never reset.
 * No counterpart in the reference (it is single-GPU for this path).                              */
int hk_peer_signal(int* const* flag_ptrs, int n_ranks, int my_rank, int epoch, void* stream);

/* One split-KV decode step of one rank in one call: the partial over this rank's shard (n_split local
 * splits in `workspace`, merged on the GPU) into exchange set (step & 1) of its region, the signal
 * (withheld when signal == 0: failure injection in tests), the bounded-wait combine.  The step number
 * lives in device memory (step_ctr, one int of this rank, zero at set-up, advanced by the call), so a
 * CUDA graph that captured this call can be replayed.  part_*0 / part_*1: the two exchange sets of THIS
 * rank; ptrs_*: DEVICE arrays of 2 * n_ranks pointers, [set][rank]; other arguments as in
 * hk_mla_dense_partial_ws, hk_peer_signal and hk_lse_combine_peers.                               */
int hk_mla_splitkv_step(const void* q_lat, const void* ckv_shard, const int64_t* kv_base, const int* kv_len,
                        float* part_m0, float* part_l0, float* part_acc0, float* part_m1, float* part_l1,
                        float* part_acc1, int m, int n_heads, float scale, int n_split, int n_keys_hint,
                        void* workspace, size_t workspace_bytes, int* const* flag_ptrs,
                        const float* const* ptrs_m, const float* const* ptrs_l, const float* const* ptrs_acc,
                        int n_ranks, int my_rank, int* step_ctr, const int* local_flags, void* out_f16,
                        int max_wait_ms, int signal, void* stream);

/* Sparse split-KV decode across GPUs (one sequence, pools and cache rows split over the ranks), selection part.
 * Rank g has scored ITS pools (hk_indexer_score with q_pos made relative to its slice): scores [m][s_stride] fp16,
 * n_local_pools valid entries per row, the first being global pool pool_base.  The call takes the local top-k
 * (local_idx [m][512], scratch), stores the k candidates (score bits + global pool index, ascending index) into every
 * rank's candidate area, waits (bounded by max_wait_ms) for all ranks' candidates of the step, selects the k best of
 * the n_ranks * k candidates with the selection rule of hk_dsa_topk (the result equals hk_dsa_topk over the whole
 * row: an entry the whole-row selection takes is always among its rank's local top-k), and writes
 *   sel_pools [m][512]   global pool indices, -1 padded (may be NULL),
 *   raw_local [m][2052]  cache rows RELATIVE to this rank's slice [row_base, row_base + n_local_rows), -1 for rows of
 *                        other ranks, pool rows past q_pos[row] and padding; the 4 tail rows q_pos - 3 .. q_pos are
 *                        appended as hk_pool_expand does.  Feed it to hk_mla_splitkv_sparse_step.
 * cand_bases: DEVICE array of n_ranks addresses of the ranks' candidate areas (hk_dsa_select_region_bytes(m, n_ranks)
 * bytes each, zeroed, inside peer-mapped regions) as mapped in THIS process; local_cand_base == cand_bases[my_rank].
 * The step number is *step_ctr + 1 (the counter that hk_mla_splitkv_sparse_step advances), the candidate sets are
 * double buffered by its parity.  On a time-out nothing is written and the device status reports HK_ERR_TIMEOUT.
 * signal == 0 withholds this rank's flag (failure injection in tests).  k <= 512, n_ranks <= 8.  phases: 3 = the whole
 * call; 1 = local top-k and publication only, 2 = wait and selection only (two calls, e.g. several ranks' regions
 * driven by one process in turn).
 * Selection semantics: helios::aux::dsa_topk (src/cuda/aux/dsa_topk.cu:179-267); no multi-GPU counterpart there.  */
size_t hk_dsa_select_region_bytes(int m, int n_ranks);
int hk_dsa_select_splitkv(const void* scores, int s_stride, int n_local_pools, int pool_base, int* local_idx,
                          void* const* cand_bases, const void* local_cand_base, int n_ranks, int my_rank, int m, int k,
                          const int* q_pos, int row_base, int n_local_rows, int* sel_pools, int* raw_local,
                          const int* step_ctr, int max_wait_ms, int signal, int phases, void* stream);

/* hk_mla_splitkv_step over GATHERED rows of this rank's slice: raw_local [m][kidx] (negative = skipped),
 * ckv_rows = rows in ckv_shard (larger indices are skipped).  A rank without any selected row contributes an empty
 * partial.  All other arguments as in hk_mla_splitkv_step.                                                         */
int hk_mla_splitkv_sparse_step(const void* q_lat, const void* ckv_shard, int64_t ckv_rows, const int* raw_local, int kidx,
                               float* part_m0, float* part_l0, float* part_acc0, float* part_m1, float* part_l1,
                               float* part_acc1, int m, int n_heads, float scale, int n_split,
                               void* workspace, size_t workspace_bytes, int* const* flag_ptrs,
                               const float* const* ptrs_m, const float* const* ptrs_l, const float* const* ptrs_acc,
                               int n_ranks, int my_rank, int* step_ctr, const int* local_flags, void* out_f16,
                               int max_wait_ms, int signal, void* stream);

/* Split-KV across GPUs with the combine sharded by heads (n_heads = 64, 64 % n_ranks == 0): one decode step of one rank
 * in one call.  Every rank owns an exchange region of hk_splitkv_region_bytes(m, n_heads) bytes (zeroed; allocate it
 * with hk_peer_region_alloc) that every peer has mapped; region_ptrs is a DEVICE array of the n_ranks region addresses
 * as mapped in THIS process, my_region == region_ptrs[my_rank].  The step: partial over this rank's shard (n_split
 * local splits in `workspace`, sized by hk_mla_partial_bytes), merged into the region and signalled; rank g combines
 * heads [g*64/n_ranks, (g+1)*64/n_ranks) from all ranks' partials and stores the fp16 rows into every rank's region;
 * once all slices have arrived they are copied to out_f16 [m][64][512].  The step number lives in the region, so a
 * CUDA graph that captured the call can be replayed.  Every wait is bounded by max_wait_ms (1..10000): on expiry the
 * grid writes nothing, the device status word reports HK_ERR_TIMEOUT, and the ranks must stop stepping until every
 * rank has called hk_splitkv_region_reset between two host-side barriers.  signal == 0 withholds this rank's first
 * signal (failure injection in tests).  No counterpart in the reference (it is single-GPU for this path).           */
size_t hk_splitkv_region_bytes(int m, int n_heads);
int hk_splitkv_region_reset(void* region, int m, int n_heads, void* stream);
int hk_mla_splitkv_heads_step(const void* q_lat, const void* ckv_shard, const int64_t* kv_base, const int* kv_len,
                              int m, int n_heads, float scale, int n_split, int n_keys_hint, void* workspace,
                              size_t workspace_bytes, void* const* region_ptrs, int n_ranks, int my_rank,
                              void* my_region, void* out_f16, int max_wait_ms, int signal, void* stream);

/* Enables access from kernels of the current device to memory of `peer_device` (needed once per peer
 * before the two calls around this one touch buffers of another GPU that were mapped into this
 * process).  Idempotent; HK_ERR_UNSUPPORTED when the two GPUs have no peer path.                  */
int hk_enable_peer_access(int peer_device);

/* Exchange regions of the split-KV decode.  hk_peer_region_alloc: zeroed device memory on the current
 * device plus its 64-byte inter-process handle.  hk_peer_region_open (in another process, with ITS OWN
 * device current): a pointer that kernels of that device may read and write over NVLink.  A region is
 * closed by every process that opened it before its owner frees it.                               */
int hk_peer_region_alloc(size_t bytes, void** dev_ptr, void* handle_out_64);
int hk_peer_region_open(const void* handle_64, void** dev_ptr);
int hk_peer_region_close(void* dev_ptr);
int hk_peer_region_free(void* dev_ptr);
int hk_lse_combine_peers(const float* const* ptrs_m, const float* const* ptrs_l,
                         const float* const* ptrs_acc, int n_split, int64_t rows, void* out_f16,
                         const int* local_flags, int epoch, int max_wait_ms, void* stream);

/* ---------------------------------------------------------------------------------------------
 * adjacent projections (kept so the engine's layer loop links unchanged)
 * Replace helios::attn::q_latent / q_latent_t / o_absorb / o_absorb_t / wuv_transpose
 * (src/cuda/attn/attn.cuh:24-39, attn.cu:12-130).
 * ------------------------------------------------------------------------------------------- */
int hk_q_latent(const void* q_nope, const void* kv_b, void* q_lat, int m, void* stream);
int hk_o_absorb(const void* lat_out, const void* kv_b, void* o, int m, void* stream);
int hk_wuv_transpose(const void* kv_b, void* wuv_t, void* stream);
int hk_o_absorb_t(const void* lat_out, const void* wuv_t, void* o, int nrows, void* stream);

/* ---------------------------------------------------------------------------------------------
 * (b') producers of the latent cache and of the indexer keys
 * ------------------------------------------------------------------------------------------- */

/* RMS norm of the n new compressed-KV rows, written into the latent cache at rows pos .. pos+n-1:
 *   ckv[pos + r][c] = f16(kv_pre[r][c] * ln_w[c] * rsqrt(mean_c(kv_pre[r]^2) + epsilon))
 * Replaces aux::rms_norm(float in, half weight, half out, dim 512) followed by the device copy into the
 * cache (src/engine/runner.cpp:569-572; kernel src/cuda/aux/norm.cu:16-164).  kv_pre [n][512] f32,
 * ln_w [512] f16, ckv [.][512] f16; ckv_new (optional, may be NULL) [n][512] f16 receives the same rows
 * (the reference's staging buffer).                                                              */
int hk_mla_cache_append(const float* kv_pre, const void* ln_w_f16, void* ckv, void* ckv_new,
                        long long pos, int n, float epsilon, void* stream);

/* y = (x - mean) * rsqrt(var + epsilon) * w + b per row of `dim` fp16 values (in place allowed).
 * Replaces helios::glue::layernorm_f16 (src/engine/glue2.cuh:73-75, glue2.cu:420-455).            */
int hk_layernorm_f16(const void* x, const void* w, const void* b, void* y, int rows, int dim,
                     float epsilon, void* stream);

/* Everything an MLA layer does with ONE new token before its attention, in one launch: hk_mla_cache_append of the row
 * (kv_pre [512] fp32 -> ckv[pos]), hk_layernorm_f16 of the indexer key row idx_k [128] (result also to idx_kn if not
 * NULL), hk_kpool_write of (normalised key, idx_g) at position pos (ring row, and the pooled key if pos completes its
 * pool), and *q_pos_out = pos (optional device int).  The reference's decode runs rms_norm + copy, layernorm_f16 and
 * kpool_write here (src/engine/runner.cpp:569-584); results are bit-identical to those calls in turn.           */
int hk_mla_decode_prologue(const float* kv_pre, const void* ln_w_f16, void* ckv, float eps_rms, const void* idx_k,
                           const void* knorm_w, const void* knorm_b, void* idx_kn, float eps_ln, const void* idx_g,
                           void* raw_ring, int raw_rows, void* pool_k_nt, const float* ape, int pos, int* q_pos_out,
                           void* stream);

/* ---------------------------------------------------------------------------------------------
 * diagnostics
 * ------------------------------------------------------------------------------------------- */

/* Kernels never spin without a bound: a device-side wait (mbarrier, peer flag) that expires makes the
 * kernel record HK_ERR_TIMEOUT in a per-device status word and finish.  This reads (and optionally
 * clears) that word on the current device; 0 means no wait has expired since the last reset.
 * Synchronises with the device.                                                                */
int hk_read_device_status(int* host_out, int reset);

/* Tensor-core self test: D[M][N] = A[M][K] * B (fp16 in, fp32 out) through the library's tcgen05 /
 * TMEM helper layer.  b_layout bit 0: B given as [K][N] instead of [N][K]; bit 1: A given as [K][M] instead of [M][K].
 * M in {64,128}; N multiple of 16, <= 256; K multiple of 16, <= 256.  D receives the RAW accumulator, float [128 lanes][N].
 * `status` (device int) is set to 0 on success or records which bounded wait expired.                                   */
int hk_tc05_selftest(const void* a_f16, const void* b_f16, float* d, int M, int N, int K,
                     int b_layout, int* status, void* stream);


#ifdef __cplusplus
}
#endif
#endif /* HELIOS_B200_H */
