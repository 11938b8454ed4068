// Absorbed MLA projections on the 5th-generation tensor cores: per head h
//   q_lat[r][h][0:512] = q_nope[r][h][0:256] . W_uk[h]        (helios::attn::q_latent / q_latent_t)
//   o[r][h][0:256]     = lat_out[r][h][0:512] . W_uv[h]^T     (helios::attn::o_absorb / o_absorb_t)
// with kv_b the raw [64*512][512] fp16 tensor (rows h*512 .. +255 = W_uk[h], +256 .. +511 = W_uv[h]);
// reference: src/cuda/attn/attn.cu:12-130 (one block per (row, head), the head's weights re-read per row).
//
// One kernel, a batched GEMM D[128 rows x 256] = A[128 x K] B[K x 256] per CTA (grid = N tiles x row tiles
// x heads): K runs in chunks of 64 through a 3-stage ring of TMA tensor copies (128-byte-swizzle boxes:
// A [128 rows][64 k]; B either [64 k][256 n] with n contiguous - W_uk, transposed W_uv - or [256 n][64 k]
// with k contiguous - raw W_uv, so o_absorb needs no transposed copy of the weights), one thread issues
// the copies, one the tcgen05.mma (M128 N256 K16, fp32 accumulators in 256 TMEM columns), four warps
// write the tile out as fp16.  Rows past the end of the batch are zero-filled by the copy engine and not
// stored.  All waits are bounded.
#include <cuda.h>   // CUtensorMap (types only; the encoder is fetched through the runtime at first use)

#include <cstdlib>
#include <cstring>

#include "hk_common.cuh"
#include "tc05.cuh"

namespace hk {

// Two stages, not three: 97 KB of shared memory and 256 TMEM columns per CTA let TWO CTAs share an SM, so one CTA's
// epilogue (64 KB of fp16 out of TMEM) runs under the other's copies and products: 202 -> 170 us (q) and 135 -> 122 us
// (o) at 4,096 rows.  K is only 256 or 512 (4 or 8 chunks), so a deeper ring inside one CTA has little to overlap.
constexpr int AB_BM = 128, AB_BN = 256, AB_BK = 64, AB_STAGES = 2;
constexpr uint32_t AB_A_BYTES = AB_BM * AB_BK * 2;            // 16 KB
constexpr uint32_t AB_B_BYTES = AB_BN * AB_BK * 2;            // 32 KB
constexpr uint32_t AB_STAGE = AB_A_BYTES + AB_B_BYTES;        // 48 KB
constexpr uint32_t AB_SMEM = AB_STAGES * AB_STAGE + 1024;     // + slack to align the base to 1 KB
constexpr int AB_THREADS = 192;

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          tc::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(tc::smem_u32(bar))
      : "memory");
}

// B_MN: the weight tile has n contiguous ([k][n] in memory), else k contiguous ([n][k]).
// a_col0 / b_*0: element coordinates of this head's operands inside the two tensor maps.
template <bool B_MN>
__global__ __launch_bounds__(AB_THREADS, 1) void absorb_gemm_tc_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const __grid_constant__ CUtensorMap tmap_o, int use_tma_out,
    __half* __restrict__ out, int n_rows, int K, int n_out, int b_rows_per_head, int b_row_off,
    int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t full_bar[AB_STAGES], empty_bar[AB_STAGES], done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nt = blockIdx.x, row0 = blockIdx.y * AB_BM, h = blockIdx.z;
  const int nk = K / AB_BK;

  if (tid == 0) {
    for (int i = 0; i < AB_STAGES; i++) {
      tc::mbar_init(&full_bar[i], 1);
      tc::mbar_init(&empty_bar[i], 1);
    }
    tc::mbar_init(&done_bar, 1);
    tc::mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 2) tc::tmem_alloc(&tmem_slot, AB_BN);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: one A box and the B boxes of every K chunk ----
      for (int kc = 0; kc < nk; kc++) {
        const int s = kc % AB_STAGES;
        if (kc >= AB_STAGES && !tc::mbar_wait<32>(&empty_bar[s], ((kc / AB_STAGES) - 1) & 1, &abort_flag, 1)) break;
        uint8_t* sa = smem + s * AB_STAGE;
        uint8_t* sb = sa + AB_A_BYTES;
        tc::mbar_arrive_expect_tx(&full_bar[s], AB_STAGE);
        tma_load_2d(sa, &tmap_a, h * K + kc * AB_BK, row0, &full_bar[s]);
        if (B_MN) {
          // [k][n]: four boxes of 64 n x 64 k, each a stack of 8-row swizzle atoms
#pragma unroll
          for (int j = 0; j < AB_BN / 64; j++)
            tma_load_2d(sb + j * 8192, &tmap_b, nt * AB_BN + j * 64, h * b_rows_per_head + b_row_off + kc * AB_BK, &full_bar[s]);
        } else {
          // [n][k]: one box of 64 k x 256 n rows
          tma_load_2d(sb, &tmap_b, kc * AB_BK, h * b_rows_per_head + b_row_off + nt * AB_BN, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- tensor-core issue ----
      const uint32_t idesc = tc::make_idesc(AB_BM, AB_BN, tc::FMT_F16, tc::FMT_F16, false, B_MN);
      for (int kc = 0; kc < nk; kc++) {
        const int s = kc % AB_STAGES;
        if (!tc::mbar_wait<32>(&full_bar[s], (kc / AB_STAGES) & 1, &abort_flag, 2)) break;
        tc::fence_after_sync();
        const uint32_t a_addr = tc::smem_u32(smem + s * AB_STAGE), b_addr = a_addr + AB_A_BYTES;
#pragma unroll
        for (int k16 = 0; k16 < AB_BK / 16; k16++) {
          const uint64_t ad = tc::make_sdesc_sw128(a_addr + k16 * 32, 16, 1024);
          const uint64_t bd = B_MN ? tc::make_sdesc_sw128(b_addr + k16 * 2048, 8192, 1024)
                                   : tc::make_sdesc_sw128(b_addr + k16 * 32, 16, 1024);
          tc::mma_f16(tmem, ad, bd, idesc, kc > 0 || k16 > 0);
        }
        tc::mma_commit(&empty_bar[s]);
      }
      tc::mma_commit(&done_bar);
    }
  } else {
    // ---- epilogue: warps 2-5 cover the four TMEM lane quarters (a warp may only touch quarter warp % 4) ----
    const int q = warp & 3;
    const int row = row0 + q * 32 + lane;
    const bool ok = tc::mbar_wait<64>(&done_bar, 0, &abort_flag, 3);
    tc::fence_after_sync();
    if (ok && use_tma_out) {
      // The fp16 tile leaves through the copy engine: every thread lays its row into the (now idle) operand stages as
      // four 128-row x 64-column boxes in the 128-byte-swizzle pattern (16-byte piece c of row r at c ^ (r % 8):
      // conflict-free), one thread hands the four boxes over as tiled stores (rows past the end are clipped).  Direct
      // stores put 32 different rows into every warp instruction.
      const int r = q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < AB_BN; c0 += 32) {
        uint32_t rr[32];
        tc::tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + c0, rr);
        tc::tmem_ld_wait();
        uint8_t* box = smem + (c0 >> 6) * 16384 + r * 128;
#pragma unroll
        for (int u = 0; u < 4; u++) {
          uint4 p;
          __half2 h0 = __floats2half2_rn(__uint_as_float(rr[8 * u + 0]), __uint_as_float(rr[8 * u + 1]));
          __half2 h1 = __floats2half2_rn(__uint_as_float(rr[8 * u + 2]), __uint_as_float(rr[8 * u + 3]));
          __half2 h2 = __floats2half2_rn(__uint_as_float(rr[8 * u + 4]), __uint_as_float(rr[8 * u + 5]));
          __half2 h3 = __floats2half2_rn(__uint_as_float(rr[8 * u + 6]), __uint_as_float(rr[8 * u + 7]));
          p.x = *reinterpret_cast<uint32_t*>(&h0); p.y = *reinterpret_cast<uint32_t*>(&h1);
          p.z = *reinterpret_cast<uint32_t*>(&h2); p.w = *reinterpret_cast<uint32_t*>(&h3);
          const int cc = ((c0 & 63) >> 3) + u;
          *reinterpret_cast<uint4*>(box + ((cc ^ (r & 7)) << 4)) = p;
        }
      }
      tc::fence_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
#pragma unroll
        for (int j = 0; j < AB_BN / 64; j++)
          asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&tmap_o),
                       "r"(nt * AB_BN + j * 64), "r"(h), "r"(row0), "r"(tc::smem_u32(smem + j * 16384))
                       : "memory");
        tc::bulk_commit();
        tc::bulk_wait_read<0>();                  // the boxes have been read: the CTA may leave
      }
    } else if (ok) {
      __half* orow = out + ((size_t)row * 64 + h) * n_out + nt * AB_BN;
#pragma unroll 1
      for (int c0 = 0; c0 < AB_BN; c0 += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + c0, r);
        tc::tmem_ld_wait();
        if (row < n_rows) {
#pragma unroll
          for (int u = 0; u < 4; u++) {
            uint4 p;
            __half2 h0 = __floats2half2_rn(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
            __half2 h1 = __floats2half2_rn(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
            __half2 h2 = __floats2half2_rn(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
            __half2 h3 = __floats2half2_rn(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
            p.x = *reinterpret_cast<uint32_t*>(&h0); p.y = *reinterpret_cast<uint32_t*>(&h1);
            p.z = *reinterpret_cast<uint32_t*>(&h2); p.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(orow + c0 + 8 * u) = p;
          }
        }
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 2) tc::tmem_dealloc(tmem, AB_BN);
  if (tid == 0 && abort_flag && status) atomicExch(status, HK_ERR_TIMEOUT);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool looked_up = false;
  if (!looked_up) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    looked_up = true;
  }
  return fn;
}

// fp16 matrix [rows][cols] (cols contiguous), box [box_rows][box_cols], 128-byte swizzle, zero fill outside
static bool make_map_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// a [n_rows][64*K], weights as described above, out [n_rows][64*n_out]; returns HK_ERR_UNSUPPORTED when the
// tensor maps cannot be built (the caller then uses the CUDA-core kernels)
int absorb_gemm_tc(const void* a, const void* b, void* out, int n_rows, int K, int n_out, bool b_mn,
                   uint64_t b_rows, uint64_t b_cols, int b_rows_per_head, int b_row_off, cudaStream_t s) {
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(out, 16)) return HK_ERR_UNSUPPORTED;
  alignas(64) CUtensorMap ma, mb;
  memset(&ma, 0, sizeof(ma));
  memset(&mb, 0, sizeof(mb));
  if (!make_map_2d(&ma, a, (uint64_t)n_rows, (uint64_t)64 * K, AB_BM, AB_BK)) return HK_ERR_UNSUPPORTED;
  if (!make_map_2d(&mb, b, b_rows, b_cols, b_mn ? AB_BK : AB_BN, 64)) return HK_ERR_UNSUPPORTED;
  // output as [row][head][n_out]: boxes of 64 columns x 1 head x 128 rows for the tiled stores of the epilogue
  alignas(64) CUtensorMap mo;
  memset(&mo, 0, sizeof(mo));
  int use_tma_out = 0;
  {
    EncodeTiledFn enc = encode_tiled_fn();
    const cuuint64_t dims[3] = {(cuuint64_t)n_out, 64, (cuuint64_t)n_rows};
    const cuuint64_t strides[2] = {(cuuint64_t)n_out * 2, (cuuint64_t)64 * n_out * 2};
    const cuuint32_t box[3] = {64, 1, AB_BM};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (enc && enc(&mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
      use_tma_out = 1;
  }
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(absorb_gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AB_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(absorb_gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AB_SMEM) != cudaSuccess)
      return HK_ERR_CUDA;
    attr_set[dev] = true;
  }
  const dim3 grid(n_out / AB_BN, (n_rows + AB_BM - 1) / AB_BM, 64);
  if (b_mn)
    absorb_gemm_tc_kernel<true><<<grid, AB_THREADS, AB_SMEM, s>>>(ma, mb, mo, use_tma_out, (__half*)out, n_rows, K, n_out, b_rows_per_head, b_row_off, device_status_ptr());
  else
    absorb_gemm_tc_kernel<false><<<grid, AB_THREADS, AB_SMEM, s>>>(ma, mb, mo, use_tma_out, (__half*)out, n_rows, K, n_out, b_rows_per_head, b_row_off, device_status_ptr());
  return cudaPeekAtLastError() == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

}  // namespace hk
