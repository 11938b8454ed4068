// Argument block shared by the MLA attention kernels of this library.
#pragma once
#include "hk_common.cuh"

namespace hk {

struct MlaArgs {
  const __half* q_lat;      // [m][n_heads][512]
  const __half* ckv;        // [*][512]
  int64_t ckv_rows;         // rows the cache holds (0 = not told): gathered indices beyond it count as holes, dense
                            // ranges are cut there, and the tensor map of the dense path gets this extent
  const int* raw_idx;       // sparse: [m][kidx]; dense: null
  int kidx;
  const int64_t* kv_base;   // dense: per-row first key (null = 0)
  const int* kv_len;        // dense: per-row key count (null = pos_start + r + 1)
  int pos_start;
  int m, n_heads;
  float scale;
  int n_split;
  __half* out;              // final output (n_split == 1) or null
  float* part_m;            // partials: [n_split][rows], [n_split][rows], [n_split][rows][512]
  float* part_l;
  float* part_acc;
};

}  // namespace hk
