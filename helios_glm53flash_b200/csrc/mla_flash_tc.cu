// placeholder, replaced below
#include "mla_args.cuh"
namespace hk {
int mla_flash_tc_launch(const MlaArgs&, cudaStream_t) { return HK_ERR_UNSUPPORTED; }
int mla_flash_tc_auto_splits(int m, int n_keys) {
  long ctas = (long)m * 16;
  int want = (int)((2L * sm_count() + ctas - 1) / ctas);
  int cap = (n_keys + 63) / 64;
  int s = want < 1 ? 1 : want;
  if (s > cap) s = cap < 1 ? 1 : cap;
  return s > 64 ? 64 : s;
}
}
