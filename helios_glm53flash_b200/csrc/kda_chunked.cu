// placeholder, replaced below
#include "hk_common.cuh"
HK_API size_t hk_kda_chunked_workspace_bytes(int, int, int) { return 256; }
HK_API int hk_kda_chunked_prefill(const void*, const float*, const void*, float*, void*, float*, int, int, int, const int*, void*, size_t, void*) { return HK_ERR_UNSUPPORTED; }
