// Status strings and ABI version of libhelios_b200.
#include "hk_common.cuh"

HK_API const char* hk_status_string(int status) {
  switch (status) {
    case HK_OK: return "ok";
    case HK_ERR_INVALID: return "invalid argument";
    case HK_ERR_UNSUPPORTED: return "unsupported shape";
    case HK_ERR_CUDA: return "CUDA launch error";
    case HK_ERR_WORKSPACE: return "workspace too small";
    case HK_ERR_TIMEOUT: return "bounded device wait expired";
    default: return "unknown status";
  }
}

HK_API int hk_abi_version(void) { return 1; }
