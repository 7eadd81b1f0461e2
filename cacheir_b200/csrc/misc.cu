// Library identification and error text.
#include "common.cuh"

#ifndef CB200_BUILD_INFO
#define CB200_BUILD_INFO "cacheir_b200 (sm_100a)"
#endif

extern "C" int cacheir_b200_version(void) { return 100; }

extern "C" const char* cacheir_b200_build_info(void) { return CB200_BUILD_INFO; }

extern "C" const char* cacheir_b200_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case CACHEIR_B200_EINVAL: return "cacheir_b200: invalid argument (extent, dtype, flag or null pointer)";
    case CACHEIR_B200_EALIGN: return "cacheir_b200: pointer or stride is not aligned as the kernel requires";
    case CACHEIR_B200_EWORKSPACE: return "cacheir_b200: workspace missing or smaller than *_workspace_bytes()";
    case CACHEIR_B200_EUNSUPPORTED: return "cacheir_b200: shape is outside what the kernels cover";
    case CACHEIR_B200_ELIMIT: return "cacheir_b200: argument exceeds a documented fixed maximum";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "cacheir_b200: unknown error code";
}

