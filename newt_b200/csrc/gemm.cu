// C = A @ B on tcgen05 (placeholder translation unit: entry points answer
// NB200_E_UNSUPPORTED until the kernel is in).
#include "common.cuh"
using namespace nb200;

extern "C" int nb200_gemm_check(const void*, const void*, const void*, int64_t, int64_t, int64_t,
                                int64_t, int64_t, int64_t, int, const nb200_gemm_config*) {
  return fail(NB200_E_UNSUPPORTED, "gemm kernel not built yet");
}
extern "C" int nb200_gemm(const void*, const void*, void*, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int64_t, int, const nb200_gemm_config*, void*) {
  return fail(NB200_E_UNSUPPORTED, "gemm kernel not built yet");
}
