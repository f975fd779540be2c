// Fused attention forward on tcgen05 (placeholder translation unit: the entry
// point answers NB200_E_UNSUPPORTED until the kernel is in).
#include "common.cuh"
using namespace nb200;

extern "C" int nb200_attention_fwd(const void*, const void*, const void*, void*, int64_t, int64_t,
                                   int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                   int64_t, int64_t, int64_t, float, int, int, void*) {
  return fail(NB200_E_UNSUPPORTED, "attention kernel not built yet");
}
