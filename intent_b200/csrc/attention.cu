// placeholder until the tcgen05 kernel lands
#include "common.cuh"
using namespace b200;
extern "C" int b200_flash_attention(const void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                         const void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                         const void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                         void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                         float, void *, int64_t, int64_t, int32_t, int32_t, int32_t, void *) {
  return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: not built yet");
}
