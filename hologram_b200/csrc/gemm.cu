#include "common.h"
int32_t holo_launch_matmul(holo_b200_ctx*, const void*, const void*, void*, uint32_t, uint32_t, uint32_t, uint8_t, uint8_t, const void*) {
    return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul kernel not built");
}
