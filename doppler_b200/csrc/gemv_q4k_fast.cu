// placeholder, replaced below
#include "common.h"
dp_status dpk_gemv_q4k_fast(dp_ctx *, const uint8_t *, const float *, void *, dp_dtype, int, int, float, const float *, bool *handled) { *handled = false; return DP_OK; }
