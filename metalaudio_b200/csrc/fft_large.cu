// Placeholder translation unit; replaced below in this file's history by the multi-pass path.
#include "fft_plan.h"
namespace ma {
ma_status large_plan_init(ma_fft_plan*) { return MA_ERR_UNSUPPORTED; }
void large_plan_destroy(ma_fft_plan*) {}
ma_status launch_r2c_large(ma_fft_plan*, const float*, float*, float*, float*, int, float, int64_t, int) { return MA_ERR_UNSUPPORTED; }
ma_status launch_c2r_large(ma_fft_plan*, const float*, const float*, float*, int64_t, int) { return MA_ERR_UNSUPPORTED; }
}
