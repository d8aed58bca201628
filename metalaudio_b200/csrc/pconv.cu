#include "fft_plan.h"
extern "C" {
ma_status ma_pconv_create(ma_context*, int32_t, int32_t, ma_pconv**) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_destroy(ma_pconv*) { return MA_OK; }
ma_status ma_pconv_set_kernels(ma_pconv*, const float*, int64_t, int32_t, const int32_t*) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_partition_count(ma_pconv*, int32_t*) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_reserve(ma_pconv*, int64_t) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_process_dev(ma_pconv*, const float*, int64_t, int64_t, float*, int64_t) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_process_host(ma_pconv*, const float*, int64_t, int64_t, float*, int64_t) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_step_dev(ma_pconv*, const float*, int64_t, float*, int64_t) { return MA_ERR_UNSUPPORTED; }
ma_status ma_pconv_reset(ma_pconv*) { return MA_ERR_UNSUPPORTED; }
}
