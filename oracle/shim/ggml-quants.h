/* Test infrastructure only: C-linkage prototypes for the two I2_S entry points that the
 * reference defines in src/ggml-bitnet-mad.cpp:51 and :1043, so that the compiled
 * reference exports unmangled symbols for ctypes and for oracle/ref_driver.cpp. */
#pragma once
#include "ggml.h"
#ifdef __cplusplus
extern "C" {
#endif
size_t quantize_i2_s(const float * src, void * dst, int64_t nrow, int64_t n_per_row, const float * quant_weights);
void ggml_vec_dot_i2_i8_s(int n, float * s, size_t bs, const void * vx, size_t bx, const void * vy, size_t by, int nrc);
#ifdef __cplusplus
}
#endif
