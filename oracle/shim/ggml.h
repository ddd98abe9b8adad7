/* Test infrastructure only: the minimum of ggml's public header that the reference's
 * src/ggml-bitnet-mad.cpp and include/ggml-bitnet.h need in order to compile outside
 * the llama.cpp fork (which the reference pulls in as an un-vendored submodule).
 * Nothing here is product code. */
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifndef GGML_API
#define GGML_API
#endif
#ifndef GGML_RESTRICT
#define GGML_RESTRICT __restrict__
#endif
#ifndef GGML_ASSERT
#include <assert.h>
#define GGML_ASSERT(x) assert(x)
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum ggml_type {
    GGML_TYPE_F32  = 0,
    GGML_TYPE_F16  = 1,
    GGML_TYPE_Q4_0 = 2,
    GGML_TYPE_I8   = 24,
    GGML_TYPE_I2_S = 36,
    GGML_TYPE_TL1  = 38,
    GGML_TYPE_TL2  = 39,
};

struct ggml_tensor;

/* The reference calls ggml_row_size(GGML_TYPE_I2_S, n_per_row) and divides the result
 * by four itself (src/ggml-bitnet-mad.cpp:55,95), so the element count is what it needs. */
static inline size_t ggml_row_size(enum ggml_type type, int64_t ne) {
    (void)type;
    return (size_t)ne;
}

#ifdef __cplusplus
}
#endif
