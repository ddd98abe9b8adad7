/* The reference's ggml backend entry points (include/ggml-bitnet.h:27-40 of
 * microsoft/BitNet), backed by the B200 kernels of libbitnet_b200.so.
 *
 * The reference declares these against `struct ggml_tensor` and `struct ggml_compute_params`
 * of its llama.cpp fork (3rdparty/llama.cpp, an un-vendored submodule).  That header is not
 * available, so this file declares the minimal stand-in below with the fields the entry
 * points read.  Binary compatibility with the fork's real structs is UNVERIFIED: a
 * maintainer wiring this into ggml replaces the stand-in by `#include "ggml.h"` and rebuilds.
 * All pointers here are HOST pointers (ggml's CPU tensors); device copies are made inside. */
#ifndef GGML_BITNET_B200_H
#define GGML_BITNET_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GGML_BITNET_B200_NO_STANDIN
enum ggml_type {
    GGML_TYPE_F32 = 0,
    GGML_TYPE_F16 = 1,
    GGML_TYPE_Q4_0 = 2,
    GGML_TYPE_I8 = 24,
    GGML_TYPE_I2_S = 36,
    GGML_TYPE_TL1 = 38,
    GGML_TYPE_TL2 = 39,
};
struct ggml_tensor {
    enum ggml_type type;
    int64_t ne[4];              /* ne[0] = row length, ne[1] = rows */
    size_t nb[4];
    struct ggml_tensor* src[2];
    void* data;
    void* extra;                /* set by ggml_bitnet_transform_tensor */
};
struct ggml_compute_params {
    int ith, nth;               /* thread index / count of ggml's thread pool */
    size_t wsize;
    void* wdata;                /* at least ggml_bitnet_mul_mat_get_wsize bytes */
};
#endif

/* include/ggml-bitnet.h:19-25.  Here qweights is a DEVICE pointer to the W2T-packed tensor,
 * scales a host pointer to its f32 scale, BK the K extent of a packed tile (128) and
 * n_tile_num the number of 16-row groups. */
struct bitnet_tensor_extra {
    int lut_scales_size;
    int BK;
    int n_tile_num;
    uint8_t* qweights;
    float* scales;
};

/* src/ggml-bitnet-lut.cpp:22-42: idempotent; the table of at most 8192 tensor extras
 * (include/bitnet-lut-kernels.h:5) is allocated by init and released, together with the
 * device copies, by free. */
void ggml_bitnet_init(void);
void ggml_bitnet_free(void);
/* src/ggml-bitnet-lut.cpp:52-62 with the GPU's wider coverage: true when src0 is I2_S,
 * src1 and dst are F32 and the row length is a multiple of 128 (any number of src1 rows). */
bool ggml_bitnet_can_mul_mat(const struct ggml_tensor* src0, const struct ggml_tensor* src1,
                             const struct ggml_tensor* dst);
/* src/ggml-bitnet-lut.cpp:64-76: bytes of host work space for one mul_mat: the int8
 * activations plus one scale and one sum per src1 row, rounded up to 64. */
size_t ggml_bitnet_mul_mat_get_wsize(const struct ggml_tensor* src0, const struct ggml_tensor* src1,
                                     const struct ggml_tensor* dst);
/* Declared at include/ggml-bitnet.h:35, called at src/ggml-bitnet-lut.cpp:112 (no definition
 * in the reference checkout).  Activation pre-processing: src1 f32 [m, k] -> qlut int8 [m, k]
 * (per-row absmax quantisation), lut_scales f32 [m] = 127/absmax, lut_biases f32 [m] = the
 * row sums of qlut.  n is the row length as well (the reference passes ne10 and ne00). */
void ggml_bitnet_mul_mat_task_init(void* src1, void* qlut, void* lut_scales, void* lut_biases,
                                   int n, int k, int m, int bits);
/* Declared at include/ggml-bitnet.h:36, called at src/ggml-bitnet-lut.cpp:125.  src0 is
 * bitnet_tensor_extra::qweights of a transformed tensor, scales its scale; dst f32 [m, rows]
 * = (sum_k w*q) / lut_scales[m] * scales[0], the rescale of include/bitnet-lut-kernels.h:993-999. */
void ggml_bitnet_mul_mat_task_compute(void* src0, void* scales, void* qlut, void* lut_scales,
                                      void* lut_biases, void* dst, int n, int k, int m, int bits);
/* include/bitnet-lut-kernels.h:1126-1170: no-op unless the tensor is I2_S and has no extra;
 * otherwise reads the f32 scale behind the packed data, moves the weights to the device in
 * the W2T layout and attaches a bitnet_tensor_extra. */
void ggml_bitnet_transform_tensor(struct ggml_tensor* tensor);
/* src/ggml-bitnet-lut.cpp:88-133: thread 0 runs task_init and task_compute (one GPU launch
 * sequence); the other threads of the pool return at once. */
void ggml_bitnet_mul_mat(const struct ggml_compute_params* params, struct ggml_tensor* dst);
/* src/ggml-bitnet-lut.cpp:78-86: 2 for I2_S (and TL1/TL2), 4 for Q4_0, else 0. */
int ggml_bitnet_get_type_bits(enum ggml_type type);
/* Recorded only: the GPU path does not use ggml's threads. */
void ggml_bitnet_set_n_threads(int n_threads);

/* ---- the x86 TL2 kernel entry points (include/ggml-bitnet.h:46-47) on the GPU -------------
 * The reference generates these two per model shape (include/bitnet-lut-kernels.h:1003-1124 is
 * the preset for 3200/8640): the pre-processor quantises a batch of f32 activation rows and
 * builds look-up tables; the matmul is then called twice per output tile, first for the part of
 * K that is grouped in threes (BK = three_k; writes int32 sums to C), then for the remainder
 * (BK = two_k; adds its sums and turns C into floats, (float)sum / LUT_Scales[b] * Scales[0],
 * :993-999).  This library keeps the signatures and the two-call protocol, and gives them the
 * same result, but the buffers carry its own data:
 *   - A is bitnet_tensor_extra::qweights of a tensor that ggml_bitnet_transform_tensor of THIS
 *     library transformed (an I2_S tensor; the TL2 byte layout that the reference's converter
 *     writes into GGUF files is not decoded), and stands for the whole matrix, not one tile;
 *   - Three_QLUT / Two_QLUT receive the int8 activations (row b at byte b*three_k/3*32 and
 *     b*two_k/2*32, the reference's row strides; the first three_k / two_k bytes are used);
 *   - C is f32/int32 [bs, m]; `sign` is ignored.
 * The call with 2*BK >= k is the first of a pair (columns 0 .. BK-1, LUT = Three_QLUT), the other
 * one the second (columns k-BK .. k-1, LUT = Two_QLUT; BK may be 0).  All pointers are host
 * pointers.  How the llama.cpp fork drives these calls is not part of the reference
 * checkout: compatibility with its caller is unverified. */
void ggml_preprocessor(int bs, int m, int three_k, int two_k, void* B, void* LUT_Scales, void* Three_QLUT,
                       void* Two_QLUT);
void ggml_qgemm_lut(int bs, int m, int k, int BK, void* A, void* sign, void* LUT, void* Scales, void* LUT_Scales,
                    void* C);

#ifdef __cplusplus
}
#endif
#endif /* GGML_BITNET_B200_H */
