/* Test infrastructure only: a plain-C restatement of the reference's W2A8 BitLinear
 * arithmetic.  It is the checker for the CUDA path (tests, the smoke check and the CPU
 * leg of the benchmark); nothing on the product path may call it.
 *
 * Parity status: the integer part (pack, dot, matrix product) is pinned against the
 * reference's own compiled src/ggml-bitnet-mad.cpp and against golden vectors made from
 * it.  The float epilogue of the CPU path (activation quantisation, the -sum(y) offset
 * and the rescale) lives in the reference's un-vendored llama.cpp fork and has no test
 * in the reference: parity unpinned for that part; it follows the in-repo statements of
 * the same formula (gpu/model.py:68-71, gpu/bitnet_kernels/bitnet_kernels.h:80-82,
 * include/bitnet-lut-kernels.h:73-91,993-999). */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define I2S_BLOCK 128

/* src/ggml-bitnet-mad.cpp:51-96 (x86 ACT_PARALLEL form).  scale = max|src|; an element
 * with |x| < 1e-6 gets code 1, a positive one code 2, a negative one code 0.  Every 128
 * consecutive elements of the flattened matrix make 32 bytes: byte p holds elements
 * p, p+32, p+64, p+96 at bit shifts 6, 4, 2, 0.  The f32 scale follows the packed data;
 * the buffer is n/4 + 32 bytes. */
size_t port_quantize_i2_s(const float *src, void *dst, int64_t nrow, int64_t n_per_row) {
    const int64_t n = nrow * n_per_row;
    double mx = 0.0;
    for (int64_t i = 0; i < n; ++i) mx = fmax(mx, fabs((double)src[i]));
    uint8_t *out = (uint8_t *)dst;
    memset(out, 0, (size_t)(n / 4));
    for (int64_t i = 0; i < n; ++i) {
        uint8_t code;
        if (fabs((double)src[i]) < 1e-6) code = 1;
        else code = ((double)src[i] * mx > 0) ? 2 : 0;
        const int64_t blk = i / I2S_BLOCK, j = i % I2S_BLOCK;
        out[blk * 32 + (j % 32)] |= (uint8_t)(code << (6 - 2 * (j / 32)));
    }
    float sc = (float)mx;
    memcpy(out + n / 4, &sc, sizeof(float));
    return (size_t)(nrow * n_per_row / 4 + 32);
}

/* Code of element k of one packed row (inverse of the layout above). */
static inline int i2s_code(const uint8_t *row, int64_t k) {
    const int64_t blk = k / I2S_BLOCK, j = k % I2S_BLOCK;
    return (row[blk * 32 + (j % 32)] >> (6 - 2 * (j / 32))) & 3;
}

/* sum_k code_k * y_k with code in {0,1,2,3} taken literally, exact in int32.  This is
 * what ggml_vec_dot_i2_i8_s (src/ggml-bitnet-mad.cpp:198-310, :791-905) returns as a
 * float whenever none of its int16 lane partials wraps. */
int32_t port_vec_dot_i2_i8(int64_t n, const uint8_t *x, const int8_t *y) {
    int32_t acc = 0;
    for (int64_t blk = 0; blk < n / I2S_BLOCK; ++blk) {
        const uint8_t *px = x + blk * 32;
        const int8_t *py = y + blk * I2S_BLOCK;
        int32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
        for (int p = 0; p < 32; ++p) {
            const uint8_t b = px[p];
            s0 += ((b >> 6) & 3) * py[p];
            s1 += ((b >> 4) & 3) * py[p + 32];
            s2 += ((b >> 2) & 3) * py[p + 64];
            s3 += (b & 3) * py[p + 96];
        }
        acc += s0 + s1 + s2 + s3;
    }
    return acc;
}

/* acc[m * ldo + col] = sum_k code(col,k) * y[m,k]; x holds nc rows of k/4 bytes. */
void port_i2s_gemm(int64_t k, int32_t *acc, size_t ldo, const uint8_t *x, const int8_t *y,
                   int64_t nr, int64_t nc, int n_threads) {
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
    #pragma omp parallel for schedule(static)
    for (int64_t col = 0; col < nc; ++col) {
        const uint8_t *xr = x + col * k / 4;
        for (int64_t m = 0; m < nr; ++m)
            acc[m * ldo + col] = port_vec_dot_i2_i8(k, xr, y + m * k);
    }
}

/* Unpacks I2_S rows to ternary int8 {-1,0,+1} (code 3 -> +2, taken literally). */
void port_unpack_i2_s(const uint8_t *x, int8_t *w, int64_t nrow, int64_t n_per_row) {
    for (int64_t r = 0; r < nrow; ++r)
        for (int64_t k = 0; k < n_per_row; ++k)
            w[r * n_per_row + k] = (int8_t)(i2s_code(x + r * n_per_row / 4, k) - 1);
}

/* Per-token absmax quantisation, gpu/model.py:68-71 in f32:
 * a = 127 / max(absmax, 1e-5); y = clamp(round_half_even(x * a), -128, 127). */
void port_act_quant(const float *x, int8_t *y, float *a_out, int32_t *ysum, int64_t m, int64_t k) {
    for (int64_t r = 0; r < m; ++r) {
        float mx = 0.f;
        for (int64_t i = 0; i < k; ++i) mx = fmaxf(mx, fabsf(x[r * k + i]));
        const float a = 127.0f / fmaxf(mx, 1e-5f);
        int32_t s = 0;
        for (int64_t i = 0; i < k; ++i) {
            float v = rintf(x[r * k + i] * a);
            v = v < -128.f ? -128.f : (v > 127.f ? 127.f : v);
            y[r * k + i] = (int8_t)v;
            s += (int32_t)v;
        }
        a_out[r] = a;
        if (ysum) ysum[r] = s;
    }
}

/* out = (acc_code - ysum) / a * w_scale: the I2_S offset correction followed by the
 * rescale of gpu/bitnet_kernels/bitnet_kernels.h:82 (divide by the activation scale,
 * multiply by the weight scale of the row's segment).  seg_end[i] is the first row after
 * segment i. */
void port_rescale(const int32_t *acc, const int32_t *ysum, const float *a, const float *w_scale,
                  const int32_t *seg_end, int n_seg, float *out, int64_t m, int64_t n) {
    for (int64_t r = 0; r < m; ++r)
        for (int64_t c = 0; c < n; ++c) {
            int seg = 0;
            while (seg + 1 < n_seg && c >= seg_end[seg]) ++seg;
            out[r * n + c] = (float)(acc[r * n + c] - ysum[r]) / a[r] * w_scale[seg];
        }
}

double port_i2s_gemm_time(int64_t k, int32_t *acc, size_t ldo, const uint8_t *x, const int8_t *y,
                          int64_t nr, int64_t nc, int n_threads, int iters) {
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int i = 0; i < iters; ++i) port_i2s_gemm(k, acc, ldo, x, y, nr, nc, n_threads);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return ((t1.tv_sec - t0.tv_sec) + 1e-9 * (t1.tv_nsec - t0.tv_nsec)) / (iters > 0 ? iters : 1);
}

int port_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
