// Test infrastructure only: a threaded matrix driver around the reference's compiled
// I2_S dot kernel, used as the parity checker and as the timed CPU baseline. Never part
// of the product path.
//
// It restates the cache-blocked loop that the reference ships inside its kernel timer
// (utils/test_gemm_kernel.sh:137-173, ACT_PARALLEL branch; block sizes from
// include/gemm-config.h:3-6: 128 weight rows x 4 activation rows) and spreads the weight
// row blocks over OpenMP threads.  The reference's loop hands a ragged activation tail
// (M % 4 != 0) to the dot kernel as nrc = tail, which its dispatcher
// (src/ggml-bitnet-mad.cpp:1043-1056) sends to the 1x1 routine where nrc counts weight
// rows; that is only right for a tail of one, so tails are issued here one activation
// row at a time.
#include <stdint.h>
#include <stddef.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" void ggml_vec_dot_i2_i8_s(int n, float * s, size_t bs, const void * vx, size_t bx,
                                     const void * vy, size_t by, int nrc);

extern "C" {

// out[m * ldo + col] = sum_k code(col, k) * y[m, k] as float, code in {0,1,2,3}.
// x: I2_S bytes, nc weight rows of k/4 bytes; y: nr activation rows of k int8.
void ref_i2s_gemm(int k, float * out, size_t ldo, const uint8_t * x, const int8_t * y,
                  int nr, int nc, int n_threads) {
    const int64_t col_block = 128, row_block = 4;
    const int64_t n_cblocks = (nc + col_block - 1) / col_block;
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
    #pragma omp parallel for schedule(dynamic, 1)
    for (int64_t cb = 0; cb < n_cblocks; ++cb) {
        const int64_t c0 = cb * col_block;
        const int64_t c1 = c0 + col_block < nc ? c0 + col_block : nc;
        for (int64_t r0 = 0; r0 < nr; r0 += row_block) {
            const int64_t cur_r = r0 + row_block <= nr ? row_block : nr - r0;
            const int8_t * y_r = y + r0 * (int64_t)k;
            for (int64_t col = c0; col < c1; ++col) {
                const uint8_t * x_col = x + col * (int64_t)k / 4;
                if (cur_r == row_block) {
                    ggml_vec_dot_i2_i8_s(k, out + r0 * ldo + col, ldo, x_col, k, y_r, k, (int)cur_r);
                } else {
                    for (int64_t r = 0; r < cur_r; ++r)
                        ggml_vec_dot_i2_i8_s(k, out + (r0 + r) * ldo + col, ldo, x_col, k,
                                             y_r + r * (int64_t)k, k, 1);
                }
            }
        }
    }
}

// Runs ref_i2s_gemm `iters` times and returns the mean seconds per call.
double ref_i2s_gemm_time(int k, float * out, size_t ldo, const uint8_t * x, const int8_t * y,
                         int nr, int nc, int n_threads, int iters) {
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int i = 0; i < iters; ++i) ref_i2s_gemm(k, out, ldo, x, y, nr, nc, n_threads);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return ((t1.tv_sec - t0.tv_sec) + 1e-9 * (t1.tv_nsec - t0.tv_nsec)) / (iters > 0 ? iters : 1);
}

int ref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
