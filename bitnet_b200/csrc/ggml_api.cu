// The reference's ggml backend entry points (include/ggml-bitnet.h:27-40) on the GPU kernels.
// Host pointers in, host pointers out; see include/ggml-bitnet-b200.h.
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "../../include/bitnet_b200.h"
#include "../../include/ggml-bitnet-b200.h"
#include "common.cuh"
#include "kernels.h"

namespace bitnet {

namespace {

constexpr int kMaxNodes = 8192;   // GGML_BITNET_MAX_NODES, include/bitnet-lut-kernels.h:5

struct Node {
    void* w2t = nullptr;     // device
    float* scale = nullptr;  // host
    int rows = 0, k = 0;
};

std::mutex g_mutex;
bool g_initialized = false;
bitnet_tensor_extra* g_extras = nullptr;
Node* g_nodes = nullptr;
size_t g_count = 0;
int g_threads = 1;

struct DevBuf {
    void* p = nullptr;
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
};

bool supported(enum ggml_type t) { return t == GGML_TYPE_I2_S; }

// Per-row absmax quantisation of f32 activations (no norm): a = 127 / max(absmax, 1e-5),
// y = clamp(rint(x * a), -128, 127); one CTA per row.
__global__ void quant_f32_rows_kernel(const float* x, int8_t* y, float* scale, float* sum, int k) {
    __shared__ float sh[8];
    const float* row = x + (int64_t)blockIdx.x * k;
    float mx = 0.f;
    for (int i = threadIdx.x; i < k; i += 256) mx = fmaxf(mx, fabsf(row[i]));
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = sh[0];
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, sh[i]);
    __syncthreads();
    const float a = 127.0f / fmaxf(mx, 1e-5f);
    float s = 0.f;
    for (int i = threadIdx.x; i < k; i += 256) {
        float f = rintf(row[i] * a);
        f = fminf(fmaxf(f, -128.f), 127.f);
        y[(int64_t)blockIdx.x * k + i] = (int8_t)(int)f;
        s += f;
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; ++i) t += sh[i];
        scale[blockIdx.x] = a;
        sum[blockIdx.x] = t;
    }
}

const Node* find_node(const void* w2t) {
    for (size_t i = 0; i < g_count; ++i)
        if (g_nodes[i].w2t == w2t) return &g_nodes[i];
    return nullptr;
}

}  // namespace

}  // namespace bitnet

using namespace bitnet;

extern "C" {

void ggml_bitnet_init(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_initialized) return;
    g_initialized = true;
    if (!g_extras) g_extras = new bitnet_tensor_extra[kMaxNodes];
    if (!g_nodes) g_nodes = new Node[kMaxNodes];
    g_count = 0;
}

void ggml_bitnet_free(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_initialized) return;
    g_initialized = false;
    for (size_t i = 0; i < g_count; ++i) {
        if (g_nodes[i].w2t) cudaFree(g_nodes[i].w2t);
        free(g_nodes[i].scale);
    }
    delete[] g_extras;
    delete[] g_nodes;
    g_extras = nullptr;
    g_nodes = nullptr;
    g_count = 0;
}

bool ggml_bitnet_can_mul_mat(const struct ggml_tensor* src0, const struct ggml_tensor* src1,
                             const struct ggml_tensor* dst) {
    if (!src0 || !src1 || !dst) return false;
    return supported(src0->type) && src1->type == GGML_TYPE_F32 && dst->type == GGML_TYPE_F32 &&
           src0->ne[0] % 128 == 0 && src0->ne[0] == src1->ne[0];
}

size_t ggml_bitnet_mul_mat_get_wsize(const struct ggml_tensor* src0, const struct ggml_tensor* src1,
                                     const struct ggml_tensor* dst) {
    (void)src0;
    (void)dst;
    const size_t ne10 = (size_t)src1->ne[0], ne11 = (size_t)src1->ne[1];
    size_t wsize = ne10 * ne11 * sizeof(int8_t) + ne11 * 2 * sizeof(float);
    return ((wsize - 1) / 64 + 1) * 64;
}

int ggml_bitnet_get_type_bits(enum ggml_type type) {
    switch (type) {
        case GGML_TYPE_I2_S:
        case GGML_TYPE_TL1:
        case GGML_TYPE_TL2: return 2;
        case GGML_TYPE_Q4_0: return 4;
        default: return 0;
    }
}

void ggml_bitnet_set_n_threads(int n_threads) { g_threads = n_threads; }

void ggml_bitnet_transform_tensor(struct ggml_tensor* tensor) {
    set_status(kOk);
    if (!tensor || !(supported(tensor->type) && tensor->extra == nullptr)) return;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_initialized || g_count >= (size_t)kMaxNodes) {
        set_status(g_initialized ? kTooLarge : kBadArgument);
        return;
    }
    const int k = (int)tensor->ne[0], rows = (int)tensor->ne[1];
    if (k < 1 || rows < 1 || ((int64_t)k * rows) % 128 != 0 || !tensor->data) {
        set_status(kUnsupported);
        return;
    }
    const size_t packed = (size_t)k * rows / 4;
    DevBuf d_i2s;
    void* w2t = nullptr;
    if (check_cuda(d_i2s.alloc(packed)) || check_cuda(cudaMalloc(&w2t, bitnet_w2t_bytes(rows, k)))) return;
    if (check_cuda(cudaMemcpy(d_i2s.p, tensor->data, packed, cudaMemcpyHostToDevice)) ||
        pack_i2s_to_w2t(static_cast<const uint8_t*>(d_i2s.p), w2t, rows, k, nullptr) ||
        check_cuda(cudaDeviceSynchronize())) {
        cudaFree(w2t);
        return;
    }
    float* scale = static_cast<float*>(malloc(sizeof(float)));
    memcpy(scale, static_cast<const uint8_t*>(tensor->data) + packed, sizeof(float));   // src/ggml-bitnet-mad.cpp:90-91
    g_nodes[g_count] = Node{w2t, scale, rows, k};
    g_extras[g_count] = bitnet_tensor_extra{1, 128, (rows + 15) / 16, static_cast<uint8_t*>(w2t), scale};
    tensor->extra = &g_extras[g_count];
    ++g_count;
}

void ggml_bitnet_mul_mat_task_init(void* src1, void* qlut, void* lut_scales, void* lut_biases, int n, int k, int m,
                                   int bits) {
    (void)bits;
    set_status(kOk);
    if (!src1 || !qlut || !lut_scales || !lut_biases || k < 1 || m < 1 || n != k) {
        set_status(kBadArgument);
        return;
    }
    DevBuf d_x, d_y, d_s, d_b;
    const size_t ne = (size_t)m * k;
    if (check_cuda(d_x.alloc(ne * 4)) || check_cuda(d_y.alloc(ne)) || check_cuda(d_s.alloc(m * 4)) ||
        check_cuda(d_b.alloc(m * 4)))
        return;
    if (check_cuda(cudaMemcpy(d_x.p, src1, ne * 4, cudaMemcpyHostToDevice))) return;
    quant_f32_rows_kernel<<<m, 256>>>(static_cast<const float*>(d_x.p), static_cast<int8_t*>(d_y.p),
                                      static_cast<float*>(d_s.p), static_cast<float*>(d_b.p), k);
    if (check_cuda(cudaGetLastError())) return;
    if (check_cuda(cudaMemcpy(qlut, d_y.p, ne, cudaMemcpyDeviceToHost)) ||
        check_cuda(cudaMemcpy(lut_scales, d_s.p, m * 4, cudaMemcpyDeviceToHost)) ||
        check_cuda(cudaMemcpy(lut_biases, d_b.p, m * 4, cudaMemcpyDeviceToHost)))
        return;
}

void ggml_bitnet_mul_mat_task_compute(void* src0, void* scales, void* qlut, void* lut_scales, void* lut_biases,
                                      void* dst, int n, int k, int m, int bits) {
    (void)bits;
    (void)n;
    set_status(kOk);
    if (!src0 || !scales || !qlut || !lut_scales || !lut_biases || !dst || k < 1 || m < 1) {
        set_status(kBadArgument);
        return;
    }
    int rows = 0;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        const Node* node = find_node(src0);
        if (!node || node->k != k) {
            set_status(kBadArgument);   // not a tensor ggml_bitnet_transform_tensor produced
            return;
        }
        rows = node->rows;
    }
    DevBuf d_y, d_sum, d_acc;
    const size_t ne = (size_t)m * k;
    std::vector<int32_t> ysum(m);
    for (int t = 0; t < m; ++t) ysum[t] = (int32_t)static_cast<const float*>(lut_biases)[t];
    if (check_cuda(d_y.alloc(ne)) || check_cuda(d_sum.alloc(m * 4)) || check_cuda(d_acc.alloc((size_t)m * rows * 4)))
        return;
    if (check_cuda(cudaMemcpy(d_y.p, qlut, ne, cudaMemcpyHostToDevice)) ||
        check_cuda(cudaMemcpy(d_sum.p, ysum.data(), m * 4, cudaMemcpyHostToDevice)))
        return;
    LinearArgs a;
    a.w2t = src0;
    a.y = static_cast<const int8_t*>(d_y.p); a.ldy = k;
    a.ysum = static_cast<const int32_t*>(d_sum.p);
    a.acc_out = static_cast<int32_t*>(d_acc.p);
    a.M = m; a.N = rows; a.K = k;
    a.seg.n_seg = 1;
    if (w2a8_gemv(a, nullptr)) return;
    std::vector<int32_t> acc((size_t)m * rows);
    if (check_cuda(cudaMemcpy(acc.data(), d_acc.p, acc.size() * 4, cudaMemcpyDeviceToHost))) return;
    const float ws = static_cast<const float*>(scales)[0];
    float* out = static_cast<float*>(dst);
    for (int t = 0; t < m; ++t) {
        const float a_t = static_cast<const float*>(lut_scales)[t];
        for (int r = 0; r < rows; ++r) out[(size_t)t * rows + r] = (float)acc[(size_t)t * rows + r] / a_t * ws;
    }
}

void ggml_bitnet_mul_mat(const struct ggml_compute_params* params, struct ggml_tensor* dst) {
    set_status(kOk);
    if (!params || !dst || !dst->src[0] || !dst->src[1]) {
        set_status(kBadArgument);
        return;
    }
    if (params->ith != 0) return;   // one GPU launch sequence; ggml's other threads have nothing to do
    const struct ggml_tensor* src0 = dst->src[0];
    const struct ggml_tensor* src1 = dst->src[1];
    const bitnet_tensor_extra* extra = static_cast<const bitnet_tensor_extra*>(src0->extra);
    if (!extra || !params->wdata || params->wsize < ggml_bitnet_mul_mat_get_wsize(src0, src1, dst)) {
        set_status(kBadArgument);
        return;
    }
    const int ne00 = (int)src0->ne[0], ne10 = (int)src1->ne[0], ne11 = (int)src1->ne[1];
    const int bits = ggml_bitnet_get_type_bits(src0->type);
    // work space layout as in src/ggml-bitnet-lut.cpp:104-109, with one int8 per activation
    int8_t* qlut = static_cast<int8_t*>(params->wdata);
    float* lut_scales = reinterpret_cast<float*>(qlut + (size_t)ne10 * ne11);
    float* lut_biases = lut_scales + ne11;
    ggml_bitnet_mul_mat_task_init(src1->data, qlut, lut_scales, lut_biases, ne10, ne00, ne11, bits);
    if (bitnet_last_status() != kOk) return;
    ggml_bitnet_mul_mat_task_compute(extra->qweights, extra->scales, qlut, lut_scales, lut_biases, dst->data, ne10,
                                     ne00, ne11, bits);
}

// ---- the TL2 kernel signatures (include/ggml-bitnet.h:46-47) ------------------------------------
void ggml_preprocessor(int bs, int m, int three_k, int two_k, void* B, void* LUT_Scales, void* Three_QLUT,
                       void* Two_QLUT) {
    (void)m;
    set_status(kOk);
    const int k = three_k + two_k;
    if (!B || !LUT_Scales || bs < 1 || three_k < 0 || two_k < 0 || k < 1 || three_k % 3 != 0 || two_k % 2 != 0 ||
        (three_k && !Three_QLUT) || (two_k && !Two_QLUT)) {
        set_status(kBadArgument);
        return;
    }
    DevBuf d_x, d_y, d_s, d_b;
    const size_t ne = (size_t)bs * k;
    if (check_cuda(d_x.alloc(ne * 4)) || check_cuda(d_y.alloc(ne)) || check_cuda(d_s.alloc(bs * 4)) ||
        check_cuda(d_b.alloc(bs * 4)))
        return;
    if (check_cuda(cudaMemcpy(d_x.p, B, ne * 4, cudaMemcpyHostToDevice))) return;
    // per_tensor_quant of include/bitnet-lut-kernels.h (one scale 127/absmax per activation row)
    quant_f32_rows_kernel<<<bs, 256>>>(static_cast<const float*>(d_x.p), static_cast<int8_t*>(d_y.p),
                                       static_cast<float*>(d_s.p), static_cast<float*>(d_b.p), k);
    if (check_cuda(cudaGetLastError())) return;
    if (check_cuda(cudaMemcpy(LUT_Scales, d_s.p, bs * 4, cudaMemcpyDeviceToHost))) return;
    const int8_t* y = static_cast<const int8_t*>(d_y.p);
    if (three_k && check_cuda(cudaMemcpy2D(Three_QLUT, (size_t)three_k / 3 * 32, y, k, three_k, bs, cudaMemcpyDeviceToHost)))
        return;
    if (two_k && check_cuda(cudaMemcpy2D(Two_QLUT, (size_t)two_k / 2 * 32, y + three_k, k, two_k, bs, cudaMemcpyDeviceToHost)))
        return;
}

void ggml_qgemm_lut(int bs, int m, int k, int BK, void* A, void* sign, void* LUT, void* Scales, void* LUT_Scales,
                    void* C) {
    (void)sign;
    set_status(kOk);
    if (!A || !Scales || !LUT_Scales || !C || bs < 1 || m < 1 || k < 1 || BK < 0 || BK > k || (BK > 0 && !LUT)) {
        set_status(kBadArgument);
        return;
    }
    const bool three = 2 * BK >= k;                  // the part of K grouped in threes comes first
    const int col0 = three ? 0 : k - BK;             // the columns this call multiplies
    const size_t stride = three ? (size_t)BK / 3 * 32 : (size_t)BK / 2 * 32;
    std::vector<int32_t> part;
    if (BK > 0) {
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            const Node* node = find_node(A);
            if (!node || node->k != k || node->rows != m) {
                set_status(kBadArgument);   // not a tensor ggml_bitnet_transform_tensor produced
                return;
            }
        }
        // The int8 activations of this call's columns, zero elsewhere: a zero activation adds
        // nothing to the product nor to the row sum that the weight offset takes off.
        DevBuf d_y, d_acc;
        if (check_cuda(d_y.alloc((size_t)bs * k)) || check_cuda(d_acc.alloc((size_t)bs * m * 4))) return;
        if (check_cuda(cudaMemset(d_y.p, 0, (size_t)bs * k)) ||
            check_cuda(cudaMemcpy2D(static_cast<int8_t*>(d_y.p) + col0, k, LUT, stride, BK, bs, cudaMemcpyHostToDevice)))
            return;
        LinearArgs a;
        a.w2t = A;
        a.y = static_cast<const int8_t*>(d_y.p); a.ldy = k;
        a.acc_out = static_cast<int32_t*>(d_acc.p);
        a.M = bs; a.N = m; a.K = k;
        a.seg.n_seg = 1;
        if (w2a8_gemv(a, nullptr)) return;
        part.resize((size_t)bs * m);
        if (check_cuda(cudaMemcpy(part.data(), d_acc.p, part.size() * 4, cudaMemcpyDeviceToHost))) return;
    }
    int32_t* ci = static_cast<int32_t*>(C);
    if (three) {                                     // first call of the pair: int32 sums
        for (size_t i = 0; i < (size_t)bs * m; ++i) ci[i] = part[i];
        return;
    }
    // second call: add this part's sums and finalise as include/bitnet-lut-kernels.h:993-999 does
    const float ws = static_cast<const float*>(Scales)[0];
    float* cf = static_cast<float*>(C);
    for (int b = 0; b < bs; ++b) {
        const float a_b = static_cast<const float*>(LUT_Scales)[b];
        for (int i = 0; i < m; ++i) {
            const size_t idx = (size_t)b * m + i;
            const int32_t v = ci[idx] + (BK > 0 ? part[idx] : 0);
            cf[idx] = (float)v / a_b * ws;
        }
    }
}

}  // extern "C"
