// extern "C" entry points of libbitnet_b200.so (declared in include/bitnet_b200.h).
#include <string.h>

#include <vector>

#include "../../include/bitnet_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace bitnet {

static thread_local int g_status = kOk;
static thread_local char g_cuda_error[256] = "";

void set_status(int s) { g_status = s; }

int check_cuda(cudaError_t e) {
    if (e == cudaSuccess) return kOk;
    strncpy(g_cuda_error, cudaGetErrorString(e), sizeof(g_cuda_error) - 1);
    g_status = kCudaError;
    return kCudaError;
}

static int fail(int s) {
    g_status = s;
    return s;
}

// Equal row segments the reference's shape ladder uses for its weight scales
// (gpu/bitnet_kernels/bitnet_kernels.cu:4-33).
static ScaleSegments reference_segments(int N, int K) {
    int ws_num = 1;
    if (N == 3840 && K == 2560) ws_num = 3;
    else if (N == 13824 && K == 2560) ws_num = 2;
    else if (N == 4800 && K == 3200) ws_num = 6;
    else if (N == 20480 && K == 3200) ws_num = 2;
    ScaleSegments s{};
    s.n_seg = ws_num;
    for (int i = 0; i < 8; ++i) s.end[i] = i < ws_num ? (N / ws_num) * (i + 1) : N;
    return s;
}

// RAII device scratch for the host-pointer entry points.
struct DeviceBuf {
    void* p = nullptr;
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
    ~DeviceBuf() {
        if (p) cudaFree(p);
    }
};

}  // namespace bitnet

using namespace bitnet;

extern "C" {

int bitnet_last_status(void) { return g_status; }

const char* bitnet_status_string(int status) {
    switch (status) {
        case kOk: return "ok";
        case kBadArgument: return "bad argument";
        case kUnsupported: return "unsupported shape";
        case kCudaError: return "CUDA error";
        case kTooLarge: return "size exceeds a fixed capacity";
        default: return "unknown status";
    }
}

const char* bitnet_last_cuda_error(void) { return g_cuda_error; }

void bitlinear_int8xint2(int8_t* input0, int8_t* input1, void* output0, void* s, void* ws, int M, int N, int K,
                         void* stream) {
    g_status = kOk;
    if (!input0 || !input1 || !output0 || !s || !ws || M < 1 || N < 1 || K < 1) {
        fail(kBadArgument);
        return;
    }
    if (N % 16 != 0 || K % 128 != 0) {   // the [N, K/4] view has no room for padding
        fail(kUnsupported);
        return;
    }
    LinearArgs a;
    a.w2t = input1;
    a.y = input0; a.ldy = K;
    a.out = static_cast<__nv_bfloat16*>(output0); a.ldo = N;
    a.a_bf16 = static_cast<const __nv_bfloat16*>(s); a.a_stride = 1;
    a.ws_bf16 = static_cast<const __nv_bfloat16*>(ws);
    a.seg = reference_segments(N, K);
    a.M = M; a.N = N; a.K = K;
    w2a8_gemv(a, static_cast<cudaStream_t>(stream));
}

int bitnet_linear_w2a8(const int8_t* y, int64_t ldy, const void* w2t, void* out_bf16, int64_t ldo, int32_t* acc_out,
                       const float* act_scale, const int32_t* ysum, const float* w_scale, const int* seg_end,
                       int n_seg, int M, int N, int K, void* stream) {
    g_status = kOk;
    if (!y || !w2t || (!out_bf16 && !acc_out) || M < 1 || N < 1 || K < 1 || ldy < K) return fail(kBadArgument);
    if (out_bf16 && (!act_scale || !w_scale || !seg_end || n_seg < 1 || ldo < N)) return fail(kBadArgument);
    if (n_seg > 8) return fail(kTooLarge);
    LinearArgs a;
    a.w2t = w2t;
    a.y = y; a.ldy = ldy; a.ysum = ysum;
    a.acc_out = acc_out;
    a.out = static_cast<__nv_bfloat16*>(out_bf16); a.ldo = ldo;
    a.a_f32 = act_scale; a.a_stride = 1;
    a.ws_f32 = w_scale;
    a.seg.n_seg = out_bf16 ? n_seg : 1;
    for (int i = 0; i < 8; ++i) a.seg.end[i] = (out_bf16 && i < n_seg) ? seg_end[i] : N;
    a.M = M; a.N = N; a.K = K;
    return w2a8_gemv(a, static_cast<cudaStream_t>(stream));
}

int bitnet_linear_w2a8_add_quant(const int8_t* y, int64_t ldy, const void* w2t, const float* act_scale, const int32_t* ysum,
                                 float w_scale, int M, int N, int K, void* h_bf16, int64_t ldh, const void* gamma_bf16,
                                 float eps, int8_t* y_next, int64_t ldy_next, float* act_scale_next, int32_t* ysum_next,
                                 void* stream) {
    g_status = kOk;
    if (!y || !w2t || !act_scale || !ysum || !h_bf16 || M < 16 || N < 8 || K < 1 || ldy < K || ldh < N) return fail(kBadArgument);
    if (N % 8 != 0 || ldh % 8 != 0 || (reinterpret_cast<uintptr_t>(h_bf16) & 15) != 0) return fail(kUnsupported);
    const int64_t k_pad = (K + kTileCols - 1) / kTileCols * kTileCols;
    if (ldy % 16 != 0 || ldy < k_pad || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return fail(kUnsupported);
    if (y_next && (ldy_next < N || ldy_next % 8 != 0 || (reinterpret_cast<uintptr_t>(y_next) & 7) != 0)) return fail(kBadArgument);
    WorkspaceView ws;
    if (!workspace_view(&ws)) return kCudaError;
    const int32_t* sums = nullptr;
    bool raw = false;
    LinearArgs a;
    a.w2t = w2t;
    a.y = y; a.ldy = ldy; a.ysum = ysum;
    a.a_f32 = act_scale; a.a_stride = 1;
    a.seg.n_seg = 1;
    for (int i = 0; i < 8; ++i) a.seg.end[i] = N;
    a.M = M; a.N = N; a.K = K;
    a.sums = &sums; a.sums_raw = &raw;
    const int rc = w2a8_gemm_tc(a, ws.error_flag, ws.tc_acc, ws.tc_acc_ints, ws.n_sm, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
    QuantArgs q;
    q.x_bf16 = static_cast<const __nv_bfloat16*>(h_bf16); q.ldx = ldh;
    q.gamma = static_cast<const __nv_bfloat16*>(gamma_bf16); q.eps = eps;
    q.y = y_next; q.ldy = y_next ? ldy_next : N;
    q.a_f32 = act_scale_next; q.ysum = ysum_next;
    q.M = M; q.K = N;
    q.lin_acc = const_cast<int32_t*>(sums); q.lin_ysum = raw ? ysum : nullptr; q.lin_a = act_scale; q.lin_ws = w_scale;
    return act_quant(q, static_cast<cudaStream_t>(stream));
}

int bitnet_quant_input(const void* x_bf16, int64_t ldx, const void* gamma_bf16, float eps, int8_t* y, int64_t ldy,
                       float* act_scale, void* s_bf16, int32_t* ysum, int M, int K, void* stream) {
    g_status = kOk;
    if (!x_bf16 || !y || M < 1 || K < 1 || ldx < K || ldy < K) return fail(kBadArgument);
    if (ldy % 8 != 0 || (reinterpret_cast<uintptr_t>(y) & 7) != 0) return fail(kBadArgument);
    QuantArgs q;
    q.x_bf16 = static_cast<const __nv_bfloat16*>(x_bf16); q.ldx = ldx;
    q.gamma = static_cast<const __nv_bfloat16*>(gamma_bf16); q.eps = eps;
    q.y = y; q.ldy = ldy;
    q.a_f32 = act_scale; q.a_bf16 = static_cast<__nv_bfloat16*>(s_bf16); q.ysum = ysum;
    q.M = M; q.K = K;
    return act_quant(q, static_cast<cudaStream_t>(stream));
}

int bitnet_quant_input_glu(const void* x13_bf16, int64_t ldx, const void* gamma_bf16, float eps, int8_t* y, int64_t ldy,
                           float* act_scale, void* s_bf16, int32_t* ysum, int M, int K, void* stream) {
    g_status = kOk;
    if (!x13_bf16 || !y || M < 1 || K < 1 || ldx < 2 * (int64_t)K || ldy < K) return fail(kBadArgument);
    if (ldy % 8 != 0 || (reinterpret_cast<uintptr_t>(y) & 7) != 0) return fail(kBadArgument);
    QuantArgs q;
    q.x_bf16 = static_cast<const __nv_bfloat16*>(x13_bf16); q.ldx = ldx;
    q.gamma = static_cast<const __nv_bfloat16*>(gamma_bf16); q.eps = eps;
    q.y = y; q.ldy = ldy;
    q.a_f32 = act_scale; q.a_bf16 = static_cast<__nv_bfloat16*>(s_bf16); q.ysum = ysum;
    q.M = M; q.K = K; q.glu = true;
    return act_quant(q, static_cast<cudaStream_t>(stream));
}

size_t bitnet_w2t_bytes(int N, int K) {
    if (N < 1 || K < 1) return 0;
    return (size_t)(round_up(N, 16) * round_up(K, 128) / 4);
}

int bitnet_sample_top_p(const float* logits, int64_t ld, int batch, int vocab, float temperature, float top_p,
                        uint64_t seed, const int64_t* pos, const float* uniforms, int64_t* out, int64_t* tokens,
                        void* stream) {
    set_status(kOk);
    return sample_top_p(logits, ld, batch, vocab, temperature, top_p, seed, reinterpret_cast<const long long*>(pos),
                        uniforms, reinterpret_cast<long long*>(out), reinterpret_cast<long long*>(tokens),
                        static_cast<cudaStream_t>(stream));
}

int bitnet_pack_ternary(const int8_t* q, void* w2t, int N, int K, void* stream) {
    g_status = kOk;
    if (!q || !w2t || N < 1 || K < 1) return fail(kBadArgument);
    return pack_ternary_to_w2t(q, w2t, N, K, static_cast<cudaStream_t>(stream));
}

int bitnet_pack_from_i2s(const uint8_t* i2s, void* w2t, int N, int K, void* stream) {
    g_status = kOk;
    if (!i2s || !w2t || N < 1 || K < 1) return fail(kBadArgument);
    if (((int64_t)N * K) % 128 != 0) return fail(kUnsupported);
    return pack_i2s_to_w2t(i2s, w2t, N, K, static_cast<cudaStream_t>(stream));
}

int bitnet_pack_from_ref_int2(const int8_t* packed, void* w2t, int N, int K, void* stream) {
    g_status = kOk;
    if (!packed || !w2t || N < 1 || K < 1) return fail(kBadArgument);
    if (N % 16 != 0 || K % 32 != 0) return fail(kUnsupported);
    return pack_refgpu_to_w2t(packed, w2t, N, K, static_cast<cudaStream_t>(stream));
}

int bitnet_unpack_ternary(const void* w2t, int8_t* q, int N, int K, void* stream) {
    g_status = kOk;
    if (!q || !w2t || N < 1 || K < 1) return fail(kBadArgument);
    return unpack_w2t_to_ternary(w2t, q, N, K, static_cast<cudaStream_t>(stream));
}

size_t quantize_i2_s(const float* src, void* dst, int64_t nrow, int64_t n_per_row, const float* quant_weights) {
    (void)quant_weights;
    g_status = kOk;
    const int64_t n = nrow * n_per_row;
    if (!src || !dst || nrow < 1 || n_per_row < 1) return fail(kBadArgument), 0;
    if (n % 128 != 0) return fail(kUnsupported), 0;
    DeviceBuf d_src, d_dst, d_max;
    if (check_cuda(d_src.alloc(n * sizeof(float))) || check_cuda(d_dst.alloc(n / 4 + 32)) ||
        check_cuda(d_max.alloc(sizeof(uint32_t))))
        return 0;
    if (check_cuda(cudaMemcpy(d_src.p, src, n * sizeof(float), cudaMemcpyHostToDevice))) return 0;
    if (i2s_quantize(static_cast<const float*>(d_src.p), static_cast<uint8_t*>(d_dst.p), n,
                     static_cast<uint32_t*>(d_max.p), nullptr))
        return 0;
    if (check_cuda(cudaMemcpy(dst, d_dst.p, n / 4 + 32, cudaMemcpyDeviceToHost))) return 0;
    return (size_t)(n / 4 + 32);
}

void ggml_vec_dot_i2_i8_s(int n, float* s, size_t bs, const void* vx, size_t bx, const void* vy, size_t by, int nrc) {
    g_status = kOk;
    if (n < 1 || !s || !vx || !vy || nrc < 1) {
        fail(kBadArgument);
        return;
    }
    if (n % 128 != 0) {
        fail(kUnsupported);
        return;
    }
    // nrc % 4 == 0: one weight row against nrc activation rows; otherwise nrc weight rows
    // against one activation row (src/ggml-bitnet-mad.cpp:1043-1056 with :198 and :791).
    const bool act_parallel = (nrc % 4 == 0);
    const int M = act_parallel ? nrc : 1, N = act_parallel ? 1 : nrc;
    const size_t row_bytes = (size_t)n / 4;
    DeviceBuf d_x, d_w, d_y, d_zero, d_acc;
    if (check_cuda(d_x.alloc(N * row_bytes)) || check_cuda(d_w.alloc(bitnet_w2t_bytes(N, n))) ||
        check_cuda(d_y.alloc((size_t)M * n)) || check_cuda(d_zero.alloc(M * sizeof(int32_t))) ||
        check_cuda(d_acc.alloc((size_t)M * N * sizeof(int32_t))))
        return;
    if (check_cuda(cudaMemcpy2D(d_x.p, row_bytes, vx, bx / 4, row_bytes, N, cudaMemcpyHostToDevice))) return;
    if (check_cuda(cudaMemcpy2D(d_y.p, n, vy, act_parallel ? by : (size_t)n, n, M, cudaMemcpyHostToDevice))) return;
    if (check_cuda(cudaMemset(d_zero.p, 0, M * sizeof(int32_t)))) return;
    if (pack_i2s_to_w2t(static_cast<const uint8_t*>(d_x.p), d_w.p, N, n, nullptr)) return;
    LinearArgs a;
    a.w2t = d_w.p;
    a.y = static_cast<const int8_t*>(d_y.p); a.ldy = n;
    a.ysum = static_cast<const int32_t*>(d_zero.p);   // zero offset: the raw code sums are wanted
    a.acc_out = static_cast<int32_t*>(d_acc.p);
    a.M = M; a.N = N; a.K = n;
    a.seg.n_seg = 1;
    if (w2a8_gemv(a, nullptr)) return;
    std::vector<int32_t> h((size_t)M * N);
    if (check_cuda(cudaMemcpy(h.data(), d_acc.p, h.size() * sizeof(int32_t), cudaMemcpyDeviceToHost))) return;
    if (act_parallel) {
        for (int j = 0; j < M; ++j) s[(size_t)j * bs] = (float)h[j];
    } else {
        for (int r = 0; r < N; ++r) s[r] = (float)h[r];
    }
}

}  // extern "C"
