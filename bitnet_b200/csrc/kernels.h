// Host-side launchers shared between the translation units of libbitnet_b200.so.
#pragma once
#include "common.cuh"

namespace bitnet {

// One BitLinear call: out[M,N] = ((y[M,K] . W[N,K]^T) / a[m]) * ws[segment(n)].
struct LinearArgs {
    const void* w2t = nullptr;          // W2T packed weights (device)
    const int8_t* y = nullptr;          // int8 activations [M, ldy] (device)
    int64_t ldy = 0;
    const int32_t* ysum = nullptr;      // optional [M]
    int32_t* acc_out = nullptr;         // optional int32 [M, N]
    __nv_bfloat16* out = nullptr;       // optional bf16 [M, ldo]
    int64_t ldo = 0;
    const float* a_f32 = nullptr;       // activation scale per token (one of the two)
    const __nv_bfloat16* a_bf16 = nullptr;
    int a_stride = 1;
    const float* ws_f32 = nullptr;      // weight scale per segment (one of the two)
    const __nv_bfloat16* ws_bf16 = nullptr;
    ScaleSegments seg{1, {0, 0, 0, 0, 0, 0, 0, 0}};
    int M = 0, N = 0, K = 0;
    // tcgen05 path only: leave the exact integer sums in the work space (`sums`: [M, N]) for a
    // kernel of the caller's that finalises them, instead of finalising here.  *sums_raw tells
    // whether sum(y) still has to be taken off (split K) or already is (one CTA per output tile).
    const int32_t** sums = nullptr;
    bool* sums_raw = nullptr;
};

int w2a8_gemv(const LinearArgs& a, cudaStream_t stream);
// The same for M <= 8 through the fused decode kernel (bulk-copy weight staging, even
// tile split); uses the per-device workspace.
int fused_linear_quantized(const LinearArgs& a, cudaStream_t stream);
// M >= 16 on tcgen05 (gemm_tc.cu).  Needs ysum, 16-byte aligned y rows padded with zeros to a
// multiple of 128 columns; error_flag is a device word set when a bounded wait gave up.
int w2a8_gemm_tc(const LinearArgs& a, int* error_flag, int32_t* acc_ws, size_t acc_ws_ints, int n_sm,
                 cudaStream_t stream);
// The per-device work space of the stand-alone entry points (allocated on first use).
struct WorkspaceView {
    int* error_flag;
    int32_t* tc_acc;          // zero between launches
    size_t tc_acc_ints;
    int32_t* ysum;            // room for the row sums of callers that pass none
    size_t ysum_ints;
    int n_sm;
};
bool workspace_view(WorkspaceView* out);
// Device buffer of at least `bytes` bytes for the re-laid-out activations of the tcgen05 kernel,
// owned by the per-device workspace.  Grows by allocation, so only outside stream capture; null
// when it cannot be had (the kernel then stages the activations itself).
uint8_t* workspace_tc_activations(size_t bytes, cudaStream_t stream);

// Packers (all buffers on the device).
int pack_ternary_to_w2t(const int8_t* q, void* w2t, int N, int K, cudaStream_t stream);
int pack_i2s_to_w2t(const uint8_t* i2s, void* w2t, int N, int K, cudaStream_t stream);
int pack_refgpu_to_w2t(const int8_t* packed, void* w2t, int N, int K, cudaStream_t stream);
int unpack_w2t_to_ternary(const void* w2t, int8_t* q, int N, int K, cudaStream_t stream);
int i2s_quantize(const float* src, uint8_t* dst, int64_t n_total, uint32_t* absmax_bits_scratch, cudaStream_t stream);

// Activation prologue: optional RMSNorm, then per-token absmax int8 quantisation.
struct QuantArgs {
    const __nv_bfloat16* x_bf16 = nullptr;
    int64_t ldx = 0;
    const __nv_bfloat16* gamma = nullptr;    // RMSNorm weight [K] or null (no norm)
    float eps = 1e-5f;
    int8_t* y = nullptr;
    int64_t ldy = 0;                         // >= K, multiple of 8; bytes [K, ldy) are zero-filled
    float* a_f32 = nullptr;                  // optional [M]
    __nv_bfloat16* a_bf16 = nullptr;         // optional [M]
    int32_t* ysum = nullptr;                 // optional [M]
    int M = 0, K = 0;
    bool glu = false;                        // rows hold 2K values: quantise relu(x[k])^2 * x[K + k] (gpu/model.py:193-195)
    // Fused form behind a BitLinear whose result is added to the residual stream: the row is
    // x[m, k] += bf16( (lin_acc[m, k] - lin_ysum[m]?) / lin_a[m] * lin_ws ) first (x_bf16 is then
    // updated in place and lin_acc is cleared), and quantised afterwards unless y is null.
    int32_t* lin_acc = nullptr;              // [M, K] integer sums of the preceding BitLinear, or null
    const int32_t* lin_ysum = nullptr;       // [M] sums still to be taken off, or null
    const float* lin_a = nullptr;            // [M] its activation scales
    float lin_ws = 1.f;                      // its weight scale
};
int act_quant(const QuantArgs& a, cudaStream_t stream);

// Temperature + top-p sampling of one token per sequence from f32 logits [batch, ld] (sample.cu).
int sample_top_p(const float* logits, long long ld, int batch, int vocab, float temperature, float top_p,
                 unsigned long long seed, const long long* pos, const float* uniforms, long long* out,
                 long long* tokens, cudaStream_t stream);

}  // namespace bitnet
