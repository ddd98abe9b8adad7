// Parameter blocks and launchers of the fused decode-step kernels (decode_fused.cu).
#pragma once
#include "common.cuh"

namespace bitnet {

enum SourceKind : int {
    kSrcEmbedding = 0,   // v = embedding row of the token                         (first layer's wqkv)
    kSrcResidual = 1,    // v = h_in + rescale(acc_in)                             (wqkv of later layers, w13)
    kSrcGlu = 2,         // v = relu(x1)^2 * x3 with x1, x3 = rescale(acc_in)       (w2)
    kSrcAttention = 3,   // v = attention output, KV splits combined               (wo)
};

struct FusedLinearParams {
    // this BitLinear
    const uint8_t* w2t;
    int N, K, k_tiles, K_even;
    int grid, tiles_base, tiles_rem, r_max;      // work split (plan_linear)
    int src;
    int M;
    const __nv_bfloat16* gamma;                  // RMSNorm weight [K]
    float eps;
    int32_t* acc_out;                            // [M, N] int32, accumulated with red.add (zero on entry)
    float* a_out;                                // [M] activation scale of this BitLinear's input
    int32_t* zero_buf;                           // buffer this kernel clears after its dependency wait
    int zero_count;
    int* error_flag;
    // source operands
    const int64_t* tokens;                       // kSrcEmbedding
    const __nv_bfloat16* emb;
    const __nv_bfloat16* h_in;                   // kSrcResidual
    __nv_bfloat16* h_out;                        // new residual stream (kSrcEmbedding, kSrcResidual)
    const int32_t* acc_in;                       // previous BitLinear's int32 sums
    int ld_acc_in;
    const float* a_in;                           // previous BitLinear's activation scales [M]
    float ws_in[2];                              // previous BitLinear's weight scale(s)
    const float* part_o;                         // kSrcAttention: [M, H, S, D] normalised partial outputs
    const float* part_ml;                        //                [M, H, S, 2] (max, sum)
    int S, H, D;
};

struct AttentionParams {
    const int32_t* acc_qkv;                      // [B, ld_acc] sums of the fused wqkv
    int ld_acc;
    const float* a_in;                           // [B]
    float ws_q, ws_k, ws_v;
    const int64_t* pos;                          // [B] keys already cached
    const float* rope;                           // [L, D/2, 2] cos, sin
    __nv_bfloat16* cache_k;                      // [B, L, Hkv, D]
    __nv_bfloat16* cache_v;
    float* part_o;
    float* part_ml;
    int H, Hkv, D, L, S;
    int32_t* zero_buf;
    int zero_count;
};

struct HeadParams {
    const __nv_bfloat16* w;                      // [V, K] bf16 output projection
    const __nv_bfloat16* gamma;                  // final RMSNorm weight
    float eps;
    const __nv_bfloat16* h_in;                   // [M, K]
    const int32_t* acc_in;                       // last w2's sums [M, K]
    const float* a_in;
    float ws_in;
    float* logits;                               // [M, V] or null
    float* part_val;                             // [grid, 8]
    int* part_idx;
    int M, K, V;
    int32_t* zero_buf;
    int zero_count;
};

struct ArgmaxParams {
    const float* part_val;
    const int* part_idx;
    int n_part, M;
    int64_t* out;
    int64_t* tokens;
    int64_t* pos;
};

void plan_linear(FusedLinearParams& p, int n_sm);
size_t fused_linear_smem(const FusedLinearParams& p);
size_t attention_smem(const AttentionParams& p);
size_t head_smem(const HeadParams& p);
int prepare_fused_kernels(size_t max_linear_smem, size_t max_attn_smem, size_t max_head_smem);
int launch_fused_linear(const FusedLinearParams& p, cudaStream_t stream);
int launch_attention(const AttentionParams& p, int batch, cudaStream_t stream);
int launch_head(const HeadParams& p, int grid, cudaStream_t stream);
int launch_argmax(const ArgmaxParams& p, cudaStream_t stream);

}  // namespace bitnet
