// Parameter blocks and launchers of the fused decode kernels (decode_fused.cu).
#pragma once
#include "common.cuh"

namespace bitnet {

enum SourceKind : int {
    kSrcVector = 0,      // v = x[m, k]                                   (bf16 vector)
    kSrcEmbedding = 1,   // v = embedding row of tokens[m]; the row is also copied to h_copy
    kSrcGlu = 2,         // v = relu(x[m,k])^2 * x[m,K+k]                 (gpu/model.py:193-195)
    kSrcQuantized = 3,   // int8 activations given by the caller (no norm, no quantisation)
};

enum OutKind : int {
    kOutBf16 = 0,        // out[m, n] = bf16(acc / a * ws)
    kOutResidual = 1,    // out[m, n] = bf16(out[m, n] + bf16(acc / a * ws))   (gpu/model.py:237-243)
};

struct FusedLinearParams {
    // the BitLinear
    const uint8_t* w2t;
    int N, K, k_tiles, K_even;
    int grid, tiles_base, tiles_rem, r_max, total_tiles;   // work split (plan_linear)
    int src, out_kind, M;
    // source
    const __nv_bfloat16* x;          // kSrcVector [M, ldx], kSrcGlu [M, ldx] with ldx >= 2K
    int64_t ldx;
    const int64_t* tokens;           // kSrcEmbedding
    const __nv_bfloat16* emb;
    __nv_bfloat16* h_copy;           // [M, K]
    const int8_t* yq;                // kSrcQuantized [M, ldy]
    int64_t ldy;
    const float* a_q;                // [M] f32 scales, or
    const __nv_bfloat16* a_q_bf16;   // [M] bf16 scales
    const int32_t* ysum_q;           // [M] or null
    const __nv_bfloat16* gamma;      // RMSNorm weight [K], null = no norm
    float eps;
    // output
    __nv_bfloat16* out;              // [M, ldo], null = none
    int64_t ldo;
    int32_t* acc_out;                // [M, N] exact int32 sums, null = none
    ScaleSegments seg;
    float ws[8];                     // weight scale per segment, by value, unless one of:
    const float* ws_dev_f32;         //   device array of f32 scales
    const __nv_bfloat16* ws_dev_bf16;  // device array of bf16 scales
    // scratch owned by the caller of the launcher
    unsigned long long* acc_scratch; // [ceil16(N)/16][16][8] 64-bit slots (sum + tickets), zero between launches
    int* error_flag;
    unsigned long long* trace;       // optional: 8 phase timestamps written by CTA 0
    int debug;                       // measurement aid: 1 = skip the math, 2 = skip the waits for weights
};

struct AttentionParams {
    const __nv_bfloat16* xqkv;       // [B, ld_qkv] fused q, k, v of the new token
    int64_t ld_qkv;
    const int64_t* pos;              // [B] keys already cached
    const float* rope;               // [L, D/2, 2] cos, sin
    __nv_bfloat16* cache_k;          // [B, L, Hkv, D]
    __nv_bfloat16* cache_v;
    __nv_bfloat16* out;              // [B, H*D]
    float* part_o;                   // [B, H, S, D]
    float* part_ml;                  // [B, H, S, 2]
    int* counters;                   // [B, Hkv], zero between launches
    int H, Hkv, D, L, S;
    unsigned long long* trace;       // optional: 8 phase timestamps written by CTA (0, 0)
};

struct HeadParams {
    const __nv_bfloat16* w;          // [V, K] bf16 output projection
    const __nv_bfloat16* gamma;      // final RMSNorm weight
    float eps;
    const __nv_bfloat16* h;          // [M, K]
    float* logits;                   // [M, V] or null
    float* part_val;                 // [grid, 8]
    int* part_idx;
    int M, K, V;
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
int launch_fused_linear(const FusedLinearParams& p, cudaStream_t stream, bool pdl);
// many_sequences: the 4-warp form of the kernel (see decode_fused.cu)
int launch_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl, bool many_sequences = false);
int launch_head(const HeadParams& p, int grid, cudaStream_t stream, bool pdl);
int launch_argmax(const ArgmaxParams& p, cudaStream_t stream, bool pdl);

// The whole decode step as one persistent kernel (decode_mega.cu).  mega_create builds the
// device tables from fully filled parameter blocks - lin: [n_layers][4] in the order wqkv, wo,
// w13, w2, planned for `grid` CTAs; att: [n_layers] - and returns null with the status set when
// the step does not fit that kernel.
void* mega_create(const FusedLinearParams* lin, const AttentionParams* att, const HeadParams& hp, int n_layers, int M,
                  int grid, size_t smem_optin);
bool mega_single_round(const void* plan);
void mega_destroy(void* plan);
int mega_launch(void* plan, const HeadParams& hp, int64_t* tokens, int64_t* pos, int64_t* out, int* error_flag,
                unsigned long long* trace, cudaStream_t stream);

}  // namespace bitnet
