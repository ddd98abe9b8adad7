// Parameter blocks and launchers of the fused decode kernels (decode_fused.cu, decode_chain.cu).
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
    kOutGlu = 2,         // rows n and n + N/2 are gate and up: out[m, n] = bf16(bf16(relu(g)^2) * u)
                         // (gpu/model.py:193-195), n < N/2
};

// Error codes that kernels leave in their error word.
enum KernelError : int {
    kErrProducerWait = 1,    // the weight producer gave up waiting for a free ring stage
    kErrConsumerWait = 2,    // a consumer gave up waiting for weights
    kErrTensorCoreWait = 3,  // the tcgen05 kernel gave up on one of its barriers
    kErrPosition = 4,        // a position outside the KV cache (nothing was appended, no attention)
    kErrToken = 5,           // a token id outside the vocabulary (token 0 was used)
    kErrPeerWait = 6,        // a tensor-parallel exchange did not arrive in time
};

// ---------------------------------------------------------------------------------------
// The stand-alone fused BitLinear on caller-quantised activations (decode_fused.cu): even
// tile split over the CTAs, split-K through a scratch buffer.
// ---------------------------------------------------------------------------------------
struct FusedLinearParams {
    const uint8_t* w2t;
    int N, K, k_tiles, K_even;
    int grid, tiles_base, tiles_rem, r_max, total_tiles;   // work split (plan_linear)
    int M;
    const int8_t* yq;                // [M, ldy]
    int64_t ldy;
    const float* a_q;                // [M] f32 scales, or
    const __nv_bfloat16* a_q_bf16;   // [M] bf16 scales
    const int32_t* ysum_q;           // [M] or null
    __nv_bfloat16* out;              // [M, ldo], null = none
    int64_t ldo;
    int32_t* acc_out;                // [M, N] exact int32 sums, null = none
    ScaleSegments seg;
    const float* ws_dev_f32;         // device array of f32 scales, or
    const __nv_bfloat16* ws_dev_bf16;  // device array of bf16 scales
    // scratch owned by the caller of the launcher
    unsigned long long* acc_scratch; // [ceil16(N)/16][16][8] 64-bit slots (sum + tickets), zero between launches
    int* error_flag;
};

// Partial statistics of a vector that a producer kernel publishes for the RMSNorm + int8
// quantisation in front of the next BitLinear: the sum of squares of a slice of the vector
// and the largest |x * norm weight| in it.  Sums are kept in double precision, which makes
// the total independent (to the last bit of its f32 rounding, for all practical purposes) of
// how the vector was cut into slices and of the order in which they are added.
struct StatPart {
    double ss;
    double mx;
};

// ---------------------------------------------------------------------------------------
// BitLinear of the decode chain (decode_chain.cu): prologue (RMSNorm + int8 quantisation of
// the input vector) + W2A8 matmul + epilogue (rescale, residual or gate, statistics for the
// next prologue).  Whole 16-row groups belong to one CTA, so no sums cross CTAs.
// ---------------------------------------------------------------------------------------
struct ChainLinearParams {
    const uint8_t* w2t;
    int N, K, k_tiles;
    int n_units, n_sub, sub_stride;  // unit u = row groups u + s * sub_stride, s < n_sub (2 for kOutGlu)
    int units_max;                   // most units a CTA owns
    int grid, M, ring_stages;
    int src, out_kind;
    // source
    const __nv_bfloat16* x;          // kSrcVector [M, ldx]
    int64_t ldx;
    const int64_t* tokens;           // kSrcEmbedding
    const __nv_bfloat16* emb;
    __nv_bfloat16* h_copy;           // [M, K]
    int vocab;
    const __nv_bfloat16* gamma;      // RMSNorm weight [K], null = no norm
    float eps;
    const StatPart* stats_in;        // [M][n_stats_in] from the producer of x, null = computed here
    int n_stats_in;
    // output
    __nv_bfloat16* out;              // [M, ldo]
    int64_t ldo;
    ScaleSegments seg;
    float ws[8];                     // weight scale per segment
    const __nv_bfloat16* gamma_out;  // norm weight of the next prologue over `out`, with stats_out
    StatPart* stats_out;             // [M][n_units] or null
    int* error_flag;
    unsigned long long* trace;       // phase timestamps of CTA 0 (only in builds with BITNET_TRACE)
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
    const __nv_bfloat16* gamma_out;  // norm weight over `out` (per sequence: H*D values), with stats_out
    StatPart* stats_out;             // [B][H] or null
    __nv_bfloat16* tap;              // optional second copy of `out` (for checkers)
    int* error_flag;
    unsigned long long* trace;
};

struct HeadParams {
    const __nv_bfloat16* w;          // [V, K] bf16 output projection
    const __nv_bfloat16* gamma;      // final RMSNorm weight
    float eps;
    const __nv_bfloat16* h;          // [M, K]
    const StatPart* stats_in;        // [M][n_stats_in] or null (sum of squares computed here)
    int n_stats_in;
    float* logits;                   // [M, V] or null
    float* part_val;                 // [grid, 8]
    int* part_idx;
    int M, K, V;
    int row_offset;                  // added to the reported indices (vocabulary slice of a rank)
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
int prepare_fused_kernels(size_t max_linear_smem, size_t max_attn_smem, size_t max_head_smem);
int launch_fused_linear(const FusedLinearParams& p, cudaStream_t stream, bool pdl);

void plan_chain_linear(ChainLinearParams& p, int n_sm);
size_t chain_linear_smem(const ChainLinearParams& p);
size_t chain_attention_smem(const AttentionParams& p);
int prepare_chain_kernels(size_t smem_optin);
int launch_chain_linear(const ChainLinearParams& p, cudaStream_t stream, bool pdl);
int launch_chain_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl);

size_t attention_smem(const AttentionParams& p);
size_t head_smem(const HeadParams& p);
// many_sequences: the 4-warp form of the kernel (see decode_fused.cu)
int launch_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl, bool many_sequences = false);
int launch_head(const HeadParams& p, int grid, cudaStream_t stream, bool pdl);
int launch_argmax(const ArgmaxParams& p, cudaStream_t stream, bool pdl);

}  // namespace bitnet
