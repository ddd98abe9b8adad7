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
    kOutTpPartial = 3,   // row-parallel shard: the exact int32 sums over this rank's K slice go to
                         // every rank's exchange area; tp_reduce_kernel adds them up and rescales
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

// Statistics of a vector that its producer kernel accumulates for the RMSNorm + int8
// quantisation in front of the next BitLinear: the sum of squares of the vector and the largest
// |x * norm weight| in it.  One slot per token; the producer's CTAs add their shares with
// atomics (a double-precision add and a max on the bit pattern of a non-negative double), the
// consumer reads one slot.  The sum is kept in double precision, which makes its f32 rounding
// independent - for all practical purposes - of the order in which the shares arrive and equal
// to what a double-precision CPU evaluation gives.  A slot is cleared by the kernel that runs
// after its consumer.
struct StatPart {
    double ss;
    double mx;
};

// ---------------------------------------------------------------------------------------
// Tensor parallelism.  Every rank owns an exchange area in its own device memory that the other
// ranks of the node map through CUDA IPC; producers store tagged packets into every rank's area
// (plain 8-byte peer stores over NVLink), consumers poll the packets in their own memory, bounded
// in time.  No multicast loads, no bulk/TMA copies from peer memory, no atomics or fences between
// GPUs.  The tags derive from the rank's own step counter on the device, so that a captured CUDA
// graph can be replayed.
// ---------------------------------------------------------------------------------------
constexpr int kMaxTp = 8;

struct TpPeers {
    int rank, size;                  // size <= 1: no tensor parallelism
    uint8_t* area[kMaxTp];           // base of every rank's exchange area as mapped in this process
};

// What crosses between ranks travels as 8-byte packets {value, tag}: one store that no fence has
// to follow, since a packet whose tag is this exchange's tag carries its value with it (8-byte
// stores arrive whole).  tag = (uint32)(*step * mul + add) is different for every exchange that
// reuses a packet's address (mul = exchanges of this kind per step, add = 1 + its number within the
// step); memory starts out zero and no tag is zero... until the counter wraps after 2^32 exchanges,
// by which time the address has long held other tags.
struct TpTag {
    const unsigned long long* step;  // this rank's step counter (device); null: no exchange
    unsigned int mul, add;
    long long limit_cycles;          // a reader gives up after this many SM clock cycles
};
// Statistics of one (rank, token): three packets {ss low word, ss high word, mx bits} + padding.
struct TpStatPackets { unsigned int w[8]; };

// ---------------------------------------------------------------------------------------
// BitLinear of the decode chain (decode_chain.cu): prologue (int8 quantisation of the normalised
// input vector) + W2A8 matmul + epilogue (rescale, residual or gate, and what the next prologue
// needs).  Whole 16-row groups belong to one CTA, so no sums cross CTAs.
//
// The input arrives as t[m, k] = x[m, k] * g[k] in f32 (x the bf16 activation, g the weight of
// the RMSNorm in front of this BitLinear, both factors bf16 values, so the product is exact)
// with the statistics of x; the kernel computes r = rsqrt(mean(x^2) + eps), xn = bf16(t * r),
// a = 127 / max|xn|, y = rint(xn * a) - the arithmetic of prologue.cuh - without touching x or g.
// ---------------------------------------------------------------------------------------
struct ChainLinearParams {
    const uint8_t* w2t;
    int N, K, k_tiles;
    int n_units, n_sub, sub_stride;  // unit u = row groups u + s * sub_stride, s < n_sub (2 for kOutGlu)
    int units_max;                   // most units a CTA owns
    int units_base, units_rem;       // CTA c owns units_base units, one more if c < units_rem
    int grid, M, ring_stages;
    int big_share;                   // a CTA's share passes through the ring more than once (set by plan_chain_linear)
    int out_kind;
    // source
    const float* t;                  // [M, ldt]
    int64_t ldt;
    const StatPart* stats_in;        // [M]
    int k_norm;                      // length of the whole normalised vector (K; more for a K slice)
    float eps;
    const TpStatPackets* tp_stats_in; // tensor parallel: [size][M] packets in this rank's area instead of stats_in
    TpTag tp_tag_in;                 //   and their tag
    StatPart* zero_slot;             // [M] slot to clear (its consumer ran before this kernel), or null
    // output
    __nv_bfloat16* out;              // [M, ldo] (kOutBf16: written; kOutResidual: updated in place; others: unused)
    int64_t ldo;
    ScaleSegments seg;
    float ws[8];                     // weight scale per segment
    const __nv_bfloat16* gamma_out;  // with t_out and stats_out: the norm weight of the next prologue over the output
    float* t_out;                    // [M, ldt_out] = output * gamma_out
    int64_t ldt_out;
    StatPart* stats_out;             // [M] slot the output's statistics are added to (in every rank's area when tp.size > 1)
    // tensor parallel
    TpPeers tp;
    size_t tp_stats_off;             // kOutGlu: TpStatPackets [size][M] in every area
    size_t tp_part_off;              // kOutTpPartial: packets {int32, tag} [size][M][N] in every area
    TpTag tp_tag_out;                // tag of what this kernel sends
    float* a_out;                    // kOutTpPartial: [M] activation scales for the reduction kernel
    unsigned int* tp_ticket;         // tensor parallel: this GPU's count of CTAs that have delivered (see tp_last_cta)
    int* error_flag;
    unsigned long long* trace;       // phase timestamps of CTA 0 (only in builds with BITNET_TRACE)
};

// First kernel of a step: h[m] = embedding row of tokens[m]; t[m] = h[m] * gamma; statistics of h[m].
struct EmbedParams {
    const int64_t* tokens;
    const __nv_bfloat16* emb;
    const __nv_bfloat16* gamma;      // attention_norm of layer 0
    __nv_bfloat16* h;                // [M, K]
    float* t;                        // [M, K]
    StatPart* stats_out;             // [M], written (not added to)
    StatPart* zero_slot;             // [M] or null
    int M, K, vocab;
    int* error_flag;
};

// Second half of a row-parallel BitLinear: out[m, n] = bf16(out[m, n] + bf16(sum_r part[r][m][n] / a[m] * ws)),
// t_out = out * gamma_out and the statistics of out.  One CTA of 256 threads per 256 rows.
struct TpReduceParams {
    const uint2* part;               // packets {int32, tag} [T][M][N] in this rank's exchange area
    TpTag tag;
    const float* a;                  // [M]
    float ws;
    __nv_bfloat16* out;              // [M, ldo], updated in place
    int64_t ldo;
    const __nv_bfloat16* gamma_out;
    float* t_out;                    // [M, ldo]
    StatPart* stats_out;             // [M], added to
    int M, N, T;
    int* error_flag;
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
    const __nv_bfloat16* gamma_out;  // norm weight over `out` (per sequence: H*D values), with t_out and stats_out
    float* t_out;                    // [B, H*D] = out * gamma_out, or null
    StatPart* stats_out;             // [B] slot the statistics of a sequence's output are added to
    StatPart* zero_slot;             // [B] slot to clear, or null
    TpPeers tp;                      // tensor parallel: the statistics go to the slot at this offset of every area
    size_t tp_stats_off;             // TpStatPackets [size][B] in every area
    TpTag tp_tag_out;
    unsigned int* tp_ticket;         // tensor parallel: this GPU's count of heads whose statistics are in stats_out
    __nv_bfloat16* tap;              // optional second copy of `out` (for checkers)
    int* error_flag;
    unsigned long long* trace;
};

struct HeadParams {
    const __nv_bfloat16* w;          // [V, K] bf16 output projection
    const __nv_bfloat16* gamma;      // final RMSNorm weight
    float eps;
    const __nv_bfloat16* h;          // [M, K]
    const StatPart* stats_in;        // [M] or null (sum of squares computed here)
    float* logits;                   // [M, V] or null
    float* part_val;                 // [grid, 8]
    int* part_idx;
    int M, K, V;
    int row_offset;                  // added to the reported indices (vocabulary slice of a rank)
    TpPeers tp;                      // tensor parallel: the per-CTA maxima go to packets [size][grid][8] of every area
    size_t tp_val_off, tp_idx_off;
    TpTag tp_tag_out;
    int* error_flag;                 // set when a bounded wait for weight rows runs out (may be null)
};

struct ArgmaxParams {
    const float* part_val;
    const int* part_idx;
    int n_part, M;
    int64_t* out;
    int64_t* tokens;
    int64_t* pos;
    TpTag tag;                       // tensor parallel: part_val / part_idx hold packets {bits, tag} of all ranks' maxima
    unsigned long long* step;        // this rank's step counter, incremented here (may be null)
    int* error_flag;
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
int launch_tp_reduce(const TpReduceParams& p, cudaStream_t stream, bool pdl);
int launch_embed(const EmbedParams& p, cudaStream_t stream, bool pdl);

size_t attention_smem(const AttentionParams& p);
size_t head_smem(const HeadParams& p);
// many_sequences: the 4-warp form of the kernel (see decode_fused.cu)
int launch_attention(const AttentionParams& p, int batch, cudaStream_t stream, bool pdl, bool many_sequences = false);
int launch_head(const HeadParams& p, int grid, cudaStream_t stream, bool pdl);
int launch_argmax(const ArgmaxParams& p, cudaStream_t stream, bool pdl);

}  // namespace bitnet
