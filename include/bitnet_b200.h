/* C ABI of libbitnet_b200.so: the W2A8 BitLinear hot path of microsoft/BitNet on NVIDIA
 * B200 (sm_100a).  Plain pointers and sizes only.  Unless a function says "host", every
 * buffer pointer is a device pointer owned by the caller; the library keeps none of them.
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Functions that
 * return int return 0 on success or one of the BITNET_STATUS_* codes; all functions also
 * record that code for bitnet_last_status().  No function aborts, traps or prints.
 *
 * Paths in the comments are relative to the microsoft/BitNet checkout. */
#ifndef BITNET_B200_H
#define BITNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BITNET_STATUS_OK            0
#define BITNET_STATUS_BAD_ARGUMENT  1
#define BITNET_STATUS_UNSUPPORTED   2
#define BITNET_STATUS_CUDA_ERROR    3
#define BITNET_STATUS_TOO_LARGE     4

/* Status of the calling thread's most recent library call.  The reference reports nothing
 * (void return, a message on stdout for an unknown shape,
 * gpu/bitnet_kernels/bitnet_kernels.cu:34-36); this is the queryable replacement. */
int bitnet_last_status(void);
const char* bitnet_status_string(int status);
/* cudaGetErrorString of the last failing CUDA call on this thread ("" if none). */
const char* bitnet_last_cuda_error(void);

/* Allocates the calling thread's current device's workspace (a few MB: the scratch of the
 * split-K epilogue and of the attention splits).  Entry points that need it allocate it on
 * first use, which must then happen outside stream capture; calling this first removes
 * that constraint.  Calls that use the workspace must be ordered on one stream per device. */
int bitnet_init(void);

/* ---- the reference's GPU entry point --------------------------------------------------
 * Replaces bitlinear_int8xint2 of gpu/bitnet_kernels/bitnet_kernels.cu:3-37, which
 * gpu/model.py:21-37 and gpu/test.py:15-29 call through ctypes with exactly these
 * arguments.
 *   input0  int8 [M,K] activations         input1  packed weights, viewed int8 [N,K/4]
 *   output0 bf16 [M,N]                     s       bf16 [M] activation scales 127/absmax
 *   ws      bf16 weight scales, one per row segment
 * output0[m,n] = bf16( float(sum_k input0[m,k]*w[n,k]) / s[m] * ws[segment(n)] ).
 * Differences from the reference: any M >= 1 and any N, K with N % 16 == 0 and
 * K % 128 == 0 are accepted (the reference takes M == 1 and ten fixed shapes); s is read
 * per token (the reference reads s[0], its only token); input1 must be in this library's
 * W2T layout, as bitnet_pack_ternary / bitnet_pack_from_ref_int2 produce it (same byte
 * count and [N,K/4] shape as the reference's layout).  Row segments follow the
 * reference's shape ladder: N/ws_num equal parts with ws_num = 3 for (N,K)=(3840,2560),
 * 2 for (13824,2560) and (20480,3200), 6 for (4800,3200), else 1
 * (gpu/bitnet_kernels/bitnet_kernels.cu:4-33, bitnet_kernels.h:80-82).
 * Asynchronous on `stream`; allocates nothing; may be captured in a CUDA graph. */
void bitlinear_int8xint2(int8_t* input0, int8_t* input1, void* output0, void* s, void* ws,
                         int M, int N, int K, void* stream);

/* ---- the same entry point for callers that must not allocate device memory ------------
 * No counterpart in the reference.  Some hosts cannot call cudaMalloc at the point where
 * they run a BitLinear: a plugin that executes inside another framework's captured CUDA
 * graph or under its own memory-pool accounting, a real-time loop that forbids driver
 * allocations after start-up, a process that runs with the device memory fully
 * pre-assigned.  The other entry points for M <= 8 take their split-K scratch from a
 * workspace that bitnet_init() (or their first call) allocates; this one takes it from a
 * 1 MB array compiled into the library, which every GPU that loads the library holds until
 * the process exits.  It calls no cudaMalloc, cudaFree or other allocating routine.
 * Same arguments, arithmetic and row-segment rule as bitlinear_int8xint2, with these limits:
 * 1 <= M <= 8, N % 16 == 0, N <= 16384, K % 128 == 0, and M, K small enough for the kernel's
 * shared memory (status BITNET_STATUS_TOO_LARGE otherwise, nothing is launched).
 * The first call on a device looks up the array's device address and configures the kernel;
 * make that call before any stream capture.  All calls share the one array: calls that
 * overlap on the GPU (different streams without ordering, or different host threads) race;
 * keep them on one stream per device.  Returns 0 or a BITNET_STATUS_* code. */
int bitlinear_int8xint2_noalloc(int8_t* input0, int8_t* input1, void* output0, void* s, void* ws,
                                int M, int N, int K, void* stream);
/* The kernel behind bitlinear_int8xint2_noalloc bounds every wait; if one ever runs out, the
 * kernel leaves a non-zero code in a word of the same fixed array and returns without
 * storing results.  This reads that word on the current device (after synchronising it):
 * 0 = no call gave up since the word was last cleared, 1 or 2 = the code of the wait that
 * did; clear != 0 resets it.  Returns -1 if the word cannot be read.  Like the call itself it
 * allocates nothing.  No counterpart in the reference. */
int bitlinear_int8xint2_noalloc_error(int clear);

/* ---- the same operation with explicit arguments ---------------------------------------
 * Serves gpu/model.py:54-75 (BitLinearKernel.forward) with the row segments stated by the
 * caller instead of guessed from the shape (for the fused wqkv the segments are the q, k
 * and v row ranges that gpu/convert_checkpoint.py:41-52 quantised separately).
 *   y        int8 [M, ldy], ldy >= K         w2t     W2T packed weights (bitnet_w2t_bytes)
 *   out_bf16 bf16 [M, ldo] or NULL           acc_out int32 [M, N] or NULL: the exact
 *                                                    sum_k y[m,k]*w[n,k]
 *   act_scale f32 [M]                        ysum    int32 [M] = sum_k y[m,k], or NULL
 *                                                    (then computed inside the kernel)
 *   w_scale  f32 [n_seg]                     seg_end host int[n_seg], seg_end[i] = first
 *                                                    row after segment i; n_seg <= 8
 * Any M >= 1, N >= 1, K >= 1 (rows beyond N and columns beyond K are padding in w2t). */
int bitnet_linear_w2a8(const int8_t* y, int64_t ldy, const void* w2t, void* out_bf16, int64_t ldo,
                       int32_t* acc_out, const float* act_scale, const int32_t* ysum,
                       const float* w_scale, const int* seg_end, int n_seg,
                       int M, int N, int K, void* stream);

/* A BitLinear whose result is added to the residual stream, fused with what follows it in a
 * decoder layer (gpu/model.py:225-227, 236-242: h = h + wo(...), then ffn_norm and the next
 * BitLinear's quant_input; likewise behind w2): h[m, :] += bf16(acc / act_scale[m] * w_scale),
 * rounded to bf16 as the reference's tensor addition rounds, and then - unless y_next is NULL -
 * the RMSNorm with gamma_bf16 and the int8 quantisation of the new h, exactly as
 * bitnet_quant_input computes them.  Two launches (tensor-core matmul, one kernel for the rest)
 * instead of four.  M >= 16; N % 8 == 0; y as for the tensor-core path of bitnet_linear_w2a8
 * (16-byte aligned rows, ldy a multiple of 16 and >= ceil128(K), zero filled beyond K); ysum is
 * required; one weight scale (wo and w2 have one row segment).  Uses the workspace. */
int bitnet_linear_w2a8_add_quant(const int8_t* y, int64_t ldy, const void* w2t, const float* act_scale,
                                 const int32_t* ysum, float w_scale, int M, int N, int K, void* h_bf16, int64_t ldh,
                                 const void* gamma_bf16, float eps, int8_t* y_next, int64_t ldy_next,
                                 float* act_scale_next, int32_t* ysum_next, void* stream);

/* Activation prologue: optional RMSNorm (gamma_bf16 != NULL; gpu/model.py:159-160,
 * 195-196, 237-242) followed by BitLinearKernel.quant_input (gpu/model.py:68-71):
 * a = 127 / max(absmax, 1e-5), y = clamp(round_half_even(x*a), -128, 127).
 *   x_bf16 bf16 [M, ldx]      y int8 [M, ldy], 8-byte aligned, ldy % 8 == 0 (bytes K..ldy-1
 *                             of each row are zeroed)
 *   act_scale f32 [M] or NULL, s_bf16 bf16 [M] or NULL (the reference's `s`),
 *   ysum int32 [M] or NULL. */
int bitnet_quant_input(const void* x_bf16, int64_t ldx, const void* gamma_bf16, float eps,
                       int8_t* y, int64_t ldy, float* act_scale, void* s_bf16, int32_t* ysum,
                       int M, int K, void* stream);
/* The same behind the gate of the feed-forward block (gpu/model.py:193-196): rows of x13_bf16
 * hold 2K values [x1 | x3] (ldx >= 2K); the value that is normalised and quantised is
 * bf16(bf16(relu(x1)^2) * x3), rounded after each step as the reference's bf16 tensor
 * operations round. */
int bitnet_quant_input_glu(const void* x13_bf16, int64_t ldx, const void* gamma_bf16, float eps,
                           int8_t* y, int64_t ldy, float* act_scale, void* s_bf16, int32_t* ysum,
                           int M, int K, void* stream);

/* ---- one decode step of the whole decoder (batch <= 8) --------------------------------
 * Counterpart of the decode model that the reference captures in a CUDA graph
 * (gpu/generate.py:159-213) around Transformer.forward_with_attn_bias (gpu/model.py:269-282):
 * one call enqueues, for every layer, wqkv -> attention -> wo -> w13 -> w2 (each BitLinear
 * fused with the rescale, residual, gate, RMSNorm and int8 quantisation around it), then the
 * bf16 output projection and the greedy choice.  Kernels are chained with programmatic
 * dependent launch; the call allocates nothing and may be captured in a CUDA graph.  All
 * pointers in the structs are device pointers that must stay valid for the decoder's lifetime. */
typedef struct bitnet_decoder_config {
    int dim, n_layers, n_heads, n_kv_heads, head_dim, ffn_dim, vocab_size;
    float norm_eps;
    int batch;          /* sequences decoded together, 1..8 */
    int max_seq_len;    /* length of the KV cache */
} bitnet_decoder_config;

typedef struct bitnet_decoder_layer {
    const void *wqkv, *wo, *w13, *w2;                  /* W2T packed weights */
    float s_q, s_k, s_v, s_o, s_1, s_3, s_2;           /* weight scales (gpu/convert_checkpoint.py:41-83) */
    const void *attention_norm, *attn_sub_norm, *ffn_norm, *ffn_sub_norm;   /* bf16 RMSNorm weights */
    void *cache_k, *cache_v;                           /* bf16 [batch, max_seq_len, n_kv_heads, head_dim] */
} bitnet_decoder_layer;

/* tok_embeddings bf16 [vocab, dim]; norm bf16 [dim]; output bf16 [vocab, dim]; rope f32
 * [max_seq_len, head_dim/2, 2] (cos, sin).  dim and ffn_dim must be multiples of 8 and 16.
 * wo maps n_heads*head_dim values to dim; the two need not be equal (a tensor-parallel shard of a
 * model, run on its own, is a valid configuration).
 * Allocates the decoder's scratch buffers (the only allocation; do it outside stream
 * capture).  Returns NULL on failure (see bitnet_last_status). */
void* bitnet_decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                            const void* tok_embeddings, const void* norm, const void* output, const float* rope);
/* tokens int64 [batch]: ids to feed (overwritten with the chosen ids, so that the next
 * call continues the sequence); pos int64 [batch]: tokens already in the cache (incremented);
 * out int64 [batch]: chosen ids; logits f32 [batch, vocab] or NULL.
 * A position outside [0, max_seq_len) or a token id outside the vocabulary is not an
 * out-of-bounds access: the kernels leave a code in the decoder's error word (see
 * bitnet_decoder_error_flag), append nothing to that sequence's cache (position) or use token 0
 * (token id), and the step's results are meaningless. */
int bitnet_decoder_step(void* decoder, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, void* stream);
/* bitnet_decoder_step followed by a wait for the stream: returns when `out` (and `logits`)
 * hold the step's result.  With `tokens` and `out` in pinned host memory (which the device can
 * address) this is the whole host-in, host-out step in one call, without copy nodes.  Not for
 * use under stream capture.  No counterpart in the reference. */
int bitnet_decoder_step_sync(void* decoder, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, void* stream);
/* The attention step of that chain on its own (batch sequences, one new token each), for
 * callers that run the decoder op by op: RoPE on q and k (adjacent pairs, as the
 * interleaved rope of gpu/model.py:144-152), append k and v to the cache at pos[b], then
 * softmax(q k^T / sqrt(head_dim)) v over keys 0..pos[b] (gpu/model.py:154-158).
 *   xqkv bf16 [batch, ld_qkv]: q heads, k heads, v heads of the new token
 *   pos int64 [batch]; rope f32 [max_seq_len, head_dim/2, 2]
 *   cache_k, cache_v bf16 [batch, max_seq_len, n_kv_heads, head_dim]; out bf16 [batch, n_heads*head_dim]
 * Uses the workspace (see bitnet_init).  A position outside the cache is flagged in the
 * workspace's error word and skipped. */
int bitnet_attention_decode(const void* xqkv, int64_t ld_qkv, const int64_t* pos, const float* rope, void* cache_k,
                            void* cache_v, void* out, int batch, int n_heads, int n_kv_heads, int head_dim,
                            int max_seq_len, void* stream);
/* The next token of every sequence drawn from its logits with a temperature and a top-p cut, on
 * the device: what the reference's decode loop does between two steps (gpu/generate.py:250-257
 * with gpu/sample_utils.py:8-30) - probs = softmax(logits / temperature), keep the most probable
 * entries whose exclusive cumulative probability does not exceed top_p, draw one of them in
 * proportion to its probability.  (temperature == 0 is the reference's argmax branch: that is
 * what bitnet_decoder_step's `out` already holds.)
 *   logits f32 [batch, ld], vocab <= ld; temperature > 0; top_p >= 0 (>= 1 keeps every entry)
 *   uniforms f32 [batch] in [0, 1), the caller's random numbers, or NULL: then sequence b draws
 *     from a counter hash of (seed, b, pos[b]) (pos int64 [batch] or NULL), which gives a new
 *     number every step when the call is replayed inside a captured graph
 *   out, tokens int64 [batch]: the chosen ids are written to both (either may be NULL)
 * One kernel, no allocation, no synchronisation. */
int bitnet_sample_top_p(const float* logits, int64_t ld, int batch, int vocab, float temperature, float top_p,
                        uint64_t seed, const int64_t* pos, const float* uniforms, int64_t* out, int64_t* tokens,
                        void* stream);
/* The decoder's error word (synchronises the device): 0, or the code of what a kernel of this
 * decoder met - 1, 2: a bounded wait for weight tiles ran out; 4: a position outside the KV
 * cache; 5: a token id outside the vocabulary. */
int bitnet_decoder_error_flag(void* decoder);
/* Clears the error word and the little state the kernels keep between launches, so that the
 * next step starts clean after an error. */
int bitnet_decoder_clear_error(void* decoder);
/* Number of kernels one step launches. */
int bitnet_decoder_kernels_per_step(void* decoder);
void bitnet_decoder_destroy(void* decoder);
/* ---- tensor-parallel decode: one process per GPU of one node ----------------------------
 * The reference has no multi-GPU path (gpu/generate.py:324-326 fixes local_rank = 0); this is
 * the partition its fused layout invites (gpu/model.py:103-118 names the per-rank head counts):
 * wqkv and w13 are split over their output rows (whole kv-head groups; matching gate and up
 * rows), wo and w2 over their input columns.  A rank gives its own shards in `layers` - wqkv
 * [(H/size + 2 Hkv/size) D, dim], wo [dim, H/size D], w13 [2 F/size, dim] (gate rows, then up
 * rows), w2 [dim, F/size], norm weights whole, its slice of the KV cache [batch, max_seq_len,
 * Hkv/size, D] - and rows [rank V/size, (rank+1) V/size) of the output projection; `cfg` holds
 * the sizes of the whole model.  The ranks exchange through device memory mapped with CUDA IPC:
 * every rank creates one exchange area (bitnet_tp_area_create), passes the 64-byte handle to
 * the others by any host channel, opens theirs (bitnet_tp_area_open) and hands all `size`
 * pointers, its own at index `rank`, to bitnet_decoder_create_tp.  Per layer a step then
 * exchanges the statistics of the attention output and of the gated vector (each rank's total
 * of sum(x^2) and max|x g| per token, 24 bytes) and the exact int32 partial sums of wo and w2;
 * the greedy choice exchanges one (value, index) pair per CTA of the output head.  Everything
 * travels as 8-byte packets {value, tag} stored into every rank's area with plain peer stores;
 * the tag numbers the exchange (it is derived from a step counter on the device, so a CUDA graph
 * of the step replays), a reader polls the packet itself, bounded in time: no collective call,
 * flag, fence or atomic is on the path between two GPUs.  Every decoder needs areas of its own,
 * freshly created (bitnet_tp_area_create zero-fills them; the tags start over with each decoder).
 * Results are bit-identical to a single GPU's.  bitnet_decoder_step / _step_sync / _error_flag
 * (code 6: an exchange did not arrive in time) / _destroy work as for a single GPU; all ranks
 * must enqueue the same steps. */
size_t bitnet_tp_area_bytes(const bitnet_decoder_config* cfg, int size);
int bitnet_tp_area_create(size_t bytes, void** area, void* ipc_handle_64);
int bitnet_tp_area_open(const void* ipc_handle_64, void** peer_area);
int bitnet_tp_area_close(void* peer_area);
int bitnet_tp_area_free(void* area);
void* bitnet_decoder_create_tp(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                               const void* tok_embeddings, const void* norm, const void* output_slice, const float* rope,
                               int rank, int size, void* const* areas);
/* How long a kernel of a tensor-parallel decoder waits for another rank's contribution before it
 * gives up, records code 6 in the error word and carries on so that the step ends (default about
 * 300 ms).  Takes effect for steps enqueued (or captured) afterwards. */
int bitnet_decoder_set_wait_limit(void* decoder, double milliseconds);

/* The error word of the workspace behind the stand-alone entry points (bitlinear_int8xint2,
 * bitnet_linear_w2a8, bitnet_attention_decode) on the current device, same codes (3: a bounded
 * wait of the tensor-core kernel ran out); clear != 0 resets it together with the workspace's
 * split-K scratch.  Synchronises the device.  -1 if it cannot be read. */
int bitnet_workspace_error(int clear);

/* ---- weight layout conversion ----------------------------------------------------------
 * Size in bytes of a W2T buffer for an [N,K] matrix: ceil16(N) * ceil128(K) / 4. */
size_t bitnet_w2t_bytes(int N, int K);
/* ternary int8 [N,K] in {-1,0,+1} (gpu/convert_checkpoint.py:23-27) -> W2T.  Replaces
 * convert_weight_int8_to_int2 of gpu/pack_weight.py:76-98. */
int bitnet_pack_ternary(const int8_t* q, void* w2t, int N, int K, void* stream);
/* I2_S bytes (src/ggml-bitnet-mad.cpp:80-88; N*K % 128 == 0) -> W2T. */
int bitnet_pack_from_i2s(const uint8_t* i2s, void* w2t, int N, int K, void* stream);
/* The reference's GPU int2 bytes (gpu/pack_weight.py:76-98; N % 16 == 0, K % 32 == 0), as
 * stored in its model_state_int2.pt checkpoints -> W2T. */
int bitnet_pack_from_ref_int2(const int8_t* packed, void* w2t, int N, int K, void* stream);
/* W2T -> ternary int8 [N,K]. */
int bitnet_unpack_ternary(const void* w2t, int8_t* q, int N, int K, void* stream);

/* ---- the reference's CPU I2_S entry points, backed by the GPU (HOST pointers) ----------
 * quantize_i2_s of src/ggml-bitnet-mad.cpp:51-96: f32 (zero or +-scale) -> I2_S bytes plus
 * the f32 scale at byte nrow*n_per_row/4; returns nrow*n_per_row/4 + 32, or 0 on failure.
 * Byte-identical to the reference's x86 ACT_PARALLEL output.  quant_weights is ignored,
 * as in the reference. */
size_t quantize_i2_s(const float* src, void* dst, int64_t nrow, int64_t n_per_row, const float* quant_weights);
/* ggml_vec_dot_i2_i8_s of src/ggml-bitnet-mad.cpp:1043-1056.  As in the reference:
 * if nrc % 4 == 0, one weight row vx against nrc activation rows (stride by bytes),
 * s[j*bs] = sum_k code_k * y_j[k]; otherwise nrc weight rows (stride bx/4 bytes) against
 * the one activation row vy, s[row] = sum.  Codes are {0,1,2,3} taken literally, no
 * offset and no scale; sums are exact (the reference's int16 lanes can wrap on extreme
 * inputs, this cannot). */
void ggml_vec_dot_i2_i8_s(int n, float* s, size_t bs, const void* vx, size_t bx,
                          const void* vy, size_t by, int nrc);

#ifdef __cplusplus
}
#endif
#endif /* BITNET_B200_H */
