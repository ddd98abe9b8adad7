// Host side of the fused decode kernels: the per-device workspace behind the stand-alone
// entry points, and the decode-step object behind bitnet_decoder_create / _step / _destroy,
// which owns its scratch and enqueues one step - five kernels per layer, then the output
// head and the greedy choice - on the caller's stream.
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <new>
#include <vector>

#include "../../include/bitnet_b200.h"
#include "common.cuh"
#include "decode_fused.h"
#include "kernels.h"

namespace bitnet {

// ---------------------------------------------------------------------------------------
// Per-device workspace of the stand-alone fused kernels.  Allocated on first use on a
// device (bitnet_init does it explicitly); the first use must therefore happen outside
// stream capture.  Calls that share it must be ordered on one stream.
// ---------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
constexpr int kWsRowGroups = 1 << 15;             // BitLinear outputs up to 524288 rows
constexpr size_t kWsYsumInts = 1 << 16;           // row sums for up to 65536 tokens

struct Workspace {
    bool ready = false;
    int n_sm = 0;
    size_t smem_optin = 0;
    unsigned long long* acc_scratch = nullptr;    // [kWsRowGroups][16][8]
    int* error_flag = nullptr;
    float* attn_part = nullptr;                   // attention split partials, grown on demand
    size_t attn_part_bytes = 0;
    int* attn_counters = nullptr;                 // [4096]
    int32_t* tc_acc = nullptr;                    // split-K sums of the tcgen05 kernel, zero between launches
    size_t tc_acc_ints = 0;
    int32_t* ysum = nullptr;                      // row sums computed for callers that pass none
    uint8_t* tc_y = nullptr;                      // activations in operand layout (tcgen05 kernel), grown on demand
    size_t tc_y_bytes = 0;
};

static Workspace g_ws[kMaxDevices];
static std::mutex g_ws_mutex;

Workspace* workspace() {
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev))) return nullptr;
    if (dev < 0 || dev >= kMaxDevices) return set_status(kUnsupported), nullptr;
    Workspace& w = g_ws[dev];
    if (w.ready) return &w;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (w.ready) return &w;
    cudaDeviceProp prop;
    if (check_cuda(cudaGetDeviceProperties(&prop, dev))) return nullptr;
    w.n_sm = prop.multiProcessorCount;
    w.smem_optin = prop.sharedMemPerBlockOptin;
    const size_t acc_bytes = (size_t)kWsRowGroups * 128 * 8, ctr_bytes = 0;
    uint8_t* base = nullptr;
    const size_t tc_ints = (size_t)4 << 20;    // 16 MB: up to 128 tokens x 32768 rows
    const size_t total = acc_bytes + ctr_bytes + 4096 * 4 + 256 + tc_ints * 4 + kWsYsumInts * 4;
    if (check_cuda(cudaMalloc(&base, total)) || check_cuda(cudaMemset(base, 0, total))) return nullptr;
    w.acc_scratch = reinterpret_cast<unsigned long long*>(base);
    w.attn_counters = reinterpret_cast<int*>(base + acc_bytes + ctr_bytes);
    w.error_flag = reinterpret_cast<int*>(base + acc_bytes + ctr_bytes + 4096 * 4);
    w.tc_acc = reinterpret_cast<int32_t*>(base + acc_bytes + ctr_bytes + 4096 * 4 + 256);
    w.tc_acc_ints = tc_ints;
    w.ysum = w.tc_acc + tc_ints;
    if (prepare_fused_kernels(w.smem_optin, 96 * 1024, w.smem_optin)) return nullptr;
    w.ready = true;
    return &w;
}

bool workspace_view(WorkspaceView* out) {
    Workspace* w = workspace();
    if (!w) return false;
    *out = WorkspaceView{w->error_flag, w->tc_acc, w->tc_acc_ints, w->ysum, kWsYsumInts, w->n_sm};
    return true;
}

uint8_t* workspace_tc_activations(size_t bytes, cudaStream_t stream) {
    Workspace* w = workspace();
    if (!w) return nullptr;
    if (bytes <= w->tc_y_bytes) return w->tc_y;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;                           // no allocation while a graph is being captured
    }
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (bytes > w->tc_y_bytes) {
        uint8_t* nb = nullptr;
        const size_t want = bytes + bytes / 4;
        if (cudaMalloc(&nb, want) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        w->tc_y = nb;                             // the old buffer may still be in use by enqueued work: it is kept
        w->tc_y_bytes = want;
    }
    return w->tc_y;
}

// BitLinear on caller-quantised activations through the fused kernel (M <= 8).
int fused_linear_quantized(const LinearArgs& a, cudaStream_t stream) {
    Workspace* w = workspace();
    if (!w) return bitnet_last_status();
    if ((a.N + 15) / 16 > kWsRowGroups) return set_status(kTooLarge), kTooLarge;
    FusedLinearParams p{};
    p.w2t = static_cast<const uint8_t*>(a.w2t);
    p.N = a.N; p.K = a.K; p.M = a.M;
    p.src = kSrcQuantized; p.out_kind = kOutBf16;
    plan_linear(p, w->n_sm);
    p.yq = a.y; p.ldy = a.ldy; p.a_q = a.a_f32; p.a_q_bf16 = a.a_bf16; p.ysum_q = a.ysum;
    p.out = a.out; p.ldo = a.ldo; p.acc_out = a.acc_out;
    p.seg = a.seg;
    if (fused_linear_smem(p) > w->smem_optin) return set_status(kTooLarge), kTooLarge;
    p.ws_dev_f32 = a.ws_f32; p.ws_dev_bf16 = a.ws_bf16;
    p.acc_scratch = w->acc_scratch; p.error_flag = w->error_flag;
    return launch_fused_linear(p, stream, false);
}

struct Decoder {
    bitnet_decoder_config cfg{};
    std::vector<bitnet_decoder_layer> layers;
    const __nv_bfloat16* emb = nullptr;
    const __nv_bfloat16* final_norm = nullptr;
    const __nv_bfloat16* output = nullptr;
    const float* rope = nullptr;
    int device = 0, n_sm = 0, kv_splits = 1, head_grid = 0;
    void* scratch = nullptr;
    unsigned long long* acc_scratch = nullptr;
    int *attn_counters = nullptr, *error_flag = nullptr, *part_idx = nullptr;
    __nv_bfloat16 *h = nullptr, *xqkv = nullptr, *attn_out = nullptr, *x13 = nullptr;
    float *part_o = nullptr, *part_ml = nullptr, *part_val = nullptr;
    unsigned long long* trace = nullptr;          // [n_layers * 4][8] phase timestamps (measurement aid)
    FusedLinearParams plan_qkv{}, plan_o{}, plan_13{}, plan_2{};
    void* mega = nullptr;                         // tables of the persistent kernel, when it fits this model
    bool use_mega = false;
    bool trace_chain = false;                     // BITNET_TRACE=chain: time-stamp the chain (which then is the default)
};

static size_t align_up(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace bitnet

using namespace bitnet;

extern "C" {

int bitnet_init(void) {
    set_status(kOk);
    return workspace() ? kOk : bitnet_last_status();
}

static void layer_params(const Decoder* d, int l, const int64_t* tokens, const int64_t* pos, FusedLinearParams lin[4],
                         AttentionParams* ap);
static HeadParams head_params(const Decoder* d, float* logits);

void* bitnet_decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                            const void* tok_embeddings, const void* norm, const void* output, const float* rope) {
    set_status(kOk);
    if (!cfg || !layers || !tok_embeddings || !norm || !output || !rope) return set_status(kBadArgument), nullptr;
    const int B = cfg->batch, D = cfg->head_dim, H = cfg->n_heads, Hkv = cfg->n_kv_heads;
    if (B < 1 || B > 8 || cfg->n_layers < 1 || H < 1 || Hkv < 1 || H % Hkv != 0 || H / Hkv > 16 || D % 4 != 0 ||
        D > 128 || cfg->dim % 8 != 0 || cfg->dim != H * D || cfg->ffn_dim % 8 != 0 || cfg->max_seq_len < 2)
        return set_status(kUnsupported), nullptr;
    Decoder* d = new (std::nothrow) Decoder();
    if (!d) return set_status(kBadArgument), nullptr;
    d->cfg = *cfg;
    d->layers.assign(layers, layers + cfg->n_layers);
    d->emb = static_cast<const __nv_bfloat16*>(tok_embeddings);
    d->final_norm = static_cast<const __nv_bfloat16*>(norm);
    d->output = static_cast<const __nv_bfloat16*>(output);
    d->rope = rope;
    cudaDeviceProp prop;
    if (check_cuda(cudaGetDevice(&d->device)) || check_cuda(cudaGetDeviceProperties(&prop, d->device))) {
        delete d;
        return nullptr;
    }
    d->n_sm = prop.multiProcessorCount;
    int s = d->n_sm / (Hkv * B);
    d->kv_splits = s < 1 ? 1 : (s > 16 ? 16 : s);
    d->head_grid = d->n_sm;

    const int dim = cfg->dim, F = cfg->ffn_dim, Nqkv = (H + 2 * Hkv) * D;
    // CTAs per SM for the BitLinear kernels (measurement knob; 1 leaves room for the successor's
    // CTAs to become resident early and prefetch their weights)
    const int ctas_per_sm = getenv("BITNET_CTAS_PER_SM") ? atoi(getenv("BITNET_CTAS_PER_SM")) : 1;
    auto plan = [&](FusedLinearParams& p, int N, int K, int src, int out_kind) {
        p = FusedLinearParams{};
        p.N = N; p.K = K; p.src = src; p.out_kind = out_kind; p.M = B; p.eps = cfg->norm_eps;
        plan_linear(p, d->n_sm * (ctas_per_sm > 0 ? ctas_per_sm : 1));
    };
    plan(d->plan_qkv, Nqkv, dim, kSrcVector, kOutBf16);
    plan(d->plan_o, dim, dim, kSrcVector, kOutResidual);
    plan(d->plan_13, 2 * F, dim, kSrcVector, kOutBf16);
    plan(d->plan_2, dim, F, kSrcGlu, kOutResidual);

    AttentionParams ap{};
    ap.H = H; ap.Hkv = Hkv; ap.D = D; ap.S = d->kv_splits;
    HeadParams hp{};
    hp.M = B; hp.K = dim; hp.V = cfg->vocab_size;
    size_t lin_smem = 0;
    for (const FusedLinearParams* p : {&d->plan_qkv, &d->plan_o, &d->plan_13, &d->plan_2})
        lin_smem = fused_linear_smem(*p) > lin_smem ? fused_linear_smem(*p) : lin_smem;
    if (lin_smem > (size_t)prop.sharedMemPerBlockOptin || head_smem(hp) > (size_t)prop.sharedMemPerBlockOptin ||
        attention_smem(ap) > (size_t)prop.sharedMemPerBlockOptin) {
        delete d;
        return set_status(kTooLarge), nullptr;
    }
    if (!workspace()) {   // also sets the kernels' shared memory limits for this device
        delete d;
        return nullptr;
    }

    // one zero-initialised scratch allocation
    const int max_rg = ((2 * F > Nqkv ? 2 * F : Nqkv) + 15) / 16;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return o; };
    const size_t o_acc = take((size_t)max_rg * 128 * 8),
                 o_actr = take((size_t)B * Hkv * 4), o_err = take(4), o_h = take((size_t)B * dim * 2),
                 o_qkv = take((size_t)B * Nqkv * 2), o_att = take((size_t)B * dim * 2),
                 o_13 = take((size_t)B * 2 * F * 2), o_po = take((size_t)B * H * d->kv_splits * D * 4),
                 o_pml = take((size_t)B * H * d->kv_splits * 2 * 4), o_pv = take((size_t)d->head_grid * 8 * 4),
                 o_pi = take((size_t)d->head_grid * 8 * 4), o_tr = take((size_t)cfg->n_layers * 5 * 16 * 8);
    if (check_cuda(cudaMalloc(&d->scratch, off)) || check_cuda(cudaMemset(d->scratch, 0, off))) {
        delete d;
        return nullptr;
    }
    uint8_t* base = static_cast<uint8_t*>(d->scratch);
    d->acc_scratch = reinterpret_cast<unsigned long long*>(base + o_acc);
    d->attn_counters = reinterpret_cast<int*>(base + o_actr);
    d->error_flag = reinterpret_cast<int*>(base + o_err);
    d->h = reinterpret_cast<__nv_bfloat16*>(base + o_h);
    d->xqkv = reinterpret_cast<__nv_bfloat16*>(base + o_qkv);
    d->attn_out = reinterpret_cast<__nv_bfloat16*>(base + o_att);
    d->x13 = reinterpret_cast<__nv_bfloat16*>(base + o_13);
    d->part_o = reinterpret_cast<float*>(base + o_po);
    d->part_ml = reinterpret_cast<float*>(base + o_pml);
    d->part_val = reinterpret_cast<float*>(base + o_pv);
    d->part_idx = reinterpret_cast<int*>(base + o_pi);
    if (getenv("BITNET_TRACE")) {
        d->trace = reinterpret_cast<unsigned long long*>(base + o_tr);
        d->trace_chain = strcmp(getenv("BITNET_TRACE"), "chain") == 0;
    }

    // The persistent single-kernel step, when the model fits it and the chain's plans use one
    // CTA per SM.  The chain of kernels is the default (it is the faster one on B200, by 7 % for
    // the 2B architecture); BITNET_PERSISTENT=1 or bitnet_decoder_use_persistent select the
    // persistent kernel.
    if (ctas_per_sm <= 1 && !getenv("BITNET_NO_PERSISTENT")) {
        std::vector<FusedLinearParams> lin((size_t)cfg->n_layers * 4);
        std::vector<AttentionParams> att(cfg->n_layers);
        for (int l = 0; l < cfg->n_layers; ++l) layer_params(d, l, nullptr, nullptr, &lin[(size_t)l * 4], &att[l]);
        d->mega = mega_create(lin.data(), att.data(), head_params(d, nullptr), cfg->n_layers, B, d->n_sm,
                              prop.sharedMemPerBlockOptin);
        set_status(kOk);   // not fitting the persistent kernel is not an error: the chain remains
        const char* env = getenv("BITNET_PERSISTENT");
        d->use_mega = d->mega && env && atoi(env) != 0 && !d->trace_chain;
    }
    return d;
}

// Parameter blocks of layer l: lin[0..3] = wqkv, wo, w13, w2 and the attention between the
// first two.  `tokens` and `pos` may be null when the caller supplies them at launch.
static void layer_params(const Decoder* d, int l, const int64_t* tokens, const int64_t* pos, FusedLinearParams lin[4],
                         AttentionParams* ap) {
    const bitnet_decoder_config& c = d->cfg;
    const int D = c.head_dim, H = c.n_heads, Hkv = c.n_kv_heads, dim = c.dim, F = c.ffn_dim;
    const int Nqkv = (H + 2 * Hkv) * D;
    const bitnet_decoder_layer& L = d->layers[l];
    auto common = [&](FusedLinearParams& p, const void* w, const void* gamma) {
        p.w2t = static_cast<const uint8_t*>(w);
        p.gamma = static_cast<const __nv_bfloat16*>(gamma);
        p.acc_scratch = d->acc_scratch; p.error_flag = d->error_flag;
    };
    // wqkv: (embedding ->) h -> attention_norm -> wqkv -> xqkv
    FusedLinearParams& q = lin[0];
    q = d->plan_qkv;
    common(q, L.wqkv, L.attention_norm);
    if (l == 0) {
        q.src = kSrcEmbedding;
        q.tokens = tokens; q.emb = d->emb; q.h_copy = d->h;
    } else {
        q.x = d->h; q.ldx = dim;
    }
    q.out = d->xqkv; q.ldo = Nqkv;
    q.seg.n_seg = 3; q.seg.end[0] = H * D; q.seg.end[1] = (H + Hkv) * D; q.seg.end[2] = Nqkv;
    q.ws[0] = L.s_q; q.ws[1] = L.s_k; q.ws[2] = L.s_v;

    *ap = AttentionParams{};
    ap->xqkv = d->xqkv; ap->ld_qkv = Nqkv; ap->pos = pos; ap->rope = d->rope;
    ap->cache_k = static_cast<__nv_bfloat16*>(L.cache_k); ap->cache_v = static_cast<__nv_bfloat16*>(L.cache_v);
    ap->out = d->attn_out; ap->part_o = d->part_o; ap->part_ml = d->part_ml; ap->counters = d->attn_counters;
    ap->H = H; ap->Hkv = Hkv; ap->D = D; ap->L = c.max_seq_len; ap->S = d->kv_splits;

    // wo: attention output -> attn_sub_norm -> wo -> h += ...
    FusedLinearParams& o = lin[1];
    o = d->plan_o;
    common(o, L.wo, L.attn_sub_norm);
    o.x = d->attn_out; o.ldx = dim;
    o.out = d->h; o.ldo = dim;
    o.seg.n_seg = 1; o.seg.end[0] = dim; o.ws[0] = L.s_o;

    // w13: h -> ffn_norm -> w13 -> x13
    FusedLinearParams& u = lin[2];
    u = d->plan_13;
    common(u, L.w13, L.ffn_norm);
    u.x = d->h; u.ldx = dim;
    u.out = d->x13; u.ldo = 2 * F;
    u.seg.n_seg = 2; u.seg.end[0] = F; u.seg.end[1] = 2 * F; u.ws[0] = L.s_1; u.ws[1] = L.s_3;

    // w2: relu(x1)^2 * x3 -> ffn_sub_norm -> w2 -> h += ...
    FusedLinearParams& w = lin[3];
    w = d->plan_2;
    common(w, L.w2, L.ffn_sub_norm);
    w.x = d->x13; w.ldx = 2 * F;
    w.out = d->h; w.ldo = dim;
    w.seg.n_seg = 1; w.seg.end[0] = dim; w.ws[0] = L.s_2;
}

static HeadParams head_params(const Decoder* d, float* logits) {
    HeadParams hp{};
    hp.w = d->output; hp.gamma = d->final_norm; hp.eps = d->cfg.norm_eps;
    hp.h = d->h; hp.logits = logits; hp.part_val = d->part_val; hp.part_idx = d->part_idx;
    hp.M = d->cfg.batch; hp.K = d->cfg.dim; hp.V = d->cfg.vocab_size;
    return hp;
}

static int enqueue_step(Decoder* d, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, cudaStream_t stream,
                        bool linears_only) {
    const bitnet_decoder_config& c = d->cfg;
    if (d->mega && d->use_mega && !linears_only) {
        const int rc = mega_launch(d->mega, head_params(d, logits), tokens, pos, out, d->error_flag, d->trace, stream);
        if (rc == kOk) return rc;
        // The cooperative launch was refused (e.g. the device cannot hold all CTAs at once right
        // now): nothing ran; take the chain of kernels from here on.
        cudaGetLastError();
        set_status(kOk);
        d->use_mega = false;
    }
    static const int dbg = getenv("BITNET_DEBUG_SKIP") ? atoi(getenv("BITNET_DEBUG_SKIP")) : 0;
    for (int l = 0; l < c.n_layers; ++l) {
        FusedLinearParams lin[4];
        AttentionParams ap;
        layer_params(d, l, tokens, pos, lin, &ap);
        for (int j = 0; j < 4; ++j) {
            lin[j].trace = d->trace ? d->trace + 16 * (4 * l + j) : nullptr;
            lin[j].debug = dbg;
        }
        ap.trace = d->trace ? d->trace + 16 * (c.n_layers * 4 + l) : nullptr;
        if (launch_fused_linear(lin[0], stream, true)) return bitnet_last_status();
        if (!linears_only && launch_attention(ap, c.batch, stream, true)) return bitnet_last_status();
        for (int j = 1; j < 4; ++j)
            if (launch_fused_linear(lin[j], stream, true)) return bitnet_last_status();
    }
    if (linears_only) return kOk;
    if (launch_head(head_params(d, logits), d->head_grid, stream, true)) return bitnet_last_status();
    ArgmaxParams am{};
    am.part_val = d->part_val; am.part_idx = d->part_idx; am.n_part = d->head_grid; am.M = c.batch;
    am.out = out; am.tokens = tokens; am.pos = pos;
    return launch_argmax(am, stream, true);
}

// Chooses between the single persistent kernel (on = 1) and the chain of kernels (on = 0) for
// bitnet_decoder_step.  Returns the mode now in effect: 0 when the persistent kernel is not
// available for this model (see mega_create).
int bitnet_decoder_use_persistent(void* dec, int on) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return 0;
    d->use_mega = on != 0 && d->mega != nullptr;
    return d->use_mega ? 1 : 0;
}

int bitnet_decoder_step(void* dec, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, void* stream) {
    set_status(kOk);
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !tokens || !pos || !out) return set_status(kBadArgument), kBadArgument;
    return enqueue_step(d, tokens, pos, out, logits, static_cast<cudaStream_t>(stream), false);
}

int bitnet_decoder_step_sync(void* dec, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, void* stream) {
    const int rc = bitnet_decoder_step(dec, tokens, pos, out, logits, stream);
    if (rc != kOk) return rc;
    return check_cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}

int bitnet_decoder_bench_linears(void* dec, int64_t* tokens, void* stream) {
    set_status(kOk);
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !tokens) return set_status(kBadArgument), kBadArgument;
    return enqueue_step(d, tokens, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream), true);
}

int bitnet_decoder_error_flag(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return -1;
    int v = -1;
    if (check_cuda(cudaMemcpy(&v, d->error_flag, sizeof(int), cudaMemcpyDeviceToHost))) return -1;
    return v;
}

int bitnet_decoder_read_trace(void* dec, unsigned long long* host_out, int n_values) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !d->trace || !host_out) return set_status(kBadArgument), kBadArgument;
    const int have = d->cfg.n_layers * 5 * 16;
    return check_cuda(cudaMemcpy(host_out, d->trace, sizeof(unsigned long long) * (n_values < have ? n_values : have),
                                 cudaMemcpyDeviceToHost));
}

int bitnet_debug_read_workspace_words(unsigned long long* host_out, int n_words) {
    Workspace* w = workspace();
    if (!w || !host_out || n_words < 1 || n_words > 24) return set_status(kBadArgument), kBadArgument;
    return check_cuda(cudaMemcpy(host_out, reinterpret_cast<unsigned long long*>(w->error_flag + 16),
                                 sizeof(unsigned long long) * n_words, cudaMemcpyDeviceToHost));
}

int bitnet_decoder_kernels_per_step(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return 0;
    return d->use_mega ? 1 : 5 * d->cfg.n_layers + 2;
}

void bitnet_decoder_destroy(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return;
    if (d->scratch) cudaFree(d->scratch);
    mega_destroy(d->mega);
    delete d;
}

int bitnet_attention_decode(const void* xqkv, int64_t ld_qkv, const int64_t* pos, const float* rope, void* cache_k,
                            void* cache_v, void* out, int batch, int n_heads, int n_kv_heads, int head_dim,
                            int max_seq_len, void* stream) {
    set_status(kOk);
    if (!xqkv || !pos || !rope || !cache_k || !cache_v || !out || batch < 1) return set_status(kBadArgument), kBadArgument;
    if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > 16 || head_dim % 4 != 0 ||
        head_dim > 128 || batch * n_kv_heads > 4096)
        return set_status(kUnsupported), kUnsupported;
    Workspace* w = workspace();
    if (!w) return bitnet_last_status();
    int s = w->n_sm / (n_kv_heads * batch);
    s = s < 1 ? 1 : (s > 16 ? 16 : s);
    const size_t need = (size_t)batch * n_heads * s * (head_dim + 2) * sizeof(float);
    if (need > w->attn_part_bytes) {      // grows outside stream capture only (cudaMalloc)
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        if (need > w->attn_part_bytes) {
            float* nb = nullptr;
            if (check_cuda(cudaMalloc(&nb, need))) return bitnet_last_status();
            w->attn_part = nb;            // the old buffer may still be in use by enqueued work: it is kept
            w->attn_part_bytes = need;
        }
    }
    AttentionParams ap{};
    ap.xqkv = static_cast<const __nv_bfloat16*>(xqkv); ap.ld_qkv = ld_qkv; ap.pos = pos; ap.rope = rope;
    ap.cache_k = static_cast<__nv_bfloat16*>(cache_k); ap.cache_v = static_cast<__nv_bfloat16*>(cache_v);
    ap.out = static_cast<__nv_bfloat16*>(out);
    ap.part_o = w->attn_part;
    ap.part_ml = w->attn_part + (size_t)batch * n_heads * s * head_dim;
    ap.counters = w->attn_counters;
    ap.H = n_heads; ap.Hkv = n_kv_heads; ap.D = head_dim; ap.L = max_seq_len; ap.S = s;
    if (attention_smem(ap) > 96 * 1024) return set_status(kTooLarge), kTooLarge;
    return launch_attention(ap, batch, static_cast<cudaStream_t>(stream), false,
                            s == 1 && batch * n_kv_heads >= 2 * w->n_sm);
}

}  // extern "C"
