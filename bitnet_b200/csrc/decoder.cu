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
#include "../../include/bitnet_b200_bench.h"
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
    if (prepare_fused_kernels(w.smem_optin, 96 * 1024, w.smem_optin) || prepare_chain_kernels(w.smem_optin)) return nullptr;
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
    int *attn_counters = nullptr, *error_flag = nullptr, *part_idx = nullptr;
    __nv_bfloat16 *h = nullptr, *xqkv = nullptr, *attn_out = nullptr, *glu = nullptr;
    StatPart *stats_h = nullptr, *stats_att = nullptr, *stats_glu = nullptr;
    float *part_o = nullptr, *part_ml = nullptr, *part_val = nullptr;
    unsigned long long* trace = nullptr;          // [n_layers * 5][16] phase timestamps (builds with BITNET_TRACE)
    __nv_bfloat16* attn_tap = nullptr;            // optional [n_layers][batch][dim] copy of the attention outputs
    ChainLinearParams plan_qkv{}, plan_o{}, plan_13{}, plan_2{};
    int64_t steps_enqueued = 0;                   // host mirror of the positions' advance (bounds check)
};

static size_t align_up(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace bitnet

using namespace bitnet;

extern "C" {

int bitnet_init(void) {
    set_status(kOk);
    return workspace() ? kOk : bitnet_last_status();
}

static void layer_params(const Decoder* d, int l, const int64_t* tokens, const int64_t* pos, ChainLinearParams lin[4],
                         AttentionParams* ap);
static HeadParams head_params(const Decoder* d, float* logits);

void* bitnet_decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                            const void* tok_embeddings, const void* norm, const void* output, const float* rope) {
    set_status(kOk);
    if (!cfg || !layers || !tok_embeddings || !norm || !output || !rope) return set_status(kBadArgument), nullptr;
    const int B = cfg->batch, D = cfg->head_dim, H = cfg->n_heads, Hkv = cfg->n_kv_heads;
    if (B < 1 || B > 8 || cfg->n_layers < 1 || H < 1 || Hkv < 1 || H % Hkv != 0 || H / Hkv > 16 || D % 4 != 0 ||
        D > 128 || cfg->dim % 8 != 0 || cfg->dim != H * D || cfg->ffn_dim % 16 != 0 || cfg->max_seq_len < 2 ||
        cfg->vocab_size < 1)
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
    auto plan = [&](ChainLinearParams& p, int N, int K, int src, int out_kind, const void* gamma_probe) {
        p = ChainLinearParams{};
        p.N = N; p.K = K; p.src = src; p.out_kind = out_kind; p.M = B; p.eps = cfg->norm_eps;
        p.gamma = static_cast<const __nv_bfloat16*>(gamma_probe);   // only whether there is one matters for the layout
        p.ring_stages = 4;
        plan_chain_linear(p, d->n_sm);
    };
    plan(d->plan_qkv, Nqkv, dim, kSrcVector, kOutBf16, norm);
    plan(d->plan_o, dim, dim, kSrcVector, kOutResidual, norm);
    plan(d->plan_13, 2 * F, dim, kSrcVector, kOutGlu, norm);
    plan(d->plan_2, dim, F, kSrcVector, kOutResidual, norm);

    AttentionParams ap{};
    ap.H = H; ap.Hkv = Hkv; ap.D = D; ap.S = d->kv_splits;
    HeadParams hp{};
    hp.M = B; hp.K = dim; hp.V = cfg->vocab_size;
    size_t lin_smem = 0;
    for (const ChainLinearParams* p : {&d->plan_qkv, &d->plan_o, &d->plan_13, &d->plan_2})
        lin_smem = chain_linear_smem(*p) > lin_smem ? chain_linear_smem(*p) : lin_smem;
    if (lin_smem > (size_t)prop.sharedMemPerBlockOptin || head_smem(hp) > (size_t)prop.sharedMemPerBlockOptin ||
        chain_attention_smem(ap) > 96 * 1024) {
        delete d;
        return set_status(kTooLarge), nullptr;
    }
    if (!workspace() || prepare_chain_kernels(prop.sharedMemPerBlockOptin)) {   // shared memory limits of this device's kernels
        delete d;
        return nullptr;
    }

    // one zero-initialised scratch allocation
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return o; };
    const size_t o_actr = take((size_t)B * Hkv * 4), o_err = take(4), o_h = take((size_t)B * dim * 2),
                 o_qkv = take((size_t)B * Nqkv * 2), o_att = take((size_t)B * dim * 2), o_glu = take((size_t)B * F * 2),
                 o_sh = take((size_t)B * d->plan_o.n_units * sizeof(StatPart)),
                 o_sa = take((size_t)B * H * sizeof(StatPart)),
                 o_sg = take((size_t)B * d->plan_13.n_units * sizeof(StatPart)),
                 o_po = take((size_t)B * H * d->kv_splits * D * 4),
                 o_pml = take((size_t)B * H * d->kv_splits * 2 * 4), o_pv = take((size_t)d->head_grid * 8 * 4),
                 o_pi = take((size_t)d->head_grid * 8 * 4), o_tr = take((size_t)cfg->n_layers * 5 * 16 * 8);
    if (check_cuda(cudaMalloc(&d->scratch, off)) || check_cuda(cudaMemset(d->scratch, 0, off))) {
        delete d;
        return nullptr;
    }
    uint8_t* base = static_cast<uint8_t*>(d->scratch);
    d->attn_counters = reinterpret_cast<int*>(base + o_actr);
    d->error_flag = reinterpret_cast<int*>(base + o_err);
    d->h = reinterpret_cast<__nv_bfloat16*>(base + o_h);
    d->xqkv = reinterpret_cast<__nv_bfloat16*>(base + o_qkv);
    d->attn_out = reinterpret_cast<__nv_bfloat16*>(base + o_att);
    d->glu = reinterpret_cast<__nv_bfloat16*>(base + o_glu);
    d->stats_h = reinterpret_cast<StatPart*>(base + o_sh);
    d->stats_att = reinterpret_cast<StatPart*>(base + o_sa);
    d->stats_glu = reinterpret_cast<StatPart*>(base + o_sg);
    d->part_o = reinterpret_cast<float*>(base + o_po);
    d->part_ml = reinterpret_cast<float*>(base + o_pml);
    d->part_val = reinterpret_cast<float*>(base + o_pv);
    d->part_idx = reinterpret_cast<int*>(base + o_pi);
    d->trace = reinterpret_cast<unsigned long long*>(base + o_tr);
    return d;
}

// Parameter blocks of layer l: lin[0..3] = wqkv, wo, w13, w2 and the attention between the
// first two.
static void layer_params(const Decoder* d, int l, const int64_t* tokens, const int64_t* pos, ChainLinearParams lin[4],
                         AttentionParams* ap) {
    const bitnet_decoder_config& c = d->cfg;
    const int D = c.head_dim, H = c.n_heads, Hkv = c.n_kv_heads, dim = c.dim, F = c.ffn_dim;
    const int Nqkv = (H + 2 * Hkv) * D;
    const bitnet_decoder_layer& L = d->layers[l];
    const bool last = l + 1 == c.n_layers;
    auto common = [&](ChainLinearParams& p, const void* w, const void* gamma) {
        p.w2t = static_cast<const uint8_t*>(w);
        p.gamma = static_cast<const __nv_bfloat16*>(gamma);
        p.error_flag = d->error_flag;
    };
    // wqkv: (embedding ->) h -> attention_norm -> wqkv -> xqkv
    ChainLinearParams& q = lin[0];
    q = d->plan_qkv;
    common(q, L.wqkv, L.attention_norm);
    if (l == 0) {
        q.src = kSrcEmbedding;
        q.tokens = tokens; q.emb = d->emb; q.h_copy = d->h; q.vocab = c.vocab_size;
    } else {
        q.x = d->h; q.ldx = dim;
        q.stats_in = d->stats_h; q.n_stats_in = d->plan_o.n_units;
    }
    q.out = d->xqkv; q.ldo = Nqkv;
    q.seg.n_seg = 3; q.seg.end[0] = H * D; q.seg.end[1] = (H + Hkv) * D; q.seg.end[2] = Nqkv;
    q.ws[0] = L.s_q; q.ws[1] = L.s_k; q.ws[2] = L.s_v;

    *ap = AttentionParams{};
    ap->xqkv = d->xqkv; ap->ld_qkv = Nqkv; ap->pos = pos; ap->rope = d->rope;
    ap->cache_k = static_cast<__nv_bfloat16*>(L.cache_k); ap->cache_v = static_cast<__nv_bfloat16*>(L.cache_v);
    ap->out = d->attn_out; ap->part_o = d->part_o; ap->part_ml = d->part_ml; ap->counters = d->attn_counters;
    ap->H = H; ap->Hkv = Hkv; ap->D = D; ap->L = c.max_seq_len; ap->S = d->kv_splits;
    ap->gamma_out = static_cast<const __nv_bfloat16*>(L.attn_sub_norm); ap->stats_out = d->stats_att;
    ap->tap = d->attn_tap ? d->attn_tap + (size_t)l * c.batch * dim : nullptr;
    ap->error_flag = d->error_flag;

    // wo: attention output -> attn_sub_norm -> wo -> h += ...   (statistics for ffn_norm)
    ChainLinearParams& o = lin[1];
    o = d->plan_o;
    common(o, L.wo, L.attn_sub_norm);
    o.x = d->attn_out; o.ldx = dim;
    o.stats_in = d->stats_att; o.n_stats_in = H;
    o.out = d->h; o.ldo = dim;
    o.seg.n_seg = 1; o.seg.end[0] = dim; o.ws[0] = L.s_o;
    o.gamma_out = static_cast<const __nv_bfloat16*>(L.ffn_norm); o.stats_out = d->stats_h;

    // w13: h -> ffn_norm -> w13 -> relu(x1)^2 * x3   (statistics for ffn_sub_norm)
    ChainLinearParams& u = lin[2];
    u = d->plan_13;
    common(u, L.w13, L.ffn_norm);
    u.x = d->h; u.ldx = dim;
    u.stats_in = d->stats_h; u.n_stats_in = d->plan_o.n_units;
    u.out = d->glu; u.ldo = F;
    u.seg.n_seg = 2; u.seg.end[0] = F; u.seg.end[1] = 2 * F; u.ws[0] = L.s_1; u.ws[1] = L.s_3;
    u.gamma_out = static_cast<const __nv_bfloat16*>(L.ffn_sub_norm); u.stats_out = d->stats_glu;

    // w2: gated values -> ffn_sub_norm -> w2 -> h += ...   (statistics for the next layer's
    // attention_norm, or for the final norm)
    ChainLinearParams& w = lin[3];
    w = d->plan_2;
    common(w, L.w2, L.ffn_sub_norm);
    w.x = d->glu; w.ldx = F;
    w.stats_in = d->stats_glu; w.n_stats_in = d->plan_13.n_units;
    w.out = d->h; w.ldo = dim;
    w.seg.n_seg = 1; w.seg.end[0] = dim; w.ws[0] = L.s_2;
    w.gamma_out = last ? d->final_norm : static_cast<const __nv_bfloat16*>(d->layers[l + 1].attention_norm);
    w.stats_out = d->stats_h;
}

static HeadParams head_params(const Decoder* d, float* logits) {
    HeadParams hp{};
    hp.w = d->output; hp.gamma = d->final_norm; hp.eps = d->cfg.norm_eps;
    hp.h = d->h; hp.logits = logits; hp.part_val = d->part_val; hp.part_idx = d->part_idx;
    hp.stats_in = d->stats_h; hp.n_stats_in = d->plan_2.n_units;
    hp.M = d->cfg.batch; hp.K = d->cfg.dim; hp.V = d->cfg.vocab_size;
    return hp;
}

static int enqueue_step(Decoder* d, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, cudaStream_t stream,
                        bool linears_only) {
    const bitnet_decoder_config& c = d->cfg;
    for (int l = 0; l < c.n_layers; ++l) {
        ChainLinearParams lin[4];
        AttentionParams ap;
        layer_params(d, l, tokens, pos, lin, &ap);
#ifdef BITNET_TRACE
        for (int j = 0; j < 4; ++j) lin[j].trace = d->trace + 16 * (4 * l + j);
#endif
        if (launch_chain_linear(lin[0], stream, true)) return bitnet_last_status();
        if (!linears_only && launch_chain_attention(ap, c.batch, stream, true)) return bitnet_last_status();
        for (int j = 1; j < 4; ++j)
            if (launch_chain_linear(lin[j], stream, true)) return bitnet_last_status();
    }
    if (linears_only) return kOk;
    if (launch_head(head_params(d, logits), d->head_grid, stream, true)) return bitnet_last_status();
    ArgmaxParams am{};
    am.part_val = d->part_val; am.part_idx = d->part_idx; am.n_part = d->head_grid; am.M = c.batch;
    am.out = out; am.tokens = tokens; am.pos = pos;
    return launch_argmax(am, stream, true);
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

int bitnet_decoder_clear_error(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return set_status(kBadArgument), kBadArgument;
    // the kernels of the chain keep no state between launches besides the attention tickets
    if (check_cuda(cudaMemset(d->error_flag, 0, sizeof(int))) ||
        check_cuda(cudaMemset(d->attn_counters, 0, (size_t)d->cfg.batch * d->cfg.n_kv_heads * sizeof(int))))
        return kCudaError;
    return kOk;
}

int bitnet_decoder_set_attention_tap(void* dec, void* buffer) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return set_status(kBadArgument), kBadArgument;
    d->attn_tap = static_cast<__nv_bfloat16*>(buffer);
    return kOk;
}

int bitnet_decoder_read_trace(void* dec, unsigned long long* host_out, int n_values) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !host_out) return set_status(kBadArgument), kBadArgument;
#ifdef BITNET_TRACE
    const int have = d->cfg.n_layers * 5 * 16;
    return check_cuda(cudaMemcpy(host_out, d->trace, sizeof(unsigned long long) * (n_values < have ? n_values : have),
                                 cudaMemcpyDeviceToHost));
#else
    (void)n_values;
    return set_status(kUnsupported), kUnsupported;   // built without -DBITNET_TRACE
#endif
}

int bitnet_decoder_kernels_per_step(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return 0;
    return 5 * d->cfg.n_layers + 2;
}

void bitnet_decoder_destroy(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return;
    if (d->scratch) cudaFree(d->scratch);
    delete d;
}

int bitnet_workspace_error(int clear) {
    set_status(kOk);
    Workspace* w = workspace();
    if (!w) return -1;
    int v = 0;
    if (check_cuda(cudaDeviceSynchronize()) ||
        check_cuda(cudaMemcpy(&v, w->error_flag, sizeof(int), cudaMemcpyDeviceToHost)))
        return -1;
    if (v != 0 && clear) {
        // a kernel that gave up may have left partial sums and tickets behind: start clean
        if (check_cuda(cudaMemset(w->acc_scratch, 0, (size_t)kWsRowGroups * 128 * 8)) ||
            check_cuda(cudaMemset(w->attn_counters, 0, 4096 * 4)) ||
            check_cuda(cudaMemset(w->tc_acc, 0, w->tc_acc_ints * 4)) ||
            check_cuda(cudaMemset(w->error_flag, 0, sizeof(int))))
            return -1;
    }
    return v;
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
    ap.error_flag = w->error_flag;
    if (chain_attention_smem(ap) > 96 * 1024) return set_status(kTooLarge), kTooLarge;
    // Many sequences (at least two CTAs per SM without any split): the 4-warp form of the
    // split-KV kernel.  Otherwise the decode chain's attention kernel, so that a decoder run op
    // by op and the in-library chain compute the very same attention.
    if (s == 1 && batch * n_kv_heads >= 2 * w->n_sm)
        return launch_attention(ap, batch, static_cast<cudaStream_t>(stream), false, true);
    return launch_chain_attention(ap, batch, static_cast<cudaStream_t>(stream), false);
}

}  // extern "C"
