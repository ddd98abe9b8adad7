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

// Layout of a rank's exchange area (the same on every rank).  Everything in it is 8-byte packets
// {value, tag} written by all ranks (see TpTag).
struct TpLayout {
    size_t stats;                                           // TpStatPackets [n_layers][2][size][batch]: attention output, gated values
    size_t part_o, part_2;                                  // packets [size][batch][dim]
    size_t head_val, head_idx;                              // packets [size][grid][8]
    size_t total;
};
static TpLayout tp_layout(const bitnet_decoder_config& c, int size, int head_grid) {
    TpLayout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) / 256 * 256; return o; };
    L.stats = take((size_t)c.n_layers * 2 * size * c.batch * sizeof(TpStatPackets));
    L.part_o = take((size_t)size * c.batch * c.dim * 8);
    L.part_2 = take((size_t)size * c.batch * c.dim * 8);
    L.head_val = take((size_t)size * head_grid * 8 * 8);
    L.head_idx = take((size_t)size * head_grid * 8 * 8);
    L.total = off;
    return L;
}
constexpr long long kPeerWaitCyclesDefault = 600000000LL;   // about 0.3 s
constexpr int kTpHeadGridMax = 256;     // upper bound of the output head's grid used for sizing the area

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
    __nv_bfloat16 *h = nullptr, *xqkv = nullptr, *attn_out = nullptr;
    float *t_h = nullptr, *t_att = nullptr, *t_glu = nullptr;   // x * (next norm weight), f32
    StatPart* stats = nullptr;                    // [1 + 4 * n_layers][batch] statistics slots
    float *part_o = nullptr, *part_ml = nullptr, *part_val = nullptr;
    unsigned long long* trace = nullptr;          // [n_layers * 5][16] phase timestamps (builds with BITNET_TRACE)
    __nv_bfloat16* attn_tap = nullptr;            // optional [n_layers][batch][dim] copy of the attention outputs
    ChainLinearParams plan_qkv{}, plan_o{}, plan_13{}, plan_2{};
    // tensor parallel (tp.size > 1): cfg holds the whole model's sizes, `loc` this rank's share
    TpPeers tp{};
    bitnet_decoder_config loc{};
    unsigned long long* step_ctr = nullptr;       // steps this decoder has completed (device)
    unsigned int* tickets = nullptr;              // tensor parallel: per exchange point, CTAs of this GPU that have delivered (64 bytes apart)
    unsigned int* ticket(int which) const { return tickets + 16 * which; }
    float *a_o = nullptr, *a_2 = nullptr;         // activation scales handed from wo / w2 to their reductions
    long long wait_limit = kPeerWaitCyclesDefault;  // SM cycles a kernel waits for another rank before it gives up

    // statistics slots: 0 = embedding; per layer: attention output, h after wo, gated values, h after w2
    StatPart* slot_emb() const { return stats; }
    StatPart* slot(int layer, int which) const { return stats + (size_t)(1 + 4 * layer + which) * cfg.batch; }
};
enum { kSlotAtt = 0, kSlotHo = 1, kSlotGlu = 2, kSlotH2 = 3 };
enum { kTickAtt = 0, kTickGlu = 1 };

static size_t align_up(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace bitnet

using namespace bitnet;

extern "C" {

int bitnet_init(void) {
    set_status(kOk);
    return workspace() ? kOk : bitnet_last_status();
}

static HeadParams head_params(const Decoder* d, float* logits);

static void* decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers, const void* tok_embeddings,
                            const void* norm, const void* output, const float* rope, int rank, int size,
                            void* const* areas) {
    set_status(kOk);
    if (!cfg || !layers || !tok_embeddings || !norm || !output || !rope) return set_status(kBadArgument), nullptr;
    if (size < 1 || size > kMaxTp || rank < 0 || rank >= size || (size > 1 && !areas)) return set_status(kBadArgument), nullptr;
    const int B = cfg->batch, D = cfg->head_dim;
    if (B < 1 || B > 8 || cfg->n_layers < 1 || cfg->n_heads < 1 || cfg->n_kv_heads < 1 || cfg->n_heads % cfg->n_kv_heads != 0 ||
        cfg->n_heads / cfg->n_kv_heads > 16 || D % 4 != 0 || D > 128 || cfg->dim % 8 != 0 || (cfg->n_heads * D) % 8 != 0 ||
        cfg->ffn_dim % 16 != 0 || cfg->max_seq_len < 2 || cfg->vocab_size < 1)
        return set_status(kUnsupported), nullptr;
    // this rank's share: whole kv-head groups, a slice of the feed-forward width and of the vocabulary
    if (cfg->n_kv_heads % size != 0 || cfg->ffn_dim % (16 * size) != 0 || cfg->vocab_size % size != 0 ||
        (cfg->n_heads / size * D) % 8 != 0)
        return set_status(kUnsupported), nullptr;
    Decoder* d = new (std::nothrow) Decoder();
    if (!d) return set_status(kBadArgument), nullptr;
    d->cfg = *cfg;
    d->loc = *cfg;
    d->loc.n_heads = cfg->n_heads / size;
    d->loc.n_kv_heads = cfg->n_kv_heads / size;
    d->loc.ffn_dim = cfg->ffn_dim / size;
    d->loc.vocab_size = cfg->vocab_size / size;
    d->tp.rank = rank;
    d->tp.size = size;
    for (int r = 0; r < size && size > 1; ++r) {
        if (!areas[r]) {
            delete d;
            return set_status(kBadArgument), nullptr;
        }
        d->tp.area[r] = static_cast<uint8_t*>(areas[r]);
    }
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
    const int H = d->loc.n_heads, Hkv = d->loc.n_kv_heads, F = d->loc.ffn_dim;
    int s = d->n_sm / (Hkv * B);
    d->kv_splits = s < 1 ? 1 : (s > 32 ? 32 : s);
    d->head_grid = d->n_sm < kTpHeadGridMax ? d->n_sm : kTpHeadGridMax;

    const int dim = cfg->dim, Nqkv = (H + 2 * Hkv) * D, Ko = H * D;
    auto plan = [&](ChainLinearParams& p, int N, int K, int k_norm, int out_kind) {
        p = ChainLinearParams{};
        p.N = N; p.K = K; p.k_norm = k_norm; p.out_kind = out_kind; p.M = B; p.eps = cfg->norm_eps;
        p.ring_stages = 4;
#ifdef BITNET_TRACE
        if (getenv("BITNET_RING_STAGES")) p.ring_stages = atoi(getenv("BITNET_RING_STAGES"));   // measurement builds only
#endif
        plan_chain_linear(p, d->n_sm);
        if (p.big_share) {
            // A long stream per CTA is bound by how many warps an SM has to issue from, not by latency:
            // two CTAs per SM (16 consumer warps) with the largest ring that lets two fit; failing that,
            // one CTA with the largest ring.
            const size_t half = (size_t)prop.sharedMemPerMultiprocessor / 2 - 1024 - 256;
            bool two = false;
            for (int rs : {4, 2}) {
                ChainLinearParams q = p;
                q.ring_stages = rs;
                plan_chain_linear(q, 2 * d->n_sm);
                if (chain_linear_smem(q) <= half) {
                    p = q;
                    two = true;
                    break;
                }
            }
            if (!two) {
                p.ring_stages = 8;
                plan_chain_linear(p, d->n_sm);
                if (chain_linear_smem(p) > (size_t)prop.sharedMemPerBlockOptin) {
                    p.ring_stages = 4;
                    plan_chain_linear(p, d->n_sm);
                }
            }
        }
    };
    const bool tp = size > 1;
    plan(d->plan_qkv, Nqkv, dim, dim, kOutBf16);
    plan(d->plan_o, dim, Ko, dim, tp ? kOutTpPartial : kOutResidual);
    plan(d->plan_13, 2 * F, dim, dim, kOutGlu);
    plan(d->plan_2, dim, F, cfg->ffn_dim, tp ? kOutTpPartial : kOutResidual);

    AttentionParams ap{};
    ap.H = H; ap.Hkv = Hkv; ap.D = D; ap.S = d->kv_splits;
    HeadParams hp{};
    hp.M = B; hp.K = dim; hp.V = d->loc.vocab_size;
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
    const size_t o_actr = take((size_t)B * Hkv * 4), o_err = take(4), o_step = take(8), o_tick = take(8 * 64), o_ao = take((size_t)B * 4),
                 o_a2 = take((size_t)B * 4), o_h = take((size_t)B * dim * 2), o_qkv = take((size_t)B * Nqkv * 2),
                 o_att = take((size_t)B * Ko * 2), o_th = take((size_t)B * dim * 4), o_tatt = take((size_t)B * Ko * 4),
                 o_tglu = take((size_t)B * F * 4), o_st = take((size_t)(1 + 4 * cfg->n_layers) * B * sizeof(StatPart)),
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
    d->step_ctr = reinterpret_cast<unsigned long long*>(base + o_step);
    d->tickets = reinterpret_cast<unsigned int*>(base + o_tick);
    d->a_o = reinterpret_cast<float*>(base + o_ao);
    d->a_2 = reinterpret_cast<float*>(base + o_a2);
    d->h = reinterpret_cast<__nv_bfloat16*>(base + o_h);
    d->xqkv = reinterpret_cast<__nv_bfloat16*>(base + o_qkv);
    d->attn_out = reinterpret_cast<__nv_bfloat16*>(base + o_att);
    d->t_h = reinterpret_cast<float*>(base + o_th);
    d->t_att = reinterpret_cast<float*>(base + o_tatt);
    d->t_glu = reinterpret_cast<float*>(base + o_tglu);
    d->stats = reinterpret_cast<StatPart*>(base + o_st);
    d->part_o = reinterpret_cast<float*>(base + o_po);
    d->part_ml = reinterpret_cast<float*>(base + o_pml);
    d->part_val = reinterpret_cast<float*>(base + o_pv);
    d->part_idx = reinterpret_cast<int*>(base + o_pi);
    d->trace = reinterpret_cast<unsigned long long*>(base + o_tr);
    return d;
}

void* bitnet_decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                            const void* tok_embeddings, const void* norm, const void* output, const float* rope) {
    return decoder_create(cfg, layers, tok_embeddings, norm, output, rope, 0, 1, nullptr);
}

void* bitnet_decoder_create_tp(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                               const void* tok_embeddings, const void* norm, const void* output_slice, const float* rope,
                               int rank, int size, void* const* areas) {
    return decoder_create(cfg, layers, tok_embeddings, norm, output_slice, rope, rank, size, areas);
}

size_t bitnet_tp_area_bytes(const bitnet_decoder_config* cfg, int size) {
    if (!cfg || size < 1 || size > kMaxTp) return 0;
    return tp_layout(*cfg, size, kTpHeadGridMax).total;
}

int bitnet_tp_area_create(size_t bytes, void** area, void* ipc_handle_64) {
    set_status(kOk);
    if (!area || !ipc_handle_64 || bytes == 0) return set_status(kBadArgument), kBadArgument;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is handed over as 64 bytes");
    void* p = nullptr;
    // zero-filled before anybody can see it: no packet of a fresh area carries a valid tag
    if (check_cuda(cudaMalloc(&p, bytes)) || check_cuda(cudaMemset(p, 0, bytes)) || check_cuda(cudaDeviceSynchronize())) return kCudaError;
    cudaIpcMemHandle_t h;
    if (check_cuda(cudaIpcGetMemHandle(&h, p))) {
        cudaFree(p);
        return kCudaError;
    }
    memcpy(ipc_handle_64, &h, 64);
    *area = p;
    return kOk;
}

int bitnet_tp_area_open(const void* ipc_handle_64, void** peer_area) {
    set_status(kOk);
    if (!ipc_handle_64 || !peer_area) return set_status(kBadArgument), kBadArgument;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle_64, 64);
    return check_cuda(cudaIpcOpenMemHandle(peer_area, h, cudaIpcMemLazyEnablePeerAccess));
}

int bitnet_tp_area_close(void* peer_area) {
    set_status(kOk);
    return peer_area ? check_cuda(cudaIpcCloseMemHandle(peer_area)) : kOk;
}

int bitnet_tp_area_free(void* area) {
    set_status(kOk);
    return area ? check_cuda(cudaFree(area)) : kOk;
}

// Parameter blocks of layer l: lin[0..3] = wqkv, wo, w13, w2, the attention between the first
// two and, under tensor parallelism, the reductions behind wo and w2.  Every producer hands its
// output on as t = output * (weight of the norm in front of the consumer) with the output's
// statistics in a slot; a slot is cleared by the kernel that runs after its consumer.
static void layer_params(const Decoder* d, int l, const int64_t* pos, ChainLinearParams lin[4], AttentionParams* ap,
                         TpReduceParams red[2]) {
    const bitnet_decoder_config& c = d->cfg;
    const int D = c.head_dim, H = d->loc.n_heads, Hkv = d->loc.n_kv_heads, dim = c.dim, F = d->loc.ffn_dim;
    const int Nqkv = (H + 2 * Hkv) * D, Ko = H * D;
    const int T = d->tp.size, rank = d->tp.rank;
    const bool tp = T > 1;
    const TpLayout lay = tp_layout(c, T, kTpHeadGridMax);
    const bitnet_decoder_layer& L = d->layers[l];
    const bool last = l + 1 == c.n_layers;
    const unsigned long long nl = (unsigned long long)c.n_layers;
    auto bf = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
    uint8_t* my = tp ? d->tp.area[rank] : nullptr;
    auto area_slot = [&](int which) { return lay.stats + ((size_t)(2 * l + which) * T * c.batch) * sizeof(TpStatPackets); };
    // four exchanges per layer (attention statistics, wo sums, gate statistics, w2 sums)
    auto tag_of = [&](int which) {
        TpTag t{};
        t.step = d->step_ctr;
        t.mul = 4u * (unsigned int)nl;
        t.add = 4u * (unsigned int)l + (unsigned int)which + 1u;
        t.limit_cycles = d->wait_limit;
        return t;
    };
    // wqkv: t_h (= h * attention_norm) -> xqkv
    ChainLinearParams& q = lin[0];
    q = d->plan_qkv;
    q.w2t = static_cast<const uint8_t*>(L.wqkv); q.error_flag = d->error_flag;
    q.t = d->t_h; q.ldt = dim;
    q.stats_in = l == 0 ? d->slot_emb() : d->slot(l - 1, kSlotH2);
    if (!tp) q.zero_slot = d->slot(l == 0 ? c.n_layers - 1 : l - 1, kSlotGlu);     // its consumer, w2, has run
    q.out = d->xqkv; q.ldo = Nqkv;
    q.seg.n_seg = 3; q.seg.end[0] = H * D; q.seg.end[1] = (H + Hkv) * D; q.seg.end[2] = Nqkv;
    q.ws[0] = L.s_q; q.ws[1] = L.s_k; q.ws[2] = L.s_v;

    *ap = AttentionParams{};
    ap->xqkv = d->xqkv; ap->ld_qkv = Nqkv; ap->pos = pos; ap->rope = d->rope;
    ap->cache_k = static_cast<__nv_bfloat16*>(L.cache_k); ap->cache_v = static_cast<__nv_bfloat16*>(L.cache_v);
    ap->out = d->attn_out; ap->part_o = d->part_o; ap->part_ml = d->part_ml; ap->counters = d->attn_counters;
    ap->H = H; ap->Hkv = Hkv; ap->D = D; ap->L = c.max_seq_len; ap->S = d->kv_splits;
    ap->gamma_out = bf(L.attn_sub_norm) + (size_t)rank * Ko; ap->t_out = d->t_att; ap->stats_out = d->slot(l, kSlotAtt);
    ap->zero_slot = l == 0 ? nullptr : d->slot(l - 1, kSlotH2);           // its consumer, this layer's wqkv, has run
    ap->tap = d->attn_tap ? d->attn_tap + (size_t)l * c.batch * Ko : nullptr;
    ap->error_flag = d->error_flag;
    if (tp) {     // all ranks' wo normalise over all heads
        ap->tp = d->tp; ap->tp_stats_off = area_slot(0); ap->tp_tag_out = tag_of(0); ap->tp_ticket = d->ticket(kTickAtt);
    }

    // wo: t_att (= attention output * attn_sub_norm) -> h += ...; t_h = h * ffn_norm
    ChainLinearParams& o = lin[1];
    o = d->plan_o;
    o.w2t = static_cast<const uint8_t*>(L.wo); o.error_flag = d->error_flag;
    o.t = d->t_att; o.ldt = Ko;
    o.seg.n_seg = 1; o.seg.end[0] = dim; o.ws[0] = L.s_o;
    if (!tp) {
        o.stats_in = d->slot(l, kSlotAtt);
        o.out = d->h; o.ldo = dim;
        o.gamma_out = bf(L.ffn_norm); o.t_out = d->t_h; o.ldt_out = dim; o.stats_out = d->slot(l, kSlotHo);
    } else {
        o.tp_stats_in = reinterpret_cast<const TpStatPackets*>(my + area_slot(0)); o.tp_tag_in = tag_of(0);
        o.tp = d->tp; o.tp_part_off = lay.part_o; o.tp_tag_out = tag_of(1); o.a_out = d->a_o;
        TpReduceParams& r = red[0];
        r = TpReduceParams{};
        r.part = reinterpret_cast<const uint2*>(my + lay.part_o);
        r.tag = tag_of(1);
        r.a = d->a_o; r.ws = L.s_o; r.out = d->h; r.ldo = dim;
        r.gamma_out = bf(L.ffn_norm); r.t_out = d->t_h; r.stats_out = d->slot(l, kSlotHo);
        r.M = c.batch; r.N = dim; r.T = T; r.error_flag = d->error_flag;
    }

    // w13: t_h -> relu(x1)^2 * x3; t_glu = that * ffn_sub_norm
    ChainLinearParams& u = lin[2];
    u = d->plan_13;
    u.w2t = static_cast<const uint8_t*>(L.w13); u.error_flag = d->error_flag;
    u.t = d->t_h; u.ldt = dim;
    u.stats_in = d->slot(l, kSlotHo);
    if (!tp) u.zero_slot = d->slot(l, kSlotAtt);                          // its consumer, wo, has run
    u.seg.n_seg = 2; u.seg.end[0] = F; u.seg.end[1] = 2 * F; u.ws[0] = L.s_1; u.ws[1] = L.s_3;
    u.gamma_out = bf(L.ffn_sub_norm) + (size_t)rank * F; u.t_out = d->t_glu; u.ldt_out = F; u.stats_out = d->slot(l, kSlotGlu);
    if (tp) {     // all ranks' w2 normalise over the whole gated vector
        u.tp = d->tp; u.tp_stats_off = area_slot(1); u.tp_tag_out = tag_of(2); u.tp_ticket = d->ticket(kTickGlu);
    }

    // w2: t_glu -> h += ...; t_h = h * (the next layer's attention_norm, or the final norm)
    ChainLinearParams& w = lin[3];
    w = d->plan_2;
    w.w2t = static_cast<const uint8_t*>(L.w2); w.error_flag = d->error_flag;
    w.t = d->t_glu; w.ldt = F;
    w.zero_slot = d->slot(l, kSlotHo);                                    // its consumer, w13, has run
    w.seg.n_seg = 1; w.seg.end[0] = dim; w.ws[0] = L.s_2;
    const __nv_bfloat16* g_next = last ? d->final_norm : bf(d->layers[l + 1].attention_norm);
    if (!tp) {
        w.stats_in = d->slot(l, kSlotGlu);
        w.out = d->h; w.ldo = dim;
        w.gamma_out = g_next; w.t_out = d->t_h; w.ldt_out = dim; w.stats_out = d->slot(l, kSlotH2);
    } else {
        w.tp_stats_in = reinterpret_cast<const TpStatPackets*>(my + area_slot(1)); w.tp_tag_in = tag_of(2);
        w.tp = d->tp; w.tp_part_off = lay.part_2; w.tp_tag_out = tag_of(3); w.a_out = d->a_2;
        TpReduceParams& r = red[1];
        r = TpReduceParams{};
        r.part = reinterpret_cast<const uint2*>(my + lay.part_2);
        r.tag = tag_of(3);
        r.a = d->a_2; r.ws = L.s_2; r.out = d->h; r.ldo = dim;
        r.gamma_out = g_next; r.t_out = d->t_h; r.stats_out = d->slot(l, kSlotH2);
        r.M = c.batch; r.N = dim; r.T = T; r.error_flag = d->error_flag;
    }
}

static HeadParams head_params(const Decoder* d, float* logits) {
    HeadParams hp{};
    hp.w = d->output; hp.gamma = d->final_norm; hp.eps = d->cfg.norm_eps;
    hp.h = d->h; hp.logits = logits; hp.part_val = d->part_val; hp.part_idx = d->part_idx;
    hp.stats_in = d->slot(d->cfg.n_layers - 1, kSlotH2);
    hp.M = d->cfg.batch; hp.K = d->cfg.dim; hp.V = d->loc.vocab_size;
    hp.error_flag = d->error_flag;
    if (d->tp.size > 1) {
        const TpLayout lay = tp_layout(d->cfg, d->tp.size, kTpHeadGridMax);
        hp.row_offset = d->tp.rank * d->loc.vocab_size;
        hp.tp = d->tp; hp.tp_val_off = lay.head_val; hp.tp_idx_off = lay.head_idx;
        hp.tp_tag_out.step = d->step_ctr; hp.tp_tag_out.mul = 1; hp.tp_tag_out.add = 1; hp.tp_tag_out.limit_cycles = d->wait_limit;
    }
    return hp;
}

static int enqueue_step(Decoder* d, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, cudaStream_t stream,
                        bool linears_only) {
    const bitnet_decoder_config& c = d->cfg;
    const bool tp = d->tp.size > 1;
    if (tp && linears_only) return set_status(kUnsupported), kUnsupported;
    EmbedParams ep{};
    ep.tokens = tokens; ep.emb = d->emb; ep.gamma = static_cast<const __nv_bfloat16*>(d->layers[0].attention_norm);
    ep.h = d->h; ep.t = d->t_h; ep.stats_out = d->slot_emb();
    ep.zero_slot = d->slot(c.n_layers - 1, kSlotH2);        // its consumer, the previous step's output head, has run
    ep.M = c.batch; ep.K = c.dim; ep.vocab = c.vocab_size; ep.error_flag = d->error_flag;
    if (launch_embed(ep, stream, true)) return bitnet_last_status();
    for (int l = 0; l < c.n_layers; ++l) {
        ChainLinearParams lin[4];
        AttentionParams ap;
        TpReduceParams red[2];
        layer_params(d, l, pos, lin, &ap, red);
#ifdef BITNET_TRACE
        for (int j = 0; j < 4; ++j) lin[j].trace = d->trace + 16 * (4 * l + j);
        ap.trace = d->trace + 16 * (4 * c.n_layers + l);
#endif
        if (launch_chain_linear(lin[0], stream, true)) return bitnet_last_status();
        if (!linears_only && launch_chain_attention(ap, c.batch, stream, true)) return bitnet_last_status();
        if (launch_chain_linear(lin[1], stream, true)) return bitnet_last_status();
        if (tp && launch_tp_reduce(red[0], stream, true)) return bitnet_last_status();
        if (launch_chain_linear(lin[2], stream, true)) return bitnet_last_status();
        if (launch_chain_linear(lin[3], stream, true)) return bitnet_last_status();
        if (tp && launch_tp_reduce(red[1], stream, true)) return bitnet_last_status();
    }
    if (linears_only) return kOk;
    if (launch_head(head_params(d, logits), d->head_grid, stream, true)) return bitnet_last_status();
    ArgmaxParams am{};
    am.part_val = d->part_val; am.part_idx = d->part_idx; am.n_part = d->head_grid; am.M = c.batch;
    am.out = out; am.tokens = tokens; am.pos = pos; am.error_flag = d->error_flag;
    am.step = d->step_ctr;
    if (tp) {
        const TpLayout lay = tp_layout(c, d->tp.size, kTpHeadGridMax);
        uint8_t* my = d->tp.area[d->tp.rank];
        am.part_val = reinterpret_cast<const float*>(my + lay.head_val);
        am.part_idx = reinterpret_cast<const int*>(my + lay.head_idx);
        am.n_part = d->tp.size * d->head_grid;
        am.tag.step = d->step_ctr; am.tag.mul = 1; am.tag.add = 1; am.tag.limit_cycles = d->wait_limit;
    }
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
    // the state the kernels of the chain keep between launches: the attention tickets and the
    // statistics slots (a step that ended early may have left shares in them)
    if (check_cuda(cudaDeviceSynchronize()) || check_cuda(cudaMemset(d->error_flag, 0, sizeof(int))) ||
        check_cuda(cudaMemset(d->attn_counters, 0, (size_t)d->cfg.batch * d->cfg.n_kv_heads * sizeof(int))) ||
        check_cuda(cudaMemset(d->tickets, 0, 8 * 64)) ||
        check_cuda(cudaMemset(d->stats, 0, (size_t)(1 + 4 * d->cfg.n_layers) * d->cfg.batch * sizeof(StatPart))))
        return kCudaError;
    return kOk;
}

int bitnet_decoder_set_wait_limit(void* dec, double milliseconds) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !(milliseconds > 0.0)) return set_status(kBadArgument), kBadArgument;
    cudaDeviceProp prop;
    if (check_cuda(cudaGetDeviceProperties(&prop, d->device))) return kCudaError;
    d->wait_limit = (long long)(milliseconds * (double)prop.clockRate);   // clockRate is in kHz: cycles per millisecond
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
    return (d->tp.size > 1 ? 7 : 5) * d->cfg.n_layers + 3;
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
    s = s < 1 ? 1 : (s > 32 ? 32 : s);
    // Many sequences (at least two CTAs per SM without any split) take the op-by-op path's own
    // kernels.  Whole groups of query heads on the tensor-core loop may still be cut into up to
    // three slices at long contexts (fewer than the heads of a group, so that a group stays in
    // one CTA): hundreds of long CTAs in a wave and a fraction end in a long tail otherwise.
    const bool many = s == 1 && batch * n_kv_heads >= 2 * w->n_sm;
    const int G = n_heads / n_kv_heads;
    if (many && G > 1 && head_dim == 128) s = G - 1 < 3 ? G - 1 : 3;
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
    if (many) return launch_attention(ap, batch, static_cast<cudaStream_t>(stream), false, true);
    return launch_chain_attention(ap, batch, static_cast<cudaStream_t>(stream), false);
}

}  // extern "C"
