// The decode-step object behind bitnet_decoder_create / _step / _destroy: owns the scratch
// buffers of the fused kernel chain (decode_fused.cu) and enqueues one step - five kernels
// per layer, then the output head and the greedy choice - on the caller's stream.
#include <new>
#include <vector>

#include "../../include/bitnet_b200.h"
#include "common.cuh"
#include "decode_fused.h"

namespace bitnet {

struct Decoder {
    bitnet_decoder_config cfg{};
    std::vector<bitnet_decoder_layer> layers;
    const __nv_bfloat16* emb = nullptr;
    const __nv_bfloat16* final_norm = nullptr;
    const __nv_bfloat16* output = nullptr;
    const float* rope = nullptr;
    int device = 0, n_sm = 0, kv_splits = 1, head_grid = 0;
    // scratch (one allocation)
    void* scratch = nullptr;
    int32_t *acc_qkv = nullptr, *acc_o = nullptr, *acc_13 = nullptr, *acc_2 = nullptr;
    float *a_qkv = nullptr, *a_o = nullptr, *a_13 = nullptr, *a_2 = nullptr;
    __nv_bfloat16 *h_a = nullptr, *h_b = nullptr;
    float *part_o = nullptr, *part_ml = nullptr, *part_val = nullptr;
    int* part_idx = nullptr;
    int* error_flag = nullptr;
    FusedLinearParams plan_qkv{}, plan_o{}, plan_13{}, plan_2{};
};

static size_t align_up(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace bitnet

using namespace bitnet;

extern "C" {

void* bitnet_decoder_create(const bitnet_decoder_config* cfg, const bitnet_decoder_layer* layers,
                            const void* tok_embeddings, const void* norm, const void* output, const float* rope) {
    set_status(kOk);
    if (!cfg || !layers || !tok_embeddings || !norm || !output || !rope) return set_status(kBadArgument), nullptr;
    const int B = cfg->batch, D = cfg->head_dim, H = cfg->n_heads, Hkv = cfg->n_kv_heads;
    if (B < 1 || B > 8 || cfg->n_layers < 1 || H < 1 || Hkv < 1 || H % Hkv != 0 || H / Hkv > 16 || D % 4 != 0 ||
        D > 128 || cfg->dim % 8 != 0 || cfg->dim != H * D || cfg->max_seq_len < 2)
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
    auto plan = [&](FusedLinearParams& p, int N, int K, int src) {
        p = FusedLinearParams{};
        p.N = N; p.K = K; p.src = src; p.M = B; p.eps = cfg->norm_eps;
        plan_linear(p, d->n_sm);
    };
    plan(d->plan_qkv, Nqkv, dim, kSrcResidual);
    plan(d->plan_o, dim, dim, kSrcAttention);
    plan(d->plan_13, 2 * F, dim, kSrcResidual);
    plan(d->plan_2, dim, F, kSrcGlu);

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
    if (prepare_fused_kernels(lin_smem, attention_smem(ap), head_smem(hp))) {
        delete d;
        return nullptr;
    }

    // one zero-initialised scratch allocation
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return o; };
    const size_t o_qkv = take((size_t)B * Nqkv * 4), o_o = take((size_t)B * dim * 4), o_13 = take((size_t)B * 2 * F * 4),
                 o_2 = take((size_t)B * dim * 4), o_a = take(4 * 8 * 4), o_ha = take((size_t)B * dim * 2),
                 o_hb = take((size_t)B * dim * 2), o_po = take((size_t)B * H * d->kv_splits * D * 4),
                 o_pml = take((size_t)B * H * d->kv_splits * 2 * 4), o_pv = take((size_t)d->head_grid * 8 * 4),
                 o_pi = take((size_t)d->head_grid * 8 * 4), o_err = take(4);
    if (check_cuda(cudaMalloc(&d->scratch, off)) || check_cuda(cudaMemset(d->scratch, 0, off))) {
        delete d;
        return nullptr;
    }
    uint8_t* base = static_cast<uint8_t*>(d->scratch);
    d->acc_qkv = reinterpret_cast<int32_t*>(base + o_qkv);
    d->acc_o = reinterpret_cast<int32_t*>(base + o_o);
    d->acc_13 = reinterpret_cast<int32_t*>(base + o_13);
    d->acc_2 = reinterpret_cast<int32_t*>(base + o_2);
    float* a = reinterpret_cast<float*>(base + o_a);
    d->a_qkv = a; d->a_o = a + 8; d->a_13 = a + 16; d->a_2 = a + 24;
    d->h_a = reinterpret_cast<__nv_bfloat16*>(base + o_ha);
    d->h_b = reinterpret_cast<__nv_bfloat16*>(base + o_hb);
    d->part_o = reinterpret_cast<float*>(base + o_po);
    d->part_ml = reinterpret_cast<float*>(base + o_pml);
    d->part_val = reinterpret_cast<float*>(base + o_pv);
    d->part_idx = reinterpret_cast<int*>(base + o_pi);
    d->error_flag = reinterpret_cast<int*>(base + o_err);
    return d;
}

static int enqueue_step(Decoder* d, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, cudaStream_t stream,
                        bool linears_only) {
    const bitnet_decoder_config& c = d->cfg;
    const int B = c.batch, D = c.head_dim, H = c.n_heads, Hkv = c.n_kv_heads, dim = c.dim, F = c.ffn_dim;
    const int Nqkv = (H + 2 * Hkv) * D;
    for (int l = 0; l < c.n_layers; ++l) {
        const bitnet_decoder_layer& L = d->layers[l];
        // wqkv: residual (or embedding) -> attention_norm -> wqkv
        FusedLinearParams p = d->plan_qkv;
        p.w2t = static_cast<const uint8_t*>(L.wqkv);
        p.gamma = static_cast<const __nv_bfloat16*>(L.attention_norm);
        p.acc_out = d->acc_qkv; p.a_out = d->a_qkv;
        p.zero_buf = d->acc_13; p.zero_count = B * 2 * F;
        p.error_flag = d->error_flag;
        p.h_out = d->h_a;
        if (l == 0) {
            p.src = kSrcEmbedding;
            p.tokens = tokens; p.emb = d->emb;
        } else {
            p.src = kSrcResidual;
            p.h_in = d->h_b; p.acc_in = d->acc_2; p.ld_acc_in = dim; p.a_in = d->a_2;
            p.ws_in[0] = d->layers[l - 1].s_2;
        }
        if (launch_fused_linear(p, stream)) return bitnet_last_status();

        AttentionParams ap{};
        ap.acc_qkv = d->acc_qkv; ap.ld_acc = Nqkv; ap.a_in = d->a_qkv;
        ap.ws_q = L.s_q; ap.ws_k = L.s_k; ap.ws_v = L.s_v;
        ap.pos = pos; ap.rope = d->rope;
        ap.cache_k = static_cast<__nv_bfloat16*>(L.cache_k); ap.cache_v = static_cast<__nv_bfloat16*>(L.cache_v);
        ap.part_o = d->part_o; ap.part_ml = d->part_ml;
        ap.H = H; ap.Hkv = Hkv; ap.D = D; ap.L = c.max_seq_len; ap.S = d->kv_splits;
        ap.zero_buf = d->acc_2; ap.zero_count = B * dim;
        if (!linears_only && launch_attention(ap, B, stream)) return bitnet_last_status();

        // wo: attention output -> attn_sub_norm -> wo
        p = d->plan_o;
        p.w2t = static_cast<const uint8_t*>(L.wo);
        p.gamma = static_cast<const __nv_bfloat16*>(L.attn_sub_norm);
        p.acc_out = d->acc_o; p.a_out = d->a_o;
        p.zero_buf = d->acc_qkv; p.zero_count = B * Nqkv;
        p.error_flag = d->error_flag;
        p.part_o = d->part_o; p.part_ml = d->part_ml; p.S = d->kv_splits; p.H = H; p.D = D;
        if (launch_fused_linear(p, stream)) return bitnet_last_status();

        // w13: residual -> ffn_norm -> w13
        p = d->plan_13;
        p.w2t = static_cast<const uint8_t*>(L.w13);
        p.gamma = static_cast<const __nv_bfloat16*>(L.ffn_norm);
        p.acc_out = d->acc_13; p.a_out = d->a_13;
        p.error_flag = d->error_flag;
        p.h_in = d->h_a; p.h_out = d->h_b; p.acc_in = d->acc_o; p.ld_acc_in = dim; p.a_in = d->a_o;
        p.ws_in[0] = L.s_o;
        if (launch_fused_linear(p, stream)) return bitnet_last_status();

        // w2: relu(x1)^2 * x3 -> ffn_sub_norm -> w2
        p = d->plan_2;
        p.w2t = static_cast<const uint8_t*>(L.w2);
        p.gamma = static_cast<const __nv_bfloat16*>(L.ffn_sub_norm);
        p.acc_out = d->acc_2; p.a_out = d->a_2;
        p.zero_buf = d->acc_o; p.zero_count = B * dim;
        p.error_flag = d->error_flag;
        p.acc_in = d->acc_13; p.ld_acc_in = 2 * F; p.a_in = d->a_13;
        p.ws_in[0] = L.s_1; p.ws_in[1] = L.s_3;
        if (launch_fused_linear(p, stream)) return bitnet_last_status();
    }
    if (linears_only) return kOk;
    HeadParams hp{};
    hp.w = d->output; hp.gamma = d->final_norm; hp.eps = c.norm_eps;
    hp.h_in = d->h_b; hp.acc_in = d->acc_2; hp.a_in = d->a_2; hp.ws_in = d->layers[c.n_layers - 1].s_2;
    hp.logits = logits; hp.part_val = d->part_val; hp.part_idx = d->part_idx;
    hp.M = B; hp.K = dim; hp.V = c.vocab_size;
    if (launch_head(hp, d->head_grid, stream)) return bitnet_last_status();
    ArgmaxParams am{};
    am.part_val = d->part_val; am.part_idx = d->part_idx; am.n_part = d->head_grid; am.M = B;
    am.out = out; am.tokens = tokens; am.pos = pos;
    return launch_argmax(am, stream);
}

int bitnet_decoder_step(void* dec, int64_t* tokens, int64_t* pos, int64_t* out, float* logits, void* stream) {
    set_status(kOk);
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d || !tokens || !pos || !out) return set_status(kBadArgument), kBadArgument;
    return enqueue_step(d, tokens, pos, out, logits, static_cast<cudaStream_t>(stream), false);
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

int bitnet_decoder_kernels_per_step(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    return d ? 5 * d->cfg.n_layers + 2 : 0;
}

void bitnet_decoder_destroy(void* dec) {
    Decoder* d = static_cast<Decoder*>(dec);
    if (!d) return;
    if (d->scratch) cudaFree(d->scratch);
    delete d;
}

}  // extern "C"
