"""The decoder on the W2A8 kernels vs the bf16 fake-quantised reference form (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models():
    from bitnet_b200.model import build_synthetic, preset

    args = preset("tiny", n_layers=3)
    kern = build_synthetic(args, seed=5, device="cuda", max_seq_len=128)
    ref = build_synthetic(preset("tiny", n_layers=3, use_kernel=False), seed=5, device="cuda", max_seq_len=128)
    return args, kern, ref


def test_kernel_layers_match_torch_reference_layer_by_layer(models):
    """Each decoder layer on the kernels against the same layer in plain PyTorch, both fed
    the PyTorch model's layer input.  The two differ only by f32 rounding order and by the
    int8 values that a last-bit difference pushes across a rounding boundary (a quantiser
    amplifies such differences, so the comparison is per layer, not end to end): bf16
    outputs within 1e-2 relative for the median token, 5e-2 for all."""
    from bitnet_b200.model import make_cache

    args, kern, ref = models
    B, T = 2, 12
    toks = torch.randint(0, args.vocab_size, (B, T), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    pos = torch.zeros(B, dtype=torch.int64, device="cuda")
    cache_k, cache_r = make_cache(args, B, 128, "cuda"), make_cache(args, B, 128, "cuda")
    h = ref.tok_embeddings(toks)
    assert torch.equal(h, kern.tok_embeddings(toks))
    for lk, lr, ck, cr in zip(kern.layers, ref.layers, cache_k, cache_r):
        out_r = lr(h, cr, pos, ref.rope, T)
        out_k = lk(h, ck, pos, kern.rope, T)
        err = (out_k.float() - out_r.float()).abs().amax(-1) / out_r.float().abs().amax(-1)
        assert torch.quantile(err.flatten(), 0.5) <= 1e-2 and err.max() <= 5e-2
        h = out_r


def test_attention_kernel_matches_pytorch_attention(models):
    """The stand-alone decode attention (RoPE, cache append, split softmax) against
    apply_rope + scaled_dot_product_attention, bf16 outputs within 1e-2 relative."""
    from bitnet_b200 import ops
    from bitnet_b200.model import apply_rope, rope_table

    for B, H, Hkv, D, L, P in [(1, 20, 5, 128, 256, 200), (3, 8, 2, 64, 64, 5), (2, 32, 32, 100, 96, 37),
                               (2, 80, 8, 128, 128, 0), (64, 8, 8, 128, 64, 33), (64, 20, 5, 128, 256, 140),
                               (70, 32, 8, 128, 640, 600),
                               # groups of more than four query heads: the tensor-core key loop, one and several
                               # slices, slice ends inside and at the end of a 16-key step
                               (1, 10, 1, 128, 4224, 4096), (2, 80, 8, 128, 1100, 1000), (1, 16, 2, 128, 512, 15),
                               (1, 16, 2, 128, 512, 16), (3, 12, 2, 128, 512, 17), (1, 10, 1, 128, 512, 383),
                               (2, 20, 2, 128, 2176, 2049), (8, 10, 1, 128, 640, 531),
                               # ratios up to four at long contexts and with several sequences: the 8-row tensor-core loop
                               (1, 20, 5, 128, 1024, 900), (2, 32, 8, 128, 2176, 2049), (8, 32, 8, 128, 640, 500),
                               (1, 4, 1, 128, 2176, 2100), (3, 8, 4, 128, 512, 385), (1, 4, 2, 128, 4224, 4099)]:
        g = torch.Generator("cuda").manual_seed(B * 100 + H)
        xqkv = torch.randn((B, (H + 2 * Hkv) * D), device="cuda", generator=g).bfloat16()
        ck = torch.randn((B, L, Hkv, D), device="cuda", generator=g).bfloat16()
        cv = torch.randn((B, L, Hkv, D), device="cuda", generator=g).bfloat16()
        pos = torch.full((B,), P, dtype=torch.int64, device="cuda")
        pos[0] = max(P - 3, 0)
        rope = rope_table(D, L, 500000.0, "cuda")
        ck2, cv2 = ck.clone(), cv.clone()
        out = ops.attention_decode(xqkv, pos, rope, ck2, cv2, H, Hkv, D)
        # reference
        q = xqkv[:, : H * D].view(B, 1, H, D)
        k = xqkv[:, H * D: (H + Hkv) * D].view(B, 1, Hkv, D)
        v = xqkv[:, (H + Hkv) * D:].view(B, 1, Hkv, D)
        cs = rope[pos[:, None]]
        q, k = apply_rope(q, cs), apply_rope(k, cs)
        bidx = torch.arange(B, device="cuda")
        ck[bidx, pos] = k[:, 0]
        cv[bidx, pos] = v[:, 0]
        assert torch.equal(ck, ck2) and torch.equal(cv, cv2)               # cache append is exact
        mask = torch.arange(L, device="cuda")[None, None, None, :] <= pos[:, None, None, None]
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2).float(), ck.transpose(1, 2).float(), cv.transpose(1, 2).float(), attn_mask=mask,
            enable_gqa=True).transpose(1, 2).reshape(B, H * D)
        err = (out.float() - ref).abs().max() / ref.abs().max()
        assert err <= 1e-2, (B, H, Hkv, D, float(err))


def test_graph_decode_equals_eager_decode(models):
    from bitnet_b200.generate import Generator

    args, kern, _ = models
    prompt = torch.randint(0, args.vocab_size, (2, 8), device="cuda", generator=torch.Generator("cuda").manual_seed(2))
    a = Generator(kern, 2, 128, use_cuda_graph=True).generate(prompt, 24)
    b = Generator(kern, 2, 128, use_cuda_graph=False).generate(prompt, 24)
    assert torch.equal(a, b)


def test_prefill_equals_token_by_token(models):
    """Feeding the prompt in one pass or one token at a time leaves the same next token."""
    from bitnet_b200.model import make_cache

    args, kern, _ = models
    B, T = 1, 10
    toks = torch.randint(0, args.vocab_size, (B, T), device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    pos = torch.zeros(B, dtype=torch.int64, device="cuda")
    full = kern(toks, pos, make_cache(args, B, 128, "cuda"), kv_len=T)
    cache = make_cache(args, B, 128, "cuda")
    for layer in kern.layers:                      # same attention arithmetic on both sides
        layer.attention.kernel_attention = False
    try:
        for t in range(T):
            step = kern(toks[:, t:t + 1], pos + t, cache)
    finally:
        for layer in kern.layers:
            layer.attention.kernel_attention = True
    assert torch.allclose(step[:, -1], full[:, -1], rtol=0, atol=1e-2 * float(full.abs().max()))
    assert torch.equal(step[:, -1].argmax(-1), full[:, -1].argmax(-1))


# ---------------------------------------------------------------------------- fused decode chain


def _teacher_forced_agreement(model, args, batch, n_steps, prompt_len, max_seq, seed):
    """Runs the fused chain greedily; at every step feeds the same token to the op-by-op
    model and compares logits and the chosen token."""
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import make_cache

    gen_t = torch.Generator("cuda").manual_seed(seed)
    prompt = torch.randint(0, args.vocab_size, (batch, prompt_len), device="cuda", generator=gen_t)
    g = Generator(model, batch, max_seq, use_cuda_graph=False, fused=True)
    assert g.fused is not None
    g.prefill(prompt)
    # the op-by-op path keeps its own cache, filled by the same prefill
    cache = make_cache(args, batch, max_seq, "cuda")
    pos = torch.zeros(batch, dtype=torch.int64, device="cuda")
    model(prompt, pos, cache, kv_len=prompt_len)
    logits_f = torch.empty((batch, args.vocab_size), dtype=torch.float32, device="cuda")
    agree, rel = [], []
    for step in range(n_steps):
        tok_in = g.tokens.clone()
        p = g.pos.clone()
        g.fused.step(g.tokens, g.pos, g.out, logits_f)
        ref = model(tok_in, p, cache)[:, -1]
        torch.cuda.synchronize()
        agree.append((ref.argmax(-1) == g.out).float().mean().item())
        rel.append(((logits_f - ref).abs().amax(-1) / ref.abs().amax(-1)).max().item())
    assert g.fused.error_flag() == 0
    return agree, rel


def test_fused_chain_matches_op_by_op_tiny(models):
    """The chain and the op-by-op path run the same arithmetic kernel for kernel (shared
    prologue code, same attention kernel); only the bf16 output projection differs (own
    kernel vs library GEMM)."""
    args, kern, _ = models
    agree, rel = _teacher_forced_agreement(kern, args, batch=2, n_steps=100, prompt_len=9, max_seq=128, seed=11)
    assert sum(agree) / len(agree) >= 0.99
    assert max(rel) <= 1e-2


@pytest.mark.parametrize("batch", [1, 3])
def test_fused_chain_2b_shapes_256_greedy_steps(batch):
    """Two layers of the 2B architecture (real BitLinear shapes, small vocabulary):
    >= 99 % top-1 agreement over 256 greedy steps, logits within 1e-2 relative."""
    from bitnet_b200.model import build_synthetic, preset

    args = preset("2b", n_layers=2, vocab_size=4096)
    model = build_synthetic(args, seed=21, device="cuda", max_seq_len=384)
    agree, rel = _teacher_forced_agreement(model, args, batch=batch, n_steps=256, prompt_len=17, max_seq=384, seed=12)
    assert sum(agree) / len(agree) >= 0.99
    assert max(rel) <= 1e-2


def test_fused_chain_in_cuda_graph_equals_eager(models):
    from bitnet_b200.generate import Generator

    args, kern, _ = models
    prompt = torch.randint(0, args.vocab_size, (1, 8), device="cuda", generator=torch.Generator("cuda").manual_seed(4))
    a = Generator(kern, 1, 128, use_cuda_graph=True, fused=True).generate(prompt, 40)
    b = Generator(kern, 1, 128, use_cuda_graph=False, fused=True).generate(prompt, 40)
    assert torch.equal(a, b)


def test_fused_chain_odd_head_dim():
    """head_dim 100 and an FFN width that is not a multiple of 128 (the 3B preset's shapes)."""
    from bitnet_b200.model import build_synthetic, preset

    args = preset("3b", n_layers=2, vocab_size=2048)
    model = build_synthetic(args, seed=22, device="cuda", max_seq_len=128)
    agree, rel = _teacher_forced_agreement(model, args, batch=2, n_steps=64, prompt_len=5, max_seq=128, seed=13)
    assert sum(agree) / len(agree) >= 0.99
    assert max(rel) <= 1e-2


def test_chain_flags_positions_and_tokens_outside_their_ranges(models):
    """A position beyond the KV cache or a token id beyond the vocabulary must not become an
    out-of-bounds access: the kernels skip the access and leave a code in the decoder's error
    word; after clear_error the decoder works again and gives the same bits as a fresh one."""
    from bitnet_b200.generate import Generator

    args, kern, _ = models
    max_seq = 32
    prompt = torch.randint(0, args.vocab_size, (1, 6), device="cuda", generator=torch.Generator("cuda").manual_seed(8))
    g = Generator(kern, 1, max_seq, use_cuda_graph=False, fused=True)
    g.prefill(prompt)
    good_tok, good_pos = g.tokens.clone(), g.pos.clone()
    logits = torch.empty((1, args.vocab_size), dtype=torch.float32, device="cuda")
    # position == max_seq_len: flagged (4), nothing appended
    g.pos.fill_(max_seq)
    cache_before = [(k.clone(), v.clone()) for k, v in g.cache]
    g.fused.step(g.tokens, g.pos, g.out, logits)
    assert g.fused.error_flag() == 4
    for (k0, v0), (k1, v1) in zip(cache_before, g.cache):
        assert torch.equal(k0, k1) and torch.equal(v0, v1)
    g.fused.clear_error()
    assert g.fused.error_flag() == 0
    # token id == vocab_size: flagged (5)
    g.tokens.fill_(args.vocab_size)
    g.pos.copy_(good_pos)
    g.fused.step(g.tokens, g.pos, g.out, logits)
    assert g.fused.error_flag() == 5
    g.fused.clear_error()
    # a clean step afterwards equals a fresh decoder's (the first failed step appended nothing;
    # the second one wrote position good_pos, which the clean step overwrites)
    g.tokens.copy_(good_tok)
    g.pos.copy_(good_pos)
    g.fused.step(g.tokens, g.pos, g.out, logits)
    fresh = Generator(kern, 1, max_seq, use_cuda_graph=False, fused=True)
    fresh.prefill(prompt)
    logits2 = torch.empty_like(logits)
    fresh.fused.step(fresh.tokens, fresh.pos, fresh.out, logits2)
    torch.cuda.synchronize()
    assert g.fused.error_flag() == 0 and torch.equal(logits, logits2) and torch.equal(g.out, fresh.out)
    # the host side refuses a step beyond the cache before anything is launched
    h = Generator(kern, 1, 8, use_cuda_graph=False, fused=True)
    h.prefill(prompt)               # 6 tokens: positions 6 and 7 are left
    h.decode_step()
    h.decode_step()
    with pytest.raises(ValueError):
        h.decode_step()


@pytest.mark.parametrize("batch,over", [(16, {}), (33, {}), (64, dict(dim=384, n_heads=3, n_kv_heads=3, ffn_dim=200 * 4))])
def test_batched_decode_with_fused_residual_norm_quant_equals_plain_path(batch, over):
    """Batches of 16 and more decode with the residual addition, the RMSNorm and the next
    quantisation fused behind wo and w2 (bitnet_linear_w2a8_add_quant): logits and KV caches must be
    bit-identical to the same steps through the per-module path."""
    from bitnet_b200.model import build_synthetic, make_cache, preset

    args = preset("tiny", n_layers=3, **over)
    model = build_synthetic(args, seed=11, device="cuda", max_seq_len=64)
    g = torch.Generator("cuda").manual_seed(batch)
    prompt = torch.randint(0, args.vocab_size, (batch, 5), device="cuda", generator=g)
    outs = []
    for fused in (True, False):
        model.fused_decode = fused
        cache = make_cache(args, batch, 64, "cuda")
        pos = torch.zeros(batch, dtype=torch.int64, device="cuda")
        lg = model(prompt, pos, cache, kv_len=5, last_only=True)
        tok = lg[:, -1].argmax(-1, keepdim=True)
        steps = []
        for s in range(6):
            lg = model(tok, pos + 5 + s, cache)
            steps.append(lg.clone())
            tok = lg[:, -1].argmax(-1, keepdim=True)
        outs.append((torch.stack(steps), [c[0].clone() for c in cache], [c[1].clone() for c in cache]))
    model.fused_decode = True
    assert torch.equal(outs[0][0], outs[1][0])
    for a, b in zip(outs[0][1] + outs[0][2], outs[1][1] + outs[1][2]):
        assert torch.equal(a, b)
