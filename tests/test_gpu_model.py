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


def test_kernel_model_matches_fake_quant_reference(models):
    """Same ternary weights, same arithmetic up to bf16 rounding: logits within 1e-2
    relative (of the logit scale) and the same greedy token."""
    from bitnet_b200.model import make_cache

    args, kern, ref = models
    B, T = 2, 12
    toks = torch.randint(0, args.vocab_size, (B, T), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    pos = torch.zeros(B, dtype=torch.int64, device="cuda")
    lk = kern(toks, pos, make_cache(args, B, 128, "cuda"), kv_len=T)
    lr = ref(toks, pos, make_cache(args, B, 128, "cuda"), kv_len=T)
    scale = lr.abs().max()
    assert (lk - lr).abs().max() / scale <= 1e-2
    assert (lk.argmax(-1) == lr.argmax(-1)).float().mean() >= 0.99


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
    for t in range(T):
        step = kern(toks[:, t:t + 1], pos + t, cache)
    assert torch.allclose(step[:, -1], full[:, -1], rtol=0, atol=1e-2 * float(full.abs().max()))
    assert torch.equal(step[:, -1].argmax(-1), full[:, -1].argmax(-1))
