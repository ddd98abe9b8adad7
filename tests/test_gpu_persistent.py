"""The decode step as one persistent kernel against the chain of kernels: same bits.

Both run the same arithmetic in the same order (shared prologue, attention and head code),
so logits and chosen tokens must be identical step after step, not merely close.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(args, seed, batch, max_seq, graph=False):
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import build_synthetic

    model = build_synthetic(args, seed=seed, device="cuda", max_seq_len=max_seq)
    chain = Generator(model, batch, max_seq, use_cuda_graph=graph, fused=True, persistent=False)
    pers = Generator(model, batch, max_seq, use_cuda_graph=graph, fused=True, persistent=True)
    assert not chain.persistent
    assert pers.persistent, "the persistent kernel should fit this model"
    assert pers.fused.kernels_per_step == 1
    return model, chain, pers


def _lockstep(args, chain, pers, batch, n_steps, prompt_len, seed):
    gen_t = torch.Generator("cuda").manual_seed(seed)
    prompt = torch.randint(0, args.vocab_size, (batch, prompt_len), device="cuda", generator=gen_t)
    chain.prefill(prompt)
    pers.prefill(prompt)
    la = torch.empty((batch, args.vocab_size), dtype=torch.float32, device="cuda")
    lb = torch.empty_like(la)
    for step in range(n_steps):
        chain.fused.step(chain.tokens, chain.pos, chain.out, la)
        pers.fused.step(pers.tokens, pers.pos, pers.out, lb)
        torch.cuda.synchronize()
        assert pers.fused.error_flag() == 0
        assert torch.equal(la, lb), f"logits differ at step {step}"
        assert torch.equal(chain.out, pers.out)
        assert torch.equal(chain.pos, pers.pos)
        assert torch.equal(chain.tokens, pers.tokens)
    for (ka, va), (kb, vb) in zip(chain.cache, pers.cache):
        assert torch.equal(ka, kb) and torch.equal(va, vb)


@pytest.mark.parametrize("batch", [1, 2, 8])
def test_persistent_equals_chain_tiny(batch):
    from bitnet_b200.model import preset

    args = preset("tiny")
    _, chain, pers = _pair(args, seed=31, batch=batch, max_seq=160)
    _lockstep(args, chain, pers, batch, n_steps=120, prompt_len=7, seed=5)


@pytest.mark.parametrize("batch", [1, 3, 8])
def test_persistent_equals_chain_2b_shapes(batch):
    """Three layers of the 2B architecture (real BitLinear shapes, small vocabulary)."""
    from bitnet_b200.model import preset

    args = preset("2b", n_layers=3, vocab_size=4096)
    _, chain, pers = _pair(args, seed=32, batch=batch, max_seq=320)
    _lockstep(args, chain, pers, batch, n_steps=200, prompt_len=33, seed=6)


def test_persistent_equals_chain_odd_shapes():
    """head_dim 100 and an FFN width that is not a multiple of 128 (the 3B preset's shapes)."""
    from bitnet_b200.model import preset

    args = preset("3b", n_layers=2, vocab_size=2048)
    _, chain, pers = _pair(args, seed=33, batch=2, max_seq=128)
    _lockstep(args, chain, pers, 2, n_steps=64, prompt_len=5, seed=7)


def test_persistent_in_cuda_graph():
    from bitnet_b200.model import preset

    args = preset("2b", n_layers=2, vocab_size=4096)
    _, chain, pers = _pair(args, seed=34, batch=1, max_seq=128, graph=True)
    prompt = torch.randint(0, args.vocab_size, (1, 8), device="cuda", generator=torch.Generator("cuda").manual_seed(4))
    a = chain.generate(prompt, 60)
    b = pers.generate(prompt, 60)
    assert pers.graph is not None
    assert torch.equal(a, b)
    assert pers.fused.error_flag() == 0


@pytest.mark.parametrize("persistent", [False, True])
def test_host_buffer_steps_equal_device_steps(persistent):
    """decode_step_host (ids read from and written to pinned host memory by the kernels
    themselves) gives the same tokens as device-resident steps, also when the two are mixed."""
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import build_synthetic, preset

    args = preset("2b", n_layers=2, vocab_size=4096)
    model = build_synthetic(args, seed=35, device="cuda", max_seq_len=128)
    prompt = torch.randint(0, args.vocab_size, (2, 8), device="cuda", generator=torch.Generator("cuda").manual_seed(9))
    a = Generator(model, 2, 128, fused=True, persistent=persistent)
    b = Generator(model, 2, 128, fused=True, persistent=persistent)
    ref = a.generate(prompt, 40)
    first = b.prefill(prompt)
    b.capture()
    got = [first.clone().cpu()]
    for i in range(39):
        if i % 10 < 6:
            got.append(b.decode_step_host().clone())
        else:
            with torch.cuda.stream(b.stream):
                b.decode_step()
                b.stream.synchronize()
            got.append(b.out.clone().cpu())
    assert torch.equal(torch.stack(got, dim=1), ref.cpu())
