"""Temperature + top-p sampling: the checker's restatement against the reference's formula
(gpu/sample_utils.py:8-30 evaluated with torch on the CPU), and the CUDA kernel against the checker."""
import numpy as np
import pytest
import torch

from oracle import np_oracle as o


def reference_nucleus(logits: np.ndarray, temperature: float, top_p: float) -> np.ndarray:
    """The mask of gpu/sample_utils.py:24-26 on softmax(logits / temperature) (gpu/generate.py:252)."""
    probs = torch.softmax(torch.from_numpy(logits) / temperature, dim=-1)
    ps, pi = torch.sort(probs, dim=-1, descending=True)
    drop = torch.cumsum(ps, dim=-1) - ps > top_p
    kept = np.zeros(logits.shape, dtype=bool)
    kept[pi[~drop].numpy()] = True
    return kept


@pytest.mark.parametrize("scale", [0.5, 2.0, 6.0])
@pytest.mark.parametrize("temperature,top_p", [(0.8, 0.9), (0.6, 0.95), (1.0, 0.5), (1.3, 1.0)])
def test_checker_nucleus_equals_reference_formula(scale, temperature, top_p):
    rng = np.random.default_rng(int(scale * 10) + int(top_p * 100))
    logits = (rng.standard_normal(20000) * scale).astype(np.float32)
    e, kept, margin = o.top_p_weights(logits, temperature, top_p)
    ref = reference_nucleus(logits, temperature, top_p)
    differ = np.nonzero(ref != kept)[0]
    # the reference accumulates in f32: only entries that sit on the cut within f32 rounding may
    # differ (with top_p = 1 that is the whole far tail, whose cumulative share rounds to 1)
    assert len(differ) == 0 or margin[differ].max() < 1e-5
    if top_p < 1.0:
        assert len(differ) <= 2
    assert kept[np.argmax(logits)]


def test_checker_draw_covers_the_nucleus_in_proportion():
    e = np.array([0.1, 0.4, 0.0, 0.3, 0.2], dtype=np.float32)
    kept = np.array([False, True, True, True, False])
    assert o.top_p_draw(e, kept, 0.0) == 1
    assert o.top_p_draw(e, kept, 0.5) == 1
    assert o.top_p_draw(e, kept, 0.58) == 3
    assert o.top_p_draw(e, kept, 0.999) == 3
    lo, hi = o.top_p_interval(e, kept, 3)
    assert abs(lo - 4 / 7) < 1e-6 and abs(hi - 1.0) < 1e-6  # f32 weights


def test_counter_uniform_known_values():
    # the hash is part of the interface (a seed reproduces a generation): pin it
    vals = [float(o.counter_uniform(s, r, p)) for s, r, p in ((0, 0, 0), (1234, 0, 5), (1234, 1, 5), (2**63 + 7, 63, 4095))]
    assert all(0.0 <= v < 1.0 for v in vals)
    assert vals[1] == pytest.approx(0.74680084, abs=1e-7) and vals[2] == pytest.approx(0.7388201, abs=1e-7)
    many = np.array([o.counter_uniform(7, r, p) for r in range(8) for p in range(512)])
    assert abs(many.mean() - 0.5) < 0.03 and len(np.unique(many)) > 4000


# ----------------------------------------------------------------------------------------------
# the CUDA kernel against the checker
# ----------------------------------------------------------------------------------------------

def _check_rows(logits: np.ndarray, temperature: float, top_p: float, u: np.ndarray, got: np.ndarray):
    for r in range(logits.shape[0]):
        e, kept, margin = o.top_p_weights(logits[r], temperature, top_p)
        t = int(got[r])
        assert 0 <= t < logits.shape[1]
        assert kept[t] or margin[t] < 1e-5, (r, t)
        on_cut = (margin < 1e-5).sum()
        if kept[t] and on_cut == 0:
            lo, hi = o.top_p_interval(e, kept, t)
            assert lo - 2e-6 <= u[r] <= hi + 2e-6, (r, t, lo, hi, u[r])


def _logit_cases(v: int, rows: int, kind: str, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if kind == "flat":
        return (rng.standard_normal((rows, v)) * 0.3).astype(np.float32)
    if kind == "peaked":
        return (rng.standard_normal((rows, v)) * 5.0).astype(np.float32)
    if kind == "ties":      # few distinct values: every value class has many members
        return rng.integers(-3, 4, size=(rows, v)).astype(np.float32)
    raise ValueError(kind)


@pytest.mark.gpu
@pytest.mark.parametrize("v", [1, 33, 5000, 128256])
@pytest.mark.parametrize("kind", ["flat", "peaked", "ties"])
@pytest.mark.parametrize("temperature,top_p", [(0.8, 0.9), (0.6, 0.95), (1.0, 0.3)])
def test_kernel_draw_equals_checker(v, kind, temperature, top_p):
    from bitnet_b200 import ops
    rows = 6
    logits = _logit_cases(v, rows, kind, seed=v + int(100 * top_p))
    u = np.array([0.0, 0.17, 0.5, 0.83, 0.999, 0.31], dtype=np.float32)
    got = ops.sample_top_p(torch.from_numpy(logits).cuda(), temperature, top_p, uniforms=torch.from_numpy(u).cuda())
    _check_rows(logits, temperature, top_p, u, got.cpu().numpy())


@pytest.mark.gpu
def test_kernel_limits_of_top_p_and_row_stride():
    from bitnet_b200 import ops
    logits = _logit_cases(4096, 8, "peaked", 3)
    padded = torch.zeros((8, 4100), dtype=torch.float32, device="cuda")
    padded[:, :4096] = torch.from_numpy(logits).cuda()
    padded[:, 4096:] = 100.0            # beyond the vocabulary: must never be chosen
    u = torch.rand(8, device="cuda", generator=torch.Generator("cuda").manual_seed(9))
    view = padded[:, :4096]
    assert (ops.sample_top_p(view, 0.7, 0.0, uniforms=u).cpu().numpy() == logits.argmax(-1)).all()
    got = ops.sample_top_p(view, 1.0, 1.0, uniforms=u).cpu().numpy()
    _check_rows(logits, 1.0, 1.0, u.cpu().numpy(), got)
    tokens = torch.full((8,), -1, dtype=torch.int64, device="cuda")
    out = ops.sample_top_p(view, 1.0, 5.0, uniforms=u, tokens=tokens)
    assert (out == tokens).all() and (out.cpu().numpy() == got).all()


@pytest.mark.gpu
def test_kernel_counter_hash_equals_checker():
    from bitnet_b200 import ops
    logits = _logit_cases(5000, 16, "flat", 11)
    pos = np.arange(100, 116, dtype=np.int64) * 37
    dev = torch.from_numpy(logits).cuda()
    for seed in (0, 1234, 2**63 + 7):
        u = np.array([o.counter_uniform(seed, r, int(pos[r])) for r in range(16)], dtype=np.float32)
        a = ops.sample_top_p(dev, 0.9, 0.9, seed=seed, pos=torch.from_numpy(pos).cuda())
        b = ops.sample_top_p(dev, 0.9, 0.9, uniforms=torch.from_numpy(u).cuda())
        assert (a == b).all()
    _check_rows(logits, 0.9, 0.9, u, a.cpu().numpy())


@pytest.mark.gpu
def test_kernel_frequencies_follow_the_renormalised_nucleus():
    from bitnet_b200 import ops
    row = np.array([2.0, 1.0, 0.5, 0.0, -1.0, 1.5, -3.0, 0.7], dtype=np.float32)
    n = 40000
    logits = torch.from_numpy(row).cuda().repeat(n, 1).contiguous()
    g = torch.Generator(device="cuda").manual_seed(5)
    got = ops.sample_top_p(logits, 0.8, 0.9, uniforms=torch.rand(n, device="cuda", generator=g)).cpu().numpy()
    e, kept, _ = o.top_p_weights(row, 0.8, 0.9)
    want = np.where(kept, e.astype(np.float64), 0.0)
    want /= want.sum()
    freq = np.bincount(got, minlength=8) / n
    assert (freq[~kept] == 0).all()
    assert np.abs(freq - want).max() < 5 * np.sqrt(0.25 / n)


@pytest.mark.gpu
def test_bad_arguments_are_refused():
    from bitnet_b200 import _lib, ops
    logits = torch.zeros((2, 16), dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.BitnetError):
        ops.sample_top_p(logits, 0.0, 0.9)
    with pytest.raises(_lib.BitnetError):
        ops.sample_top_p(logits, 1.0, -0.1)


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])
def test_generator_samples_reproducibly(fused):
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import build_synthetic, preset

    args = preset("tiny", n_layers=2)
    model = build_synthetic(args, seed=5, device="cuda", max_seq_len=64)
    # a fixed prompt: with a random one the tiny model now and then falls into a loop whose next
    # token has probability > top_p, where sampling and argmax rightly agree on every token
    prompt = torch.randint(0, args.vocab_size, (2, 8), device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    runs = []
    for seed, graph in ((3, True), (3, False), (4, True)):
        gen = Generator(model, batch=2, max_seq_len=64, use_cuda_graph=graph, fused=fused, temperature=0.8, top_p=0.9, seed=seed)
        runs.append(gen.generate(prompt, 24).cpu().numpy())
        assert runs[-1].min() >= 0 and runs[-1].max() < args.vocab_size
    assert (runs[0] == runs[1]).all()          # graph replay draws the same numbers as eager launches
    assert (runs[0] != runs[2]).any()          # another seed, another continuation
    greedy = Generator(model, batch=2, max_seq_len=64, fused=fused).generate(prompt, 24).cpu().numpy()
    assert (greedy != runs[0]).any()


# ----------------------------------------------------------------------------------------------
# properties of the checker itself (any logits)
# ----------------------------------------------------------------------------------------------

def test_checker_properties_on_random_rows():
    from hypothesis import given, settings, strategies as st
    from hypothesis.extra import numpy as hnp

    @settings(max_examples=60, deadline=None)
    @given(hnp.arrays(np.float32, st.integers(1, 300), elements=st.floats(-30, 30, width=32)),
           st.floats(0.05, 2.0), st.floats(0.0, 1.0), st.floats(0.0, 0.999))
    def check(logits, temperature, top_p, u):
        e, kept, _ = o.top_p_weights(logits, temperature, top_p)
        # the most probable entry is always kept; what is kept is a prefix of the descending order
        assert kept[np.argmax(e)]
        assert e[kept].min() >= e[~kept].max() if (~kept).any() else True
        # the kept mass reaches top_p of the total as soon as anything is dropped
        if (~kept).any():
            assert e[kept].astype(np.float64).sum() >= top_p * e.astype(np.float64).sum() * (1 - 1e-12)
        # a draw is a kept entry of positive mass whose interval holds u
        t = o.top_p_draw(e, kept, u)
        assert kept[t] and e[t] > 0
        lo, hi = o.top_p_interval(e, kept, t)
        assert lo <= u < hi or abs(u - lo) < 1e-12 or abs(u - hi) < 1e-12

    check()
