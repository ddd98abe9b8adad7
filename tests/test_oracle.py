"""The CPU checkers against the reference's golden vectors (no GPU needed)."""
import os

import numpy as np
import pytest

from oracle import np_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_ref_gpu_pack_matches_reference_packer(golden_dir):
    g = _load(golden_dir, "ref_gpu_pack.npz")
    for i in range(4):
        q, packed = g[f"q_{i}"], g[f"packed_{i}"]
        mine = O.ref_gpu_pack(q)
        assert mine.dtype == np.int8 and mine.shape == packed.shape
        assert np.array_equal(mine, packed)
        assert np.array_equal(O.ref_gpu_unpack(packed, *q.shape), q)


def test_i2s_pack_and_dot_match_compiled_reference(golden_dir, port_lib):
    g = _load(golden_dir, "ref_i2s.npz")
    for i in range(6):
        w, buf, y = g[f"w_{i}"], g[f"i2s_{i}"], g[f"y_{i}"]
        n, k = w.shape
        # bytes + scale: C port, NumPy restatement
        assert np.array_equal(port_lib.quantize_i2_s(w), buf)
        scale = np.abs(w).max()
        q = np.sign(w).astype(np.int8)
        assert np.array_equal(O.i2s_pack(q, scale), buf)
        assert O.i2s_scale(buf, n, k) == np.float32(scale)
        assert np.array_equal(O.i2s_codes(buf, n, k).astype(np.int8) - 1, q)
        # exact int32 code sums == what the reference kernel returned as floats
        exact = O.matmul_i32(y, q + 1)
        assert np.array_equal(exact.astype(np.float32), g[f"dot_{i}"])
        assert np.array_equal(exact.astype(np.float32), g[f"gemm_{i}"])
        assert np.array_equal(port_lib.gemm(buf, y, n, k), exact)


def test_code3_is_taken_literally(golden_dir, port_lib):
    g = _load(golden_dir, "ref_i2s.npz")
    raw, y = g["raw_bytes"], g["raw_y"]
    n, k = 8, 512
    codes = O.i2s_codes(raw, n, k)
    assert (codes == 3).any()
    exact = O.matmul_i32(y, codes.astype(np.int8))
    assert np.array_equal(exact.astype(np.float32), g["raw_gemm"])
    assert np.array_equal(port_lib.gemm(raw, y, n, k), exact)


def test_gpu_known_answer_vectors(golden_dir):
    g = _load(golden_dir, "ref_gpu_test_kat.npz")
    import torch

    for i in range(3):
        n, k, seed = (int(v) for v in g[f"shape_{i}"])
        rng = np.random.default_rng(seed)
        q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
        y = rng.integers(-128, 127, size=(1, k), dtype=np.int8)
        if f"q_{i}" in g:
            assert np.array_equal(q, g[f"q_{i}"]) and np.array_equal(y, g[f"y_{i}"])
            assert np.array_equal(O.ref_gpu_pack(q), g[f"ref_packed_{i}"])
        acc = O.matmul_i32(y, q)
        bits = torch.from_numpy(O.to_bf16(acc.astype(np.float32))).to(torch.bfloat16).view(torch.int16).numpy()
        assert np.array_equal(bits, g[f"expect_bf16_bits_{i}"])


def test_live_reference_agrees_with_port(ref_lib, port_lib):
    """Random shapes through the compiled reference (when present) vs the exact port,
    restricted to inputs whose int16 lane partials cannot wrap in the reference."""
    rng = np.random.default_rng(7)
    for n, k, m in [(16, 2560, 1), (12, 6912, 4), (130, 384, 5), (4, 128, 9)]:
        q, s = O.synth_weights(n, k, seed=int(rng.integers(1 << 30)))
        y, a, ysum = O.act_quant(O.synth_acts(m, k, seed=int(rng.integers(1 << 30))))
        w = q.astype(np.float32) * s
        buf = ref_lib.quantize_i2_s(w)
        assert np.array_equal(buf, port_lib.quantize_i2_s(w))
        got = ref_lib.gemm(buf, y, n, k, threads=2)
        exact = port_lib.gemm(buf, y, n, k)
        assert np.array_equal(got, exact.astype(np.float32))
        assert np.array_equal(exact - ysum[:, None], O.matmul_i32(y, q))


def test_reference_int16_lanes_wrap_on_adversarial_input(ref_lib, port_lib):
    """All +1 weights x all 127 activations overflow the reference's int16 partial sums
    (src/ggml-bitnet-mad.cpp:218-254); exact parity is defined only away from that."""
    n, k = 4, 2560
    w = np.ones((n, k), dtype=np.float32)
    y = np.full((1, k), 127, dtype=np.int8)
    buf = ref_lib.quantize_i2_s(w)
    exact = port_lib.gemm(buf, y, n, k)
    assert (exact == 2 * 127 * k).all()
    assert not np.array_equal(ref_lib.gemm(buf, y, n, k), exact.astype(np.float32))


def test_act_quant_port_equals_numpy(port_lib):
    x = O.synth_acts(7, 2560, seed=3)
    x[3] = 0.0                      # all-zero token: absmax clamps at 1e-5
    x[4, 0] = 1e9
    y0, a0, s0 = O.act_quant(x)
    y1, a1, s1 = port_lib.act_quant(x)
    assert np.array_equal(y0, y1) and np.array_equal(a0, a1) and np.array_equal(s0, s1)
    assert (y0[3] == 0).all() and a0[3] == np.float32(127.0) / np.float32(1e-5)


def test_ternarize_distribution():
    q, s = O.synth_weights(256, 2560, seed=11)
    frac0 = (q == 0).mean()
    assert 0.28 < frac0 < 0.36 and abs((q == 1).mean() - (q == -1).mean()) < 0.01
    assert set(np.unique(q)) == {-1, 0, 1}


@pytest.mark.parametrize("n,k", [(16, 128), (48, 384), (20, 200), (2560, 2560)])
def test_w2t_layout_roundtrip(n, k):
    rng = np.random.default_rng(n * 131 + k)
    q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
    buf = O.w2t_pack(q)
    n_pad, k_pad = O.w2t_shape(n, k)
    assert buf.size == n_pad * k_pad // 4
    assert np.array_equal(O.w2t_codes(buf, n, k).astype(np.int8) - 1, q)


def test_w2t_lane_view():
    """The layout as a warp sees it: lane (g,q) word r AND-masked with 0x03030303 << 2j is
    4^j times the codes of row g+8(r&1), columns 32q+8j+4(r>>1)+[0..3]."""
    rng = np.random.default_rng(5)
    q = rng.integers(-1, 2, size=(16, 128), dtype=np.int8)
    words = O.w2t_pack(q).view(np.uint32)
    for lane in range(32):
        g, qq = lane // 4, lane % 4
        for r in range(4):
            w = int(words[lane * 4 + r])
            for j in range(4):
                f = (w & (0x03030303 << (2 * j))) >> (2 * j)
                for b in range(4):
                    code = (f >> (8 * b)) & 0xFF
                    assert code == q[g + 8 * (r & 1), 32 * qq + 8 * j + 4 * (r >> 1) + b] + 1
