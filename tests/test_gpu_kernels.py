"""Parity of the CUDA kernels with the CPU oracle, called through the C ABI (needs a B200)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import np_oracle as O

pytestmark = pytest.mark.gpu

S2B = [(3840, 2560), (2560, 2560), (13824, 2560), (2560, 6912)]


@pytest.fixture(scope="module")
def bn():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from bitnet_b200 import _lib, ops, pack_weight

    class NS:
        pass

    ns = NS()
    ns.lib, ns.ops, ns.pack, ns._lib = _lib.lib, ops, pack_weight, _lib
    return ns


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ---------------------------------------------------------------------------- layouts


@pytest.mark.parametrize("n,k", [(16, 128), (48, 384), (20, 200), (2560, 2560), (100, 8640)])
def test_pack_ternary_matches_layout_definition(bn, n, k):
    rng = np.random.default_rng(n + k)
    q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
    packed = bn.pack.convert_weight_int8_to_int2(_dev(q))
    n_pad, k_pad = O.w2t_shape(n, k)
    assert tuple(packed.shape) == (n_pad, k_pad // 4) and packed.dtype == torch.int8
    assert np.array_equal(packed.cpu().numpy().reshape(-1).view(np.uint8), O.w2t_pack(q))
    assert np.array_equal(bn.pack.unpack_int2_to_int8(packed, n, k).cpu().numpy(), q)


def test_pack_from_reference_gpu_layout(bn, golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_gpu_pack.npz"))
    for i in range(4):
        q, ref_packed = g[f"q_{i}"], g[f"packed_{i}"]
        got = bn.pack.convert_ref_int2_to_w2t(_dev(ref_packed))
        assert np.array_equal(got.cpu().numpy().reshape(-1).view(np.uint8), O.w2t_pack(q))


def test_pack_from_i2s_and_code3(bn, golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_i2s.npz"))
    for i in range(6):
        w, buf = g[f"w_{i}"], g[f"i2s_{i}"]
        n, k = w.shape
        got = bn.pack.convert_i2s_to_w2t(_dev(buf), n, k)
        assert np.array_equal(got.cpu().numpy().reshape(-1).view(np.uint8), O.w2t_pack(np.sign(w).astype(np.int8)))
    # raw bytes: code 3 survives the conversion and is used literally by the matmul
    raw, y = g["raw_bytes"], g["raw_y"]
    n, k = 8, 512
    w2t = bn.pack.convert_i2s_to_w2t(_dev(raw), n, k)
    zero = torch.zeros(y.shape[0], dtype=torch.int32, device="cuda")
    acc = bn.ops.linear_w2a8(_dev(y), None, zero, w2t, None, [n], n, k, want_acc=True, want_out=False)
    assert np.array_equal(acc.cpu().numpy().astype(np.float32), g["raw_gemm"])


def test_quantize_i2_s_bytes_identical_to_reference(bn, golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_i2s.npz"))
    for i in range(6):
        w, buf = np.ascontiguousarray(g[f"w_{i}"]), g[f"i2s_{i}"]
        n, k = w.shape
        out = np.full(n * k // 4 + 32, 0xAB, dtype=np.uint8)
        sz = bn.lib.quantize_i2_s(w.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), n, k, None)
        assert sz == out.size and bn.lib.bitnet_last_status() == 0
        assert np.array_equal(out, buf)


def test_vec_dot_shim_matches_reference_results(bn, golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_i2s.npz"))
    for i in range(6):
        buf, y, dot = g[f"i2s_{i}"], np.ascontiguousarray(g[f"y_{i}"]), g[f"dot_{i}"]
        m, k = y.shape
        n = dot.shape[1]
        for r in range(min(n, 3)):
            row = np.ascontiguousarray(buf[r * k // 4:(r + 1) * k // 4])
            for nrc in ([4] if m >= 4 else []) + [1]:
                s = np.zeros(nrc, dtype=np.float32)
                bn.lib.ggml_vec_dot_i2_i8_s(k, s.ctypes.data_as(ctypes.c_void_p), 1, row.ctypes.data_as(ctypes.c_void_p),
                                            k, y.ctypes.data_as(ctypes.c_void_p), k, nrc)
                assert bn.lib.bitnet_last_status() == 0
                assert np.array_equal(s, dot[:nrc, r])
        # several weight rows against one activation row (the 1x1 form, nrc % 4 != 0)
        if n >= 3:
            s = np.zeros(3, dtype=np.float32)
            x3 = np.ascontiguousarray(buf[: 3 * k // 4])
            bn.lib.ggml_vec_dot_i2_i8_s(k, s.ctypes.data_as(ctypes.c_void_p), 1, x3.ctypes.data_as(ctypes.c_void_p), k,
                                        y.ctypes.data_as(ctypes.c_void_p), k, 3)
            assert np.array_equal(s, dot[0, :3])


# ---------------------------------------------------------------------------- matmul parity


def _oracle_case(n, k, m, seed, port_lib, ref_lib=None):
    q, ws = O.synth_weights(n, k, seed)
    x = O.synth_acts(m, k, seed + 1)
    y, a, ysum = O.act_quant(x)
    acc = O.matmul_i32(y, q)
    if k % 128 == 0 and (n * k) % 128 == 0:
        buf = O.i2s_pack(q, ws)
        code_sum = port_lib.gemm(buf, y, n, k)
        assert np.array_equal(code_sum - ysum[:, None], acc)
        if ref_lib is not None:                       # the reference's own compiled kernel
            assert np.array_equal(ref_lib.gemm(buf, y, n, k, threads=4), code_sum.astype(np.float32))
    return q, ws, x, y, a, ysum, acc


@pytest.mark.parametrize("n,k", S2B)
@pytest.mark.parametrize("m", [1, 8, 32])
def test_gemv_sweep_int32_exact_and_bf16(bn, port_lib, ref_lib, n, k, m):
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=n + k + m, port_lib=port_lib,
                                              ref_lib=ref_lib if m <= 8 else None)
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    wsd = _dev(np.array([ws], dtype=np.float32))
    for ys in (None, _dev(ysum)):
        out, got = bn.ops.linear_w2a8(_dev(y), _dev(a), ys, w2t, wsd, [n], n, k, want_acc=True)
        assert np.array_equal(got.cpu().numpy(), acc)                       # bit-exact int32
        want = O.to_bf16(O.rescale(acc, a, [ws]))
        got_f = out.float().cpu().numpy()
        assert np.array_equal(got_f, want)                                   # same f32 ops -> same bf16
        rel = np.abs(got_f - want) / np.maximum(np.abs(want), 1e-6)
        assert rel.max() <= 1e-2                                             # the stated tolerance


@pytest.mark.parametrize("n,k", S2B)
@pytest.mark.parametrize("m", [128, 512, 2048])
def test_kernel_sweep_grid_large_m(bn, port_lib, n, k, m):
    """The remaining cells of the isolated-kernel sweep (the four 2B shapes x M in {1, 8, 32,
    128, 512, 2048}; the small M are covered above): padded int8 activations with their sums, as
    the model hands them over, int32 sums bit-exact against the C port of the reference kernel
    and bf16 outputs equal to the oracle's rescale."""
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=3 * n + k + m, port_lib=port_lib)
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    gy, ga, gs = bn.ops.quant_input(_dev(x).bfloat16())
    assert np.array_equal(gy.cpu().numpy()[:, :k], y) and np.array_equal(gs.cpu().numpy(), ysum)
    wsd = _dev(np.array([ws], dtype=np.float32))
    out, got = bn.ops.linear_w2a8(gy, ga, gs, w2t, wsd, [n], n, k, want_acc=True)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), acc)                           # bit-exact int32
    want = O.to_bf16(O.rescale(acc, a, [ws]))
    got_f = out.float().cpu().numpy()
    assert (np.abs(got_f - want) <= 1e-2 * np.maximum(np.abs(want), 1e-6)).all()   # the stated tolerance
    assert np.array_equal(got_f, want)                                       # same f32 operations -> same bf16


@pytest.mark.parametrize("n,k,m", [(2560, 2560, 128), (3840, 2560, 16), (13824, 2560, 512), (2560, 6912, 130)])
def test_reference_entry_point_many_tokens(bn, port_lib, n, k, m):
    """bitlinear_int8xint2 with M >= 16 (the reference's symbol takes plain [M, K] int8 rows and
    no row sums, gpu/model.py:21-37): same bf16 results as the oracle, per-token scales."""
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=n + 7 * m, port_lib=port_lib)
    s_bf = O.to_bf16(a)
    ws_bf = O.to_bf16(np.array([0.5, 1.25, 0.875, 2.0], dtype=np.float32))
    seg = O.ref_gpu_scale_segments(n, k)
    weight = bn.pack.convert_weight_int8_to_int2(_dev(q))
    out = bn.ops.bitnet_int8xint2_linear(_dev(y), weight, _dev(s_bf).bfloat16(), _dev(ws_bf).bfloat16())
    torch.cuda.synchronize()
    want = O.to_bf16(O.rescale(acc, s_bf, ws_bf[: len(seg)], seg))
    assert np.array_equal(out.float().cpu().numpy(), want)


def test_reference_gpu_kernel_agrees(bn):
    """The reference's own GPU kernel (gpu/bitnet_kernels/bitnet_kernels.cu, built with its own
    command line, loaded from PTX) on its own packing against this library's symbol on the W2T
    packing of the same weights: identical bf16 outputs for the four 2B shapes at M = 1."""
    from oracle import build_oracle

    path = build_oracle.build_ref_gpu()
    if not path:
        pytest.skip("the reference's GPU kernel library is not available")
    try:
        ref = ctypes.CDLL(path)
    except OSError as exc:
        pytest.skip(f"the reference's GPU kernel library does not load here: {exc}")
    ref.bitlinear_int8xint2.restype = None
    ref.bitlinear_int8xint2.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    for n, k in S2B:
        q, _ = O.synth_weights(n, k, seed=n + k)
        y, a, ysum = O.act_quant(O.synth_acts(1, k, seed=k + 1))
        s_bf = _dev(O.to_bf16(a)).bfloat16()
        ws_bf = _dev(O.to_bf16(np.array([0.5, 1.25, 0.875, 2.0], dtype=np.float32))).bfloat16()
        yd = _dev(y)
        ref_w = _dev(O.ref_gpu_pack(q))
        ref_out = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        ref.bitlinear_int8xint2(bn._lib.ptr(yd), bn._lib.ptr(ref_w), bn._lib.ptr(ref_out), bn._lib.ptr(s_bf),
                                bn._lib.ptr(ws_bf), 1, n, k, bn._lib.stream_ptr())
        torch.cuda.synchronize()
        ours = bn.ops.bitnet_int8xint2_linear(yd, bn.pack.convert_ref_int2_to_w2t(ref_w), s_bf, ws_bf)
        torch.cuda.synchronize()
        if not ref_out.any():
            pytest.skip("the reference kernel's PTX produced no output on this GPU")
        assert torch.equal(ours, ref_out), (n, k)


@pytest.mark.parametrize("n,k,m", [(2560, 2560, 128), (3840, 2560, 65), (2560, 6912, 130), (13824, 2560, 512)])
def test_large_m_int32_exact(bn, port_lib, n, k, m):
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=5 * n + m, port_lib=port_lib)
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    got = bn.ops.linear_w2a8(_dev(y), None, None, w2t, None, [n], n, k, want_acc=True, want_out=False)
    assert np.array_equal(got.cpu().numpy(), acc)


@pytest.mark.parametrize("n,k,m", [(16, 128, 1), (20, 200, 3), (33, 8640, 9), (130, 384, 17), (3200, 8640, 1),
                                    (48, 128, 33), (64, 3200, 64), (17, 131, 2)])
def test_ragged_shapes(bn, port_lib, n, k, m):
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=n * 7 + k + m, port_lib=port_lib)
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    # unpadded activation rows (ldy = K, possibly unaligned) and padded ones
    got = bn.ops.linear_w2a8(_dev(y), None, None, w2t, None, [n], n, k, want_acc=True, want_out=False)
    assert np.array_equal(got.cpu().numpy(), acc)
    k_pad = (k + 127) // 128 * 128
    ypad = np.zeros((m, k_pad), dtype=np.int8)
    ypad[:, :k] = y
    got = bn.ops.linear_w2a8(_dev(ypad), None, _dev(ysum), w2t, None, [n], n, k, want_acc=True, want_out=False)
    assert np.array_equal(got.cpu().numpy(), acc)


def test_extreme_values_do_not_overflow(bn):
    """All +1 weights x all -128 / +127 activations at the largest K of the configs."""
    n, k = 32, 32768
    q = np.ones((n, k), dtype=np.int8)
    y = np.stack([np.full(k, 127, dtype=np.int8), np.full(k, -128, dtype=np.int8)])
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    got = bn.ops.linear_w2a8(_dev(y), None, None, w2t, None, [n], n, k, want_acc=True, want_out=False)
    assert np.array_equal(got.cpu().numpy(), O.matmul_i32(y, q))


def test_scale_segments(bn, port_lib):
    n, k, m = 3840, 2560, 4
    q, _, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=99, port_lib=port_lib)
    ws = np.array([0.75, 1.5, 0.31], dtype=np.float32)
    seg = [2560, 3200, 3840]                       # q, k, v rows of the fused wqkv
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    out = bn.ops.linear_w2a8(_dev(y), _dev(a), _dev(ysum), w2t, _dev(ws), seg, n, k)
    assert np.array_equal(out.float().cpu().numpy(), O.to_bf16(O.rescale(acc, a, ws, seg)))


def test_reference_entry_point_known_answer(bn, golden_dir):
    """gpu/test.py:42-61 through the unchanged symbol: all scales 1, bf16 equality."""
    g = np.load(os.path.join(golden_dir, "ref_gpu_test_kat.npz"))
    for i in range(3):
        n, k, seed = (int(v) for v in g[f"shape_{i}"])
        if n % 16 or k % 128:
            continue
        rng = np.random.default_rng(seed)
        q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
        y = rng.integers(-128, 127, size=(1, k), dtype=np.int8)
        weight = bn.pack.convert_weight_int8_to_int2(_dev(q))
        if f"ref_packed_{i}" in g:                  # a checkpoint packed by the reference converts to the same bytes
            assert torch.equal(bn.pack.convert_ref_int2_to_w2t(_dev(g[f"ref_packed_{i}"])), weight)
        s = torch.ones(1, dtype=torch.bfloat16, device="cuda")
        ws = torch.ones(6, dtype=torch.bfloat16, device="cuda")
        ret = torch.empty((1, n), dtype=torch.bfloat16, device="cuda")
        out = bn.ops.bitnet_int8xint2_linear(_dev(y), weight, s, ws, ret)
        assert np.array_equal(out.view(torch.int16).cpu().numpy(), g[f"expect_bf16_bits_{i}"])


@pytest.mark.parametrize("n,k", [(3840, 2560), (13824, 2560), (4800, 3200), (3200, 3200)])
def test_reference_entry_point_scale_ladder(bn, n, k):
    """The reference picks ws[row // (N/ws_num)] with ws_num fixed per shape
    (gpu/bitnet_kernels/bitnet_kernels.cu:4-33); the drop-in symbol does the same."""
    q, _ = O.synth_weights(n, k, seed=n)
    y, a, ysum = O.act_quant(O.synth_acts(1, k, seed=k))
    s_bf = O.to_bf16(a)
    ws_bf = O.to_bf16(np.array([0.5, 1.25, 0.875, 2.0, 0.75, 1.5], dtype=np.float32))
    seg = O.ref_gpu_scale_segments(n, k)
    weight = bn.pack.convert_weight_int8_to_int2(_dev(q))
    out = bn.ops.bitnet_int8xint2_linear(_dev(y), weight, _dev(s_bf).bfloat16(), _dev(ws_bf).bfloat16())
    want = O.to_bf16(O.rescale(O.matmul_i32(y, q), s_bf, ws_bf[: len(seg)], seg))
    assert np.array_equal(out.float().cpu().numpy(), want)


def test_reference_entry_point_rejects_bad_shapes(bn):
    t = torch.zeros(64, dtype=torch.int8, device="cuda")
    b = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    bn.lib.bitlinear_int8xint2(bn._lib.ptr(t), bn._lib.ptr(t), bn._lib.ptr(b), bn._lib.ptr(b), bn._lib.ptr(b), 1, 20, 128, None)
    assert bn.lib.bitnet_last_status() == 2
    bn.lib.bitlinear_int8xint2(bn._lib.ptr(t), None, bn._lib.ptr(b), bn._lib.ptr(b), bn._lib.ptr(b), 1, 16, 128, None)
    assert bn.lib.bitnet_last_status() == 1
    assert not b.any()                              # nothing was launched


# ---------------------------------------------------------------------------- activation prologue


def test_quant_input_exact(bn):
    x = O.synth_acts(9, 2560, seed=1)
    x[3] = 0.0
    x[5, 7] = 3e4
    x = O.to_bf16(x)
    y, a, ysum = O.act_quant(x)
    gy, ga, gs = bn.ops.quant_input(_dev(x).bfloat16())
    assert np.array_equal(gy.cpu().numpy(), y)
    assert np.array_equal(ga.cpu().numpy(), a) and np.array_equal(gs.cpu().numpy(), ysum)


def test_quant_input_pads_ragged_k(bn):
    x = O.synth_acts(3, 8640, seed=2)
    y, a, ysum = O.act_quant(x)
    gy, ga, gs = bn.ops.quant_input(_dev(x).bfloat16())
    assert gy.shape[1] == 8704 and not gy[:, 8640:].any()
    assert np.array_equal(gy[:, :8640].cpu().numpy(), y) and np.array_equal(gs.cpu().numpy(), ysum)


def test_rmsnorm_quant_close_to_oracle(bn):
    k = 6912
    x = O.synth_acts(5, k, seed=3)
    g = O.to_bf16(np.random.default_rng(4).uniform(0.5, 1.5, k).astype(np.float32))
    xn = O.to_bf16(O.rmsnorm(x, g, 1e-5))
    y, a, ysum = O.act_quant(xn)
    gy, ga, gs = bn.ops.quant_input(_dev(x).bfloat16(), _dev(g).bfloat16(), 1e-5)
    d = np.abs(gy.cpu().numpy().astype(np.int32) - y.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01   # rsqrt rounding may move a value across a .5 boundary
    assert np.allclose(ga.cpu().numpy(), a, rtol=1e-2)
    assert np.array_equal(gs.cpu().numpy(), gy.cpu().numpy().astype(np.int32).sum(-1))


@pytest.mark.parametrize("m,k", [(1, 6912), (5, 8640), (64, 6912), (3, 200)])
def test_quant_input_glu_equals_gate_then_quant(bn, m, k):
    """The gate of the feed-forward block fused into the quantisation kernel gives the bytes that
    the bf16 tensor operations followed by the plain kernel give."""
    g = torch.Generator("cuda").manual_seed(100 * m + k)
    x13 = (torch.randn((m, 2 * k), generator=g, device="cuda") * 2).bfloat16()
    gamma = (torch.rand((k,), generator=g, device="cuda") + 0.5).bfloat16()
    x1, x3 = x13.chunk(2, -1)
    gated = torch.relu(x1) ** 2 * x3
    for gm in (None, gamma):
        want = bn.ops.quant_input(gated, gm, 1e-5)
        got = bn.ops.quant_input_glu(x13, gm, 1e-5)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


# ---------------------------------------------------------------------------- tcgen05 path (M >= 16)


@pytest.mark.parametrize("n,k,m", [(2560, 2560, 16), (3840, 2560, 33), (48, 384, 64), (2560, 6912, 100),
                                    (13824, 2560, 128), (272, 200, 130), (2560, 2560, 300)])
def test_tensor_core_path_int32_exact_and_bf16(bn, port_lib, n, k, m):
    """Batches of 16 and more tokens with padded activations and their sums go to the tcgen05
    kernel; its int32 sums are exact and its bf16 outputs equal the oracle's."""
    q, ws, x, y, a, ysum, acc = _oracle_case(n, k, m, seed=11 * n + m, port_lib=port_lib)
    w2t = bn.pack.convert_weight_int8_to_int2(_dev(q))
    gy, ga, gs = bn.ops.quant_input(_dev(x).bfloat16())            # padded to 128 columns, with sums
    assert np.array_equal(gy.cpu().numpy()[:, :k], y)
    wsd = _dev(np.array([ws], dtype=np.float32))
    out, got = bn.ops.linear_w2a8(gy, ga, gs, w2t, wsd, [n], n, k, want_acc=True)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), acc)
    assert np.array_equal(out.float().cpu().numpy(), O.to_bf16(O.rescale(acc, a, [ws])))
