"""The reference's ggml backend entry points (include/ggml-bitnet.h:27-40) on the GPU kernels."""
import ctypes

import numpy as np
import pytest

from oracle import np_oracle as O

GGML_TYPE_F32, GGML_TYPE_Q4_0, GGML_TYPE_I2_S, GGML_TYPE_TL2 = 0, 2, 36, 39


class Tensor(ctypes.Structure):
    pass


Tensor._fields_ = [("type", ctypes.c_int), ("ne", ctypes.c_int64 * 4), ("nb", ctypes.c_size_t * 4),
                   ("src", ctypes.POINTER(Tensor) * 2), ("data", ctypes.c_void_p), ("extra", ctypes.c_void_p)]


class Params(ctypes.Structure):
    _fields_ = [("ith", ctypes.c_int), ("nth", ctypes.c_int), ("wsize", ctypes.c_size_t), ("wdata", ctypes.c_void_p)]


class Extra(ctypes.Structure):
    _fields_ = [("lut_scales_size", ctypes.c_int), ("BK", ctypes.c_int), ("n_tile_num", ctypes.c_int),
                ("qweights", ctypes.c_void_p), ("scales", ctypes.POINTER(ctypes.c_float))]


def _tensor(ttype, ne0, ne1, array=None):
    t = Tensor()
    t.type = ttype
    t.ne[0], t.ne[1], t.ne[2], t.ne[3] = ne0, ne1, 1, 1
    if array is not None:
        t.data = array.ctypes.data
    return t


@pytest.fixture(scope="module")
def L():
    from bitnet_b200 import _lib

    return _lib.lib


def test_host_side_logic_without_gpu(L):
    L.ggml_bitnet_init()
    L.ggml_bitnet_init()                                   # idempotent
    assert L.ggml_bitnet_get_type_bits(GGML_TYPE_I2_S) == 2
    assert L.ggml_bitnet_get_type_bits(GGML_TYPE_TL2) == 2
    assert L.ggml_bitnet_get_type_bits(GGML_TYPE_Q4_0) == 4
    assert L.ggml_bitnet_get_type_bits(GGML_TYPE_F32) == 0
    w, x, d = _tensor(GGML_TYPE_I2_S, 2560, 3840), _tensor(GGML_TYPE_F32, 2560, 5), _tensor(GGML_TYPE_F32, 3840, 5)
    assert L.ggml_bitnet_can_mul_mat(ctypes.byref(w), ctypes.byref(x), ctypes.byref(d))
    bad = _tensor(GGML_TYPE_Q4_0, 2560, 3840)
    assert not L.ggml_bitnet_can_mul_mat(ctypes.byref(bad), ctypes.byref(x), ctypes.byref(d))
    odd = _tensor(GGML_TYPE_I2_S, 2500, 3840)
    assert not L.ggml_bitnet_can_mul_mat(ctypes.byref(odd), ctypes.byref(_tensor(GGML_TYPE_F32, 2500, 5)), ctypes.byref(d))
    ws = L.ggml_bitnet_mul_mat_get_wsize(ctypes.byref(w), ctypes.byref(x), ctypes.byref(d))
    assert ws % 64 == 0 and ws >= 2560 * 5 + 5 * 8
    L.ggml_bitnet_set_n_threads(8)
    # a tensor of an unsupported type, or one that already has an extra, is left alone
    L.ggml_bitnet_transform_tensor(ctypes.byref(bad))
    assert not bad.extra
    w.extra = 1234
    L.ggml_bitnet_transform_tensor(ctypes.byref(w))
    assert w.extra == 1234
    L.ggml_bitnet_free()
    L.ggml_bitnet_free()                                   # idempotent


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,m", [(256, 2560, 1), (100 * 16, 640, 5), (2560, 6912, 33)])
def test_transform_and_mul_mat_match_oracle(L, port_lib, rows, k, m):
    q, ws = O.synth_weights(rows, k, seed=rows + k)
    x = O.synth_acts(m, k, seed=m + k).astype(np.float32)
    buf = port_lib.quantize_i2_s(q.astype(np.float32) * ws)        # I2_S tensor data as a GGUF holds it
    y, a, ysum = O.act_quant(x)
    want = O.rescale(O.matmul_i32(y, q), a, [ws])                   # f32, not rounded to bf16

    L.ggml_bitnet_init()
    w_t = _tensor(GGML_TYPE_I2_S, k, rows, buf)
    L.ggml_bitnet_transform_tensor(ctypes.byref(w_t))
    assert L.bitnet_last_status() == 0 and w_t.extra
    extra = ctypes.cast(w_t.extra, ctypes.POINTER(Extra)).contents
    assert extra.BK == 128 and extra.n_tile_num == (rows + 15) // 16 and extra.scales[0] == np.float32(ws)
    x_t, out = _tensor(GGML_TYPE_F32, k, m, x), np.zeros((m, rows), dtype=np.float32)
    d_t = _tensor(GGML_TYPE_F32, rows, m, out)
    d_t.src[0], d_t.src[1] = ctypes.pointer(w_t), ctypes.pointer(x_t)
    wsize = L.ggml_bitnet_mul_mat_get_wsize(ctypes.byref(w_t), ctypes.byref(x_t), ctypes.byref(d_t))
    work = np.zeros(wsize, dtype=np.uint8)
    for ith in (1, 0):                                              # other threads do nothing, thread 0 computes
        p = Params(ith, 2, wsize, work.ctypes.data)
        L.ggml_bitnet_mul_mat(ctypes.byref(p), ctypes.byref(d_t))
        assert L.bitnet_last_status() == 0
        assert (out != 0).any() == (ith == 0)
    assert np.array_equal(work[: m * k].view(np.int8).reshape(m, k), y)          # qlut
    assert np.array_equal(work[m * k: m * k + 4 * m].view(np.float32), a)        # lut_scales
    assert np.array_equal(out, want)
    L.ggml_bitnet_free()


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,three_k,two_k", [(3200, 8640, 8640, 0), (3200, 3200, 3168, 32), (8640, 3200, 3168, 32)])
@pytest.mark.parametrize("bs", [1, 8])
def test_tl2_signature_entry_points_match_oracle(L, port_lib, m, k, three_k, two_k, bs):
    """ggml_preprocessor + the pair of ggml_qgemm_lut calls (include/ggml-bitnet.h:46-47) on the
    3B preset's shapes (include/bitnet-lut-kernels.h:1003-1124): C = (sum w*q) / LUT_Scales * Scales,
    the rescale of :993-999, equal to the oracle's f32 result."""
    q, ws = O.synth_weights(m, k, seed=m + k)
    x = O.synth_acts(bs, k, seed=bs + k).astype(np.float32)
    y, a, ysum = O.act_quant(x)
    want = O.rescale(O.matmul_i32(y, q), a, [ws])
    buf = port_lib.quantize_i2_s(q.astype(np.float32) * ws)

    L.ggml_bitnet_init()
    w_t = _tensor(GGML_TYPE_I2_S, k, m, buf)
    L.ggml_bitnet_transform_tensor(ctypes.byref(w_t))
    assert L.bitnet_last_status() == 0 and w_t.extra
    extra = ctypes.cast(w_t.extra, ctypes.POINTER(Extra)).contents
    lut_scales = np.zeros(bs, dtype=np.float32)
    three = np.zeros(bs * three_k // 3 * 32, dtype=np.int8)
    two = np.zeros(max(bs * two_k // 2 * 32, 1), dtype=np.int8)
    vp = lambda arr: arr.ctypes.data_as(ctypes.c_void_p)
    L.ggml_preprocessor(bs, m, three_k, two_k, vp(x), vp(lut_scales), vp(three), vp(two))
    assert L.bitnet_last_status() == 0
    assert np.array_equal(lut_scales, a)
    assert np.array_equal(three.reshape(bs, -1)[:, :three_k], y[:, :three_k])
    if two_k:
        assert np.array_equal(two.reshape(bs, -1)[:, :two_k], y[:, three_k:])
    c = np.zeros((bs, m), dtype=np.float32)
    scales = np.array([ws], dtype=np.float32)
    qw = ctypes.c_void_p(extra.qweights)
    L.ggml_qgemm_lut(bs, m, k, three_k, qw, None, vp(three), vp(scales), vp(lut_scales), vp(c))
    assert L.bitnet_last_status() == 0
    L.ggml_qgemm_lut(bs, m, k, two_k, qw, None, vp(two), vp(scales), vp(lut_scales), vp(c))
    assert L.bitnet_last_status() == 0
    assert np.array_equal(c, want)
    # a pointer that no transform produced is refused
    L.ggml_qgemm_lut(bs, m, k, three_k, vp(three), None, vp(three), vp(scales), vp(lut_scales), vp(c))
    assert L.bitnet_last_status() == 1
    L.ggml_bitnet_free()
