"""NumPy restatement of the reference's W2A8 BitLinear data formats and arithmetic.

Test infrastructure only: it is the checker that the CUDA path is compared with (tests,
the smoke check, the CPU leg of the benchmark) and must never sit on the product path.

Parity status: the integer parts (ternarise, I2_S bytes, the GPU int2 layout, int32
matrix products) are pinned by golden vectors produced from the reference's own code
(``tests/golden/make_golden.py``).  The float epilogue of the CPU path is in the
reference's un-vendored llama.cpp fork and is tested nowhere in the reference: parity
unpinned for it; it follows the in-repo statements of the formula cited below.

Paths cited are relative to the microsoft/BitNet checkout.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# ----------------------------------------------------------------------------------------
# ternarisation and activation quantisation
# ----------------------------------------------------------------------------------------


def ternarize(w: np.ndarray):
    """absmean ternarisation, gpu/convert_checkpoint.py:23-27 and
    utils/convert-hf-to-gguf-bitnet.py:1055-1060: s = 1/max(mean|w|, 1e-5);
    q = clamp(round_half_even(w*s), -1, 1); the dequantisation scale is 1/s."""
    w = np.asarray(w, dtype=np.float32)
    s = np.float32(1.0) / np.maximum(np.abs(w).mean(dtype=np.float32), np.float32(1e-5))
    q = np.clip(np.rint(w * s), -1, 1).astype(np.int8)
    return q, np.float32(1.0) / s


def act_quant(x: np.ndarray):
    """Per-token absmax int8 quantisation, gpu/model.py:68-71 evaluated in f32:
    a = 127/max(absmax, 1e-5); y = clamp(round_half_even(x*a), -128, 127).
    Returns (y int8 [M,K], a f32 [M], ysum int32 [M])."""
    x = np.asarray(x, dtype=np.float32)
    mx = np.maximum(np.abs(x).max(axis=-1), np.float32(1e-5)).astype(np.float32)
    a = (np.float32(127.0) / mx).astype(np.float32)
    y = np.clip(np.rint(x * a[:, None]), -128, 127).astype(np.int8)
    return y, a, y.astype(np.int32).sum(axis=-1, dtype=np.int32)


def rmsnorm(x: np.ndarray, g: np.ndarray, eps: float = 1e-5):
    """RMSNorm as the reference's decode model applies it before each BitLinear
    (gpu/model.py:159-160,195-196,237-242): (x * g) * rsqrt(mean(x^2) + eps) in f32.  The
    sum of squares is taken in f64 (so that it does not depend on the order of addition) and
    rounded to f32 once; the mean, the root and the reciprocal are IEEE f32 operations."""
    x = np.asarray(x, dtype=np.float32)
    ss = (x.astype(np.float64) ** 2).sum(axis=-1, keepdims=True).astype(np.float32)
    v = (ss / np.float32(x.shape[-1])).astype(np.float32) + np.float32(eps)
    r = (np.float32(1.0) / np.sqrt(v.astype(np.float32))).astype(np.float32)
    return (x * g.astype(np.float32) * r).astype(np.float32)


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Rounds f32 to bf16 (round to nearest even) and returns the value as f32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(x.shape)


def matmul_i32(y: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Exact int32 y[M,K] @ w[N,K]^T (what gpu/test.py:46-50 computes with NumPy).  Evaluated
    in f64 through BLAS: every partial sum is an integer far below 2^53, so the result is
    exact, and large cases finish in seconds."""
    return (y.astype(np.float64) @ w.astype(np.float64).T).astype(np.int64).astype(np.int32)


def rescale(acc: np.ndarray, a: np.ndarray, w_scale, seg_end=None) -> np.ndarray:
    """f32 out = acc / a * w_scale[segment(row)], gpu/bitnet_kernels/bitnet_kernels.h:80-82
    and include/bitnet-lut-kernels.h:993-999.  `acc` already has the offset removed
    (acc = sum (code-1)*y).  seg_end[i] = first output row after segment i."""
    acc = np.asarray(acc)
    n = acc.shape[-1]
    w_scale = np.atleast_1d(np.asarray(w_scale, dtype=np.float32))
    if seg_end is None:
        seg_end = [n]
    col_scale = np.empty(n, dtype=np.float32)
    lo = 0
    for i, hi in enumerate(seg_end):
        col_scale[lo:hi] = w_scale[i]
        lo = hi
    return (acc.astype(np.float32) / np.asarray(a, dtype=np.float32)[:, None]) * col_scale[None, :]


def ref_gpu_scale_segments(n: int, k: int):
    """Row segments the reference GPU kernel's shape ladder implies:
    ws[row // (N / ws_num)] with ws_num fixed per (N, K)
    (gpu/bitnet_kernels/bitnet_kernels.cu:4-33, bitnet_kernels.h:80-82)."""
    ws_num = {(3840, 2560): 3, (13824, 2560): 2, (4800, 3200): 6, (20480, 3200): 2}.get((n, k), 1)
    step = n // ws_num
    return [step * (i + 1) for i in range(ws_num)]


# ----------------------------------------------------------------------------------------
# I2_S (CPU / GGUF) byte format
# ----------------------------------------------------------------------------------------


def i2s_pack(q: np.ndarray, scale: float) -> np.ndarray:
    """Ternary int8 [N,K] -> I2_S bytes (x86 ACT_PARALLEL form), src/ggml-bitnet-mad.cpp:80-96
    and utils/convert-hf-to-gguf-bitnet.py:700-725: code = q+1; every 128 consecutive
    elements of the flattened matrix give 32 bytes, byte p = c[p]<<6 | c[p+32]<<4 |
    c[p+64]<<2 | c[p+96]; one f32 scale at byte n/4; total n/4 + 32 bytes."""
    q = np.asarray(q)
    n = q.size
    assert n % 128 == 0
    c = (q.reshape(-1).astype(np.int16) + 1).astype(np.uint8).reshape(n // 128, 4, 32)
    packed = (c[:, 0] << 6) | (c[:, 1] << 4) | (c[:, 2] << 2) | c[:, 3]
    out = np.zeros(n // 4 + 32, dtype=np.uint8)
    out[: n // 4] = packed.reshape(-1)
    out[n // 4 : n // 4 + 4] = np.frombuffer(np.float32(scale).tobytes(), dtype=np.uint8)
    return out


def i2s_codes(buf: np.ndarray, n_rows: int, k: int) -> np.ndarray:
    """I2_S bytes -> codes uint8 [N,K] in {0,1,2,3} (inverse of i2s_pack)."""
    n = n_rows * k
    b = np.asarray(buf[: n // 4], dtype=np.uint8).reshape(n // 128, 32)
    c = np.stack([(b >> 6) & 3, (b >> 4) & 3, (b >> 2) & 3, b & 3], axis=1)
    return c.reshape(n_rows, k)


def i2s_scale(buf: np.ndarray, n_rows: int, k: int) -> np.float32:
    off = n_rows * k // 4
    return np.frombuffer(np.asarray(buf[off : off + 4], dtype=np.uint8).tobytes(), dtype=np.float32)[0]


# ----------------------------------------------------------------------------------------
# the reference's GPU int2 layout (gpu/pack_weight.py)
# ----------------------------------------------------------------------------------------


def _ref_gpu_tile_map():
    """(ii, jj) of the stored 16x32 tile -> (row, col) of the source tile,
    gpu/pack_weight.py:5-14."""
    rows = np.zeros((16, 32), dtype=np.int64)
    cols = np.zeros((16, 32), dtype=np.int64)
    for ii in range(16):
        for jj in range(32):
            t = ii * 2 + jj // 16
            rows[ii, jj] = (t // 16) * 8 + (t % 8)
            cols[ii, jj] = (jj % 16) + 16 * ((t % 16) // 8)
    return rows, cols


def ref_gpu_pack(q: np.ndarray) -> np.ndarray:
    """Ternary int8 [N,K] -> the reference's GPU int2 bytes, int8 [N, K/4]
    (gpu/pack_weight.py:76-98): code = q+2; 16x32 tiles permuted by the map above; four
    codes per byte, lowest bits first (:46-53); then the 16 codes of every int32 are
    re-ordered so that byte b holds elements b, b+4, b+8, b+12 (:56-72)."""
    q = np.asarray(q, dtype=np.int8)
    n, k = q.shape
    assert n % 16 == 0 and k % 32 == 0
    rows, cols = _ref_gpu_tile_map()
    t = (q.astype(np.int16) + 2).astype(np.uint32).reshape(n // 16, 16, k // 32, 32).transpose(0, 2, 1, 3)
    perm = t[:, :, rows, cols]                              # [N/16, K/32, 16, 32]
    e = perm.reshape(n // 16, k // 32, 16, 2, 16)            # 16 codes per int32
    word = np.zeros(e.shape[:-1], dtype=np.uint32)
    for idx in range(16):
        shift = (idx % 4) * 8 + (idx // 4) * 2
        word |= e[..., idx] << np.uint32(shift)
    return word.reshape(-1).view(np.int8).reshape(n, k // 4)


def ref_gpu_unpack(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """Inverse of ref_gpu_pack -> ternary int8 [N,K]."""
    rows, cols = _ref_gpu_tile_map()
    word = np.ascontiguousarray(packed).reshape(-1).view(np.uint32).reshape(n // 16, k // 32, 16, 2)
    e = np.zeros(word.shape + (16,), dtype=np.int16)
    for idx in range(16):
        shift = (idx % 4) * 8 + (idx // 4) * 2
        e[..., idx] = (word >> np.uint32(shift)) & 3
    perm = e.reshape(n // 16, k // 32, 16, 32)
    src = np.zeros_like(perm)
    src[:, :, rows, cols] = perm
    return (src.transpose(0, 2, 1, 3).reshape(n, k) - 2).astype(np.int8)


# ----------------------------------------------------------------------------------------
# the re-tiled device layout of this library ("W2T": 16 rows x 128 columns per 512-byte tile)
# ----------------------------------------------------------------------------------------


def w2t_shape(n: int, k: int):
    return (n + 15) // 16 * 16, (k + 127) // 128 * 128


def _w2t_index(n_pad: int, k_pad: int):
    """For every (row, col) of the padded matrix: the 32-bit word index and the bit shift
    of its 2-bit field.  Tile (tn, tk) is 128 words; lane = g*4+q owns words 4*lane..+3;
    word r, byte b, field j hold row 16*tn + g + 8*(r&1), col 128*tk + 32q + 8j + 4*(r>>1) + b."""
    row = np.arange(n_pad)[:, None]
    col = np.arange(k_pad)[None, :]
    tn, rr = row // 16, row % 16
    tk, kk = col // 128, col % 128
    g, rlo = rr % 8, rr // 8
    q, rem = kk // 32, kk % 32
    j, rem2 = rem // 8, rem % 8
    h, b = rem2 // 4, rem2 % 4
    r = rlo + 2 * h
    word = (tn * (k_pad // 128) + tk) * 128 + (g * 4 + q) * 4 + r
    shift = 8 * b + 2 * j
    return word, shift


def w2t_pack(q: np.ndarray) -> np.ndarray:
    """Ternary int8 [N,K] -> W2T bytes uint8 [N_pad*K_pad/4]; code = q+1, padding = code 1."""
    q = np.asarray(q, dtype=np.int8)
    n, k = q.shape
    n_pad, k_pad = w2t_shape(n, k)
    c = np.ones((n_pad, k_pad), dtype=np.uint32)
    c[:n, :k] = (q.astype(np.int16) + 1).astype(np.uint32)
    word, shift = _w2t_index(n_pad, k_pad)
    out = np.zeros(n_pad * k_pad // 16, dtype=np.uint32)
    word = np.broadcast_to(word, c.shape).reshape(-1)
    shift = np.broadcast_to(shift, c.shape).astype(np.uint32)
    np.bitwise_or.at(out, word, (c << shift).reshape(-1))
    return out.view(np.uint8)


def w2t_codes(buf: np.ndarray, n: int, k: int) -> np.ndarray:
    """W2T bytes -> codes uint8 [N,K] (padding dropped)."""
    n_pad, k_pad = w2t_shape(n, k)
    words = np.ascontiguousarray(buf).view(np.uint32)
    word, shift = _w2t_index(n_pad, k_pad)
    word = np.broadcast_to(word, (n_pad, k_pad))
    shift = np.broadcast_to(shift, (n_pad, k_pad)).astype(np.uint32)
    return ((words[word] >> shift) & 3).astype(np.uint8)[:n, :k]


# ----------------------------------------------------------------------------------------
# ctypes access to the two compiled checkers
# ----------------------------------------------------------------------------------------


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class PortLib:
    """oracle/liboracle_port.so (built from i2s_port.c)."""

    def __init__(self, path=None):
        self.lib = ctypes.CDLL(path or os.path.join(HERE, "liboracle_port.so"))
        L = self.lib
        L.port_quantize_i2_s.restype = ctypes.c_size_t
        L.port_quantize_i2_s.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.port_vec_dot_i2_i8.restype = ctypes.c_int32
        L.port_vec_dot_i2_i8.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.port_i2s_gemm.restype = None
        L.port_i2s_gemm.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
        L.port_i2s_gemm_time.restype = ctypes.c_double
        L.port_i2s_gemm_time.argtypes = L.port_i2s_gemm.argtypes + [ctypes.c_int]
        L.port_act_quant.restype = None
        L.port_act_quant.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64]
        L.port_unpack_i2_s.restype = None
        L.port_unpack_i2_s.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.port_rescale.restype = None
        L.port_rescale.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.port_max_threads.restype = ctypes.c_int

    def quantize_i2_s(self, w: np.ndarray) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        out = np.zeros(n * k // 4 + 32, dtype=np.uint8)
        sz = self.lib.port_quantize_i2_s(_ptr(w), _ptr(out), n, k)
        assert sz == out.size
        return out

    def gemm(self, x_i2s: np.ndarray, y: np.ndarray, n: int, k: int, threads=0) -> np.ndarray:
        y = np.ascontiguousarray(y, dtype=np.int8)
        m = y.shape[0]
        acc = np.zeros((m, n), dtype=np.int32)
        self.lib.port_i2s_gemm(k, _ptr(acc), n, _ptr(x_i2s), _ptr(y), m, n, threads)
        return acc

    def gemm_time(self, x_i2s, y, n, k, threads, iters) -> float:
        y = np.ascontiguousarray(y, dtype=np.int8)
        m = y.shape[0]
        acc = np.zeros((m, n), dtype=np.int32)
        return self.lib.port_i2s_gemm_time(k, _ptr(acc), n, _ptr(x_i2s), _ptr(y), m, n, threads, iters)

    def act_quant(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m, k = x.shape
        y = np.zeros((m, k), dtype=np.int8)
        a = np.zeros(m, dtype=np.float32)
        ys = np.zeros(m, dtype=np.int32)
        self.lib.port_act_quant(_ptr(x), _ptr(y), _ptr(a), _ptr(ys), m, k)
        return y, a, ys

    def max_threads(self) -> int:
        return self.lib.port_max_threads()


class RefLib:
    """oracle/_ref/libref_i2s.so: the reference's src/ggml-bitnet-mad.cpp compiled in place."""

    PATH = os.path.join(HERE, "_ref", "libref_i2s.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self, path=None):
        self.lib = ctypes.CDLL(path or self.PATH)
        L = self.lib
        L.quantize_i2_s.restype = ctypes.c_size_t
        L.quantize_i2_s.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
        L.ggml_vec_dot_i2_i8_s.restype = None
        L.ggml_vec_dot_i2_i8_s.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                           ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        L.ref_i2s_gemm.restype = None
        L.ref_i2s_gemm.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                   ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.ref_i2s_gemm_time.restype = ctypes.c_double
        L.ref_i2s_gemm_time.argtypes = L.ref_i2s_gemm.argtypes + [ctypes.c_int]
        L.ref_max_threads.restype = ctypes.c_int

    def quantize_i2_s(self, w: np.ndarray) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        out = np.zeros(n * k // 4 + 32, dtype=np.uint8)
        sz = self.lib.quantize_i2_s(_ptr(w), _ptr(out), n, k, None)
        assert sz == out.size
        return out

    def vec_dot(self, x_row: np.ndarray, y: np.ndarray, k: int) -> np.ndarray:
        """One weight row against nrc activation rows (nrc = y.shape[0])."""
        y = np.ascontiguousarray(y, dtype=np.int8)
        nrc = y.shape[0]
        s = np.zeros(nrc, dtype=np.float32)
        self.lib.ggml_vec_dot_i2_i8_s(k, _ptr(s), 1, _ptr(x_row), k, _ptr(y), k, nrc)
        return s

    def gemm(self, x_i2s: np.ndarray, y: np.ndarray, n: int, k: int, threads=0) -> np.ndarray:
        """Returns the float code sums [M,N] exactly as the reference kernel stores them."""
        y = np.ascontiguousarray(y, dtype=np.int8)
        m = y.shape[0]
        out = np.zeros((m, n), dtype=np.float32)
        self.lib.ref_i2s_gemm(k, _ptr(out), n, _ptr(x_i2s), _ptr(y), m, n, threads)
        return out

    def gemm_time(self, x_i2s, y, n, k, threads, iters) -> float:
        y = np.ascontiguousarray(y, dtype=np.int8)
        m = y.shape[0]
        out = np.zeros((m, n), dtype=np.float32)
        return self.lib.ref_i2s_gemm_time(k, _ptr(out), n, _ptr(x_i2s), _ptr(y), m, n, threads, iters)

    def max_threads(self) -> int:
        return self.lib.ref_max_threads()


# ----------------------------------------------------------------------------------------
# sampling of the next token (temperature + top-p)
# ----------------------------------------------------------------------------------------


def top_p_weights(logits: np.ndarray, temperature: float, top_p: float):
    """The nucleus of gpu/sample_utils.py:8-30 applied to softmax(logits / temperature)
    (gpu/generate.py:250-257), in exact (f64) arithmetic over f32 exponentials: sort descending
    (ties in index order), drop every entry whose exclusive cumulative mass exceeds top_p times
    the total.  Returns (e f32 [V] unnormalised probabilities, kept bool [V], margin f64 [V]):
    margin is the distance of each entry's exclusive cumulative share from top_p, so that a
    checker can excuse entries that sit on the cut within rounding."""
    lg = np.asarray(logits, dtype=np.float32)
    e = np.exp((lg - lg.max()) * np.float32(1.0 / temperature)).astype(np.float32)
    order = np.argsort(-e, kind="stable")
    es = e[order].astype(np.float64)
    total = es.sum()
    excl = np.cumsum(es) - es
    kept = np.zeros(e.shape, dtype=bool)
    kept[order] = excl <= top_p * total
    margin = np.empty(e.shape, dtype=np.float64)
    margin[order] = np.abs(excl / total - top_p)
    return e, kept, margin


def top_p_draw(e: np.ndarray, kept: np.ndarray, u: float) -> int:
    """The kept entry, in index order, at which the running kept mass first exceeds u times the
    kept mass: a draw from the renormalised nucleus (what torch.multinomial does to the sorted,
    masked probabilities in gpu/sample_utils.py:27-29, with the entries taken in another order)."""
    m = np.where(kept, e.astype(np.float64), 0.0)
    cum = np.cumsum(m)
    return int(np.searchsorted(cum, u * cum[-1], side="right"))


def top_p_interval(e: np.ndarray, kept: np.ndarray, token: int):
    """[lo, hi): the values of u for which top_p_draw returns `token` (empty if it is not kept)."""
    m = np.where(kept, e.astype(np.float64), 0.0)
    cum = np.cumsum(m)
    return (cum[token] - m[token]) / cum[-1], cum[token] / cum[-1]


def counter_uniform(seed: int, row: int, pos: int) -> np.float32:
    """The library's counter-based random number for (seed, sequence, position): a splitmix64
    finaliser (Steele, Lea, Flood 2014) over the three, top 24 bits as a fraction."""
    mask = (1 << 64) - 1
    x = (seed + 0x9E3779B97F4A7C15 * (row + 1)) & mask
    x ^= (pos * 0xD1B54A32D192ED03) & mask
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & mask
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & mask
    x ^= x >> 31
    return np.float32((x >> 40) / 16777216.0)


# ----------------------------------------------------------------------------------------
# seeded synthetic inputs with the shapes and value distributions of the kernel sweep
# ----------------------------------------------------------------------------------------


def synth_weights(n: int, k: int, seed: int):
    """N(0,1) weights, absmean-ternarised; returns (q int8 [N,K], bf16-rounded scale)."""
    rng = np.random.default_rng(seed)
    q, s = ternarize(rng.standard_normal((n, k), dtype=np.float32))
    return q, to_bf16(np.array([s], dtype=np.float32))[0]


def synth_acts(m: int, k: int, seed: int) -> np.ndarray:
    """bf16-valued N(0,1) activations with 1% of the entries multiplied by 20."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    x = np.where(rng.random((m, k)) < 0.01, x * 20.0, x).astype(np.float32)
    return to_bf16(x)
