"""Python entry points of the W2A8 BitLinear path (thin wrappers over the C ABI)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib


def bitnet_int8xint2_linear(input0: torch.Tensor, input1: torch.Tensor, s: torch.Tensor, ws: torch.Tensor,
                            ret: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same call as the reference's gpu/model.py:21-37 (and gpu/test.py:15-29 when `ret` is
    given): int8 activations [.., K] x packed weights [N, K/4] -> bf16 [.., N] through the
    `bitlinear_int8xint2` symbol, on the current stream."""
    out_shape = list(input0.shape)
    out_shape[-1] = input1.shape[0]
    m = input0.shape[0]
    if len(out_shape) == 3:
        m *= input0.shape[1]
    n = input1.shape[0]
    k = input1.shape[1] * 4
    if ret is None:
        ret = torch.empty(*out_shape, dtype=torch.bfloat16, device=input0.device)
    _lib.lib.bitlinear_int8xint2(_lib.ptr(input0), _lib.ptr(input1), _lib.ptr(ret), _lib.ptr(s), _lib.ptr(ws),
                                 m, n, k, _lib.stream_ptr())
    _lib.check()
    return ret


def quant_input(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 1e-5, pad_to: int = 128):
    """(Optional RMSNorm, then) per-token absmax int8 quantisation of bf16 x [.., K]
    (BitLinearKernel.quant_input, gpu/model.py:68-71).  Returns (y int8 [M, K_pad],
    act_scale f32 [M], ysum int32 [M]); K_pad = K rounded up to `pad_to`, zero filled."""
    assert x.dtype == torch.bfloat16 and x.is_cuda
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    m = x2.shape[0]
    k_pad = (k + pad_to - 1) // pad_to * pad_to
    y = torch.empty((m, k_pad), dtype=torch.int8, device=x.device)
    a = torch.empty((m,), dtype=torch.float32, device=x.device)
    ysum = torch.empty((m,), dtype=torch.int32, device=x.device)
    _lib.check(_lib.lib.bitnet_quant_input(_lib.ptr(x2), x2.stride(0), _lib.ptr(gamma), eps, _lib.ptr(y), k_pad,
                                           _lib.ptr(a), None, _lib.ptr(ysum), m, k, _lib.stream_ptr()))
    return y, a, ysum


def quant_input_glu(x13: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 1e-5, pad_to: int = 128):
    """quant_input of squared_relu(x1) * x3 for bf16 x13 = [x1 | x3] of shape [.., 2K]
    (gpu/model.py:193-196) without materialising the product."""
    assert x13.dtype == torch.bfloat16 and x13.is_cuda and x13.shape[-1] % 2 == 0
    k = x13.shape[-1] // 2
    x2 = x13.reshape(-1, 2 * k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    m = x2.shape[0]
    k_pad = (k + pad_to - 1) // pad_to * pad_to
    y = torch.empty((m, k_pad), dtype=torch.int8, device=x13.device)
    a = torch.empty((m,), dtype=torch.float32, device=x13.device)
    ysum = torch.empty((m,), dtype=torch.int32, device=x13.device)
    _lib.check(_lib.lib.bitnet_quant_input_glu(_lib.ptr(x2), x2.stride(0), _lib.ptr(gamma), eps, _lib.ptr(y), k_pad,
                                               _lib.ptr(a), None, _lib.ptr(ysum), m, k, _lib.stream_ptr()))
    return y, a, ysum


def linear_w2a8(y: torch.Tensor, act_scale: torch.Tensor, ysum: Optional[torch.Tensor], weight: torch.Tensor,
                w_scale: torch.Tensor, seg_end: Sequence[int], n: int, k: int,
                want_acc: bool = False, want_out: bool = True):
    """int8 y [M, ldy] x packed weight -> bf16 [M, N] (and/or the exact int32 sums)."""
    m = y.shape[0]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=y.device) if want_out else None
    acc = torch.empty((m, n), dtype=torch.int32, device=y.device) if want_acc else None
    seg = (ctypes.c_int * len(seg_end))(*seg_end)
    _lib.check(_lib.lib.bitnet_linear_w2a8(_lib.ptr(y), y.stride(0), _lib.ptr(weight), _lib.ptr(out), n, _lib.ptr(acc),
                                           _lib.ptr(act_scale), _lib.ptr(ysum), _lib.ptr(w_scale), seg, len(seg_end),
                                           m, n, k, _lib.stream_ptr()))
    if want_acc and want_out:
        return out, acc
    return acc if want_acc else out


def linear_w2a8_add_quant(y: torch.Tensor, act_scale: torch.Tensor, ysum: torch.Tensor, weight: torch.Tensor,
                          w_scale: float, n: int, k: int, h: torch.Tensor, gamma: Optional[torch.Tensor],
                          eps: float = 1e-5, pad_to: int = 128):
    """h += BitLinear(y) in place (h bf16 [M, N], contiguous), then - with gamma - RMSNorm and
    quant_input of the new h: returns (y_next int8 [M, N_pad], act_scale f32 [M], ysum int32 [M]),
    or None without gamma.  The fused form of `h = h + linear(...)` followed by the next
    BitLinear's quant_input, for 16 tokens or more (bitnet_linear_w2a8_add_quant)."""
    m = y.shape[0]
    assert h.dtype == torch.bfloat16 and h.dim() == 2 and h.shape == (m, n) and h.stride(1) == 1
    if gamma is None:
        _lib.check(_lib.lib.bitnet_linear_w2a8_add_quant(_lib.ptr(y), y.stride(0), _lib.ptr(weight), _lib.ptr(act_scale),
                                                         _lib.ptr(ysum), float(w_scale), m, n, k, _lib.ptr(h), h.stride(0),
                                                         None, 0.0, None, 0, None, None, _lib.stream_ptr()))
        return None
    n_pad = (n + pad_to - 1) // pad_to * pad_to
    y2 = torch.empty((m, n_pad), dtype=torch.int8, device=y.device)
    a2 = torch.empty((m,), dtype=torch.float32, device=y.device)
    s2 = torch.empty((m,), dtype=torch.int32, device=y.device)
    _lib.check(_lib.lib.bitnet_linear_w2a8_add_quant(_lib.ptr(y), y.stride(0), _lib.ptr(weight), _lib.ptr(act_scale),
                                                     _lib.ptr(ysum), float(w_scale), m, n, k, _lib.ptr(h), h.stride(0),
                                                     _lib.ptr(gamma), eps, _lib.ptr(y2), n_pad, _lib.ptr(a2), _lib.ptr(s2),
                                                     _lib.stream_ptr()))
    return y2, a2, s2


def attention_decode(xqkv: torch.Tensor, pos: torch.Tensor, rope: torch.Tensor, cache_k: torch.Tensor,
                     cache_v: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """One new token per sequence: RoPE, append to the KV cache, attention over the cache.
    xqkv bf16 [B, (H + 2 Hkv) D]; pos int64 [B]; rope f32 [L', D/2, 2]; caches bf16
    [B, L, Hkv, D] (updated in place).  Returns bf16 [B, H D]."""
    assert xqkv.dtype == torch.bfloat16 and xqkv.dim() == 2 and xqkv.stride(1) == 1
    assert cache_k.is_contiguous() and cache_v.is_contiguous() and rope.is_contiguous()
    b, length = cache_k.shape[0], cache_k.shape[1]
    assert rope.shape[0] >= length and pos.dtype == torch.int64
    out = torch.empty((b, n_heads * head_dim), dtype=torch.bfloat16, device=xqkv.device)
    _lib.check(_lib.lib.bitnet_attention_decode(_lib.ptr(xqkv), xqkv.stride(0), _lib.ptr(pos), _lib.ptr(rope),
                                                _lib.ptr(cache_k), _lib.ptr(cache_v), _lib.ptr(out), b, n_heads,
                                                n_kv_heads, head_dim, length, _lib.stream_ptr()))
    return out


def sample_top_p(logits: torch.Tensor, temperature: float, top_p: float, seed: int = 0,
                 pos: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of f32 logits [B, V] with temperature and top-p, on the device (the
    sampling branch of gpu/generate.py:250-257, gpu/sample_utils.py:8-30).  `uniforms` f32 [B] are
    the random numbers to use; without them row b draws from a hash of (seed, b, pos[b]).  The ids
    go to `out` (int64 [B], created if absent) and, if given, to `tokens` as well."""
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    b, v = logits.shape
    if out is None:
        out = torch.empty((b,), dtype=torch.int64, device=logits.device)
    assert uniforms is None or (uniforms.dtype == torch.float32 and uniforms.numel() == b)
    assert pos is None or (pos.dtype == torch.int64 and pos.numel() == b)
    _lib.check(_lib.lib.bitnet_sample_top_p(_lib.ptr(logits), logits.stride(0), b, v, float(temperature), float(top_p),
                                            int(seed) & 0xFFFFFFFFFFFFFFFF, _lib.ptr(pos), _lib.ptr(uniforms),
                                            _lib.ptr(out), _lib.ptr(tokens), _lib.stream_ptr()))
    return out
