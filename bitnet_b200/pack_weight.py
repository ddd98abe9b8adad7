"""Weight packing for the B200 BitLinear kernels.

Host-side mirror of the reference's gpu/pack_weight.py: `convert_weight_int8_to_int2`
keeps its name, argument and result shape (int8 [N, K/4]) but produces this library's W2T
tile layout (16 rows x 128 columns per 512-byte tile, see csrc/common.cuh), which is what
`bitlinear_int8xint2` of this library reads.  Packing runs on the GPU.
"""
from __future__ import annotations

import torch

from . import _lib


def _padded(n: int, k: int):
    return (n + 15) // 16 * 16, (k + 127) // 128 * 128


def _alloc(n: int, k: int, device) -> torch.Tensor:
    n_pad, k_pad = _padded(n, k)
    assert _lib.lib.bitnet_w2t_bytes(n, k) == n_pad * k_pad // 4
    return torch.empty((n_pad, k_pad // 4), dtype=torch.int8, device=device)


def _cuda(t: torch.Tensor) -> torch.Tensor:
    if not torch.cuda.is_available():
        raise RuntimeError("bitnet_b200 packs weights on the GPU; no CUDA device is available")
    return t.contiguous() if t.is_cuda else t.contiguous().cuda()


def convert_weight_int8_to_int2(weight: torch.Tensor) -> torch.Tensor:
    """Ternary int8 [N,K] in {-1,0,+1} -> packed int8 [ceil16(N), ceil128(K)/4].

    Counterpart of gpu/pack_weight.py:76-98.  The result lives on the input's device."""
    assert weight.dtype == torch.int8 and weight.dim() == 2
    n, k = weight.shape
    w = _cuda(weight)
    out = _alloc(n, k, w.device)
    _lib.check(_lib.lib.bitnet_pack_ternary(_lib.ptr(w), _lib.ptr(out), n, k, _lib.stream_ptr()))
    return out if weight.is_cuda else out.cpu()


def convert_ref_int2_to_w2t(packed: torch.Tensor) -> torch.Tensor:
    """Weights packed by the reference's gpu/pack_weight.py (int8 [N,K/4], as stored in its
    model_state_int2.pt checkpoints, gpu/convert_checkpoint.py:85-90) -> this library's layout."""
    assert packed.dtype == torch.int8 and packed.dim() == 2
    n, k = packed.shape[0], packed.shape[1] * 4
    p = _cuda(packed)
    out = _alloc(n, k, p.device)
    _lib.check(_lib.lib.bitnet_pack_from_ref_int2(_lib.ptr(p), _lib.ptr(out), n, k, _lib.stream_ptr()))
    return out if packed.is_cuda else out.cpu()


def convert_i2s_to_w2t(i2s: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """I2_S bytes of a GGUF tensor (uint8, at least N*K/4 long) -> this library's layout."""
    assert i2s.dtype == torch.uint8
    b = _cuda(i2s)
    out = _alloc(n, k, b.device)
    _lib.check(_lib.lib.bitnet_pack_from_i2s(_lib.ptr(b), _lib.ptr(out), n, k, _lib.stream_ptr()))
    return out if i2s.is_cuda else out.cpu()


def unpack_int2_to_int8(packed: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """This library's packed weights -> ternary int8 [N,K]."""
    p = _cuda(packed)
    out = torch.empty((n, k), dtype=torch.int8, device=p.device)
    _lib.check(_lib.lib.bitnet_unpack_ternary(_lib.ptr(p), _lib.ptr(out), n, k, _lib.stream_ptr()))
    return out if packed.is_cuda else out.cpu()
