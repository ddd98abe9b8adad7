"""Checkpoint ingestion for the B200 BitLinear kernels.

Counterpart of the reference's two converters:

* gpu/convert_safetensors.py:43-93 (`convert_back`): Hugging Face tensor names -> the fused
  layout of gpu/model.py (wqkv = [q; k; v] with the rotary row permutation, w13 = [gate; up]);
* gpu/convert_checkpoint.py:23-27,41-90 (`convert_ts_checkpoint`): per-sub-matrix absmean
  ternarisation, the bf16 `weight_scale[4]` of every BitLinear, and the packed weights.

Here the packed weights are in this library's W2T layout (pack_weight.convert_weight_int8_to_int2)
and the result can be loaded straight into `bitnet_b200.model.Transformer`.  Also read: the
reference's own `model_state_int2.pt` (its int2 bytes are re-tiled, nothing is re-quantised) and
the offline-quantised uint8 form of utils/convert-hf-to-gguf-bitnet.py:1097-1108 (four 2-bit
codes per byte along the row dimension plus a `weight_scale` tensor).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import pack_weight
from .config import ModelArgs


def quant_weight_int8(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """absmean ternarisation, gpu/convert_checkpoint.py:23-27: s = 1 / max(mean|W|, 1e-5);
    q = clamp(round(W s), -1, 1) as int8; scale = bf16(1 / s), shape [1]."""
    s = 1.0 / weight.float().abs().mean().clamp_(min=1e-5)
    q = (weight.float() * s).round().clamp(-1, 1).to(torch.int8)
    return q, (1.0 / s).to(torch.bfloat16).reshape(1)


def quant_weight_fp16(weight: torch.Tensor) -> torch.Tensor:
    """The dequantised ternary weight (gpu/convert_checkpoint.py:29-32), as the reference's
    bf16 prefill model holds it."""
    s = 1.0 / weight.float().abs().mean().clamp_(min=1e-5)
    return ((weight.float() * s).round().clamp(-1, 1) / s).to(weight.dtype)


def rope_rows_to_interleaved(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Rows of a q or k projection from the Hugging Face order (per head: first half, second
    half of the rotary pairs) to adjacent pairs, '(h l d) i -> (h d l) i' with l = 2
    (gpu/convert_safetensors.py:43-47).  The decode kernels rotate adjacent pairs."""
    n, k = w.shape
    d = n // n_heads // 2
    return w.view(n_heads, 2, d, k).transpose(1, 2).reshape(n, k)


def convert_hf_state_dict(st: Dict[str, torch.Tensor], args: ModelArgs) -> Dict[str, torch.Tensor]:
    """Hugging Face names -> the fused names of gpu/model.py (gpu/convert_safetensors.py:49-93):
    full-precision tensors, wqkv = [q (permuted); k (permuted); v], w13 = [gate; up], tied output."""
    out: Dict[str, torch.Tensor] = {}
    for layer in range(args.n_layers):
        base = f"model.layers.{layer}."
        wq = rope_rows_to_interleaved(st[f"{base}self_attn.q_proj.weight"], args.n_heads)
        wk = rope_rows_to_interleaved(st[f"{base}self_attn.k_proj.weight"], args.n_kv_heads)
        wv = st[f"{base}self_attn.v_proj.weight"]
        out[f"layers.{layer}.attention.wqkv.weight"] = torch.cat([wq, wk, wv], dim=0)
        out[f"layers.{layer}.attention.wo.weight"] = st[f"{base}self_attn.o_proj.weight"]
        out[f"layers.{layer}.attention_norm.weight"] = st[f"{base}input_layernorm.weight"]
        out[f"layers.{layer}.ffn_norm.weight"] = st[f"{base}post_attention_layernorm.weight"]
        out[f"layers.{layer}.attention.attn_sub_norm.weight"] = st[f"{base}self_attn.attn_sub_norm.weight"]
        out[f"layers.{layer}.feed_forward.ffn_sub_norm.weight"] = st[f"{base}mlp.ffn_sub_norm.weight"]
        out[f"layers.{layer}.feed_forward.w13.weight"] = torch.cat(
            [st[f"{base}mlp.gate_proj.weight"], st[f"{base}mlp.up_proj.weight"]], dim=0)
        out[f"layers.{layer}.feed_forward.w2.weight"] = st[f"{base}mlp.down_proj.weight"]
    out["tok_embeddings.weight"] = st["model.embed_tokens.weight"]
    out["output.weight"] = st.get("lm_head.weight", st["model.embed_tokens.weight"])
    out["norm.weight"] = st["model.norm.weight"]
    return out


def _split_points(key: str, args: ModelArgs):
    d = args.head_dim
    if "wqkv" in key:
        return [args.n_heads * d, args.n_kv_heads * d, args.n_kv_heads * d]
    if "w13" in key:
        return [args.ffn_dim, args.ffn_dim]
    return None


def convert_ts_checkpoint(state: Dict[str, torch.Tensor], args: ModelArgs, device="cuda",
                          want_fp16: bool = False):
    """Full-precision fused checkpoint -> the int2 state dict (gpu/convert_checkpoint.py:41-83):
    every BitLinear sub-matrix (q, k, v; gate, up; wo; w2) is ternarised on its own, the packed
    weight is stored under the same key and the scales under `<key>_scale` as bf16 [4] (unused
    entries zero).  Everything else is copied.  Returns (int2_state, fp16_state or None); the
    packed tensors are in the W2T layout and live on `device`."""
    int2: Dict[str, torch.Tensor] = {}
    fp16: Optional[Dict[str, torch.Tensor]] = {} if want_fp16 else None
    for key, value in state.items():
        is_lin = key.endswith("weight") and any(t in key for t in ("wqkv", "w13", ".w2.", ".wo."))
        if not is_lin:
            int2[key] = value.clone()
            if fp16 is not None:
                fp16[key] = value.clone()
            continue
        sizes = _split_points(key, args) or [value.shape[0]]
        assert sum(sizes) == value.shape[0], (key, sizes, tuple(value.shape))
        parts, scales, deq, lo = [], [], [], 0
        for n in sizes:
            sub = value[lo:lo + n].to(device)
            q, s = quant_weight_int8(sub)
            parts.append(q)
            scales.append(s)
            if fp16 is not None:
                deq.append(quant_weight_fp16(sub).cpu())
            lo += n
        ws = torch.zeros(4, dtype=torch.bfloat16, device=device)
        ws[: len(scales)] = torch.cat(scales)
        int2[key] = pack_weight.convert_weight_int8_to_int2(torch.cat(parts, dim=0))
        int2[key.replace("weight", "weight_scale")] = ws
        if fp16 is not None:
            fp16[key] = torch.cat(deq, dim=0)
    return int2, fp16


def convert_reference_int2_state(state: Dict[str, torch.Tensor], device="cuda") -> Dict[str, torch.Tensor]:
    """A `model_state_int2.pt` written by the reference (gpu/convert_checkpoint.py:85-90: int8
    [N, K/4] tensors in the layout of gpu/pack_weight.py) -> the same state with the packed
    tensors re-tiled to W2T.  Scales and everything else are kept."""
    out: Dict[str, torch.Tensor] = {}
    for key, value in state.items():
        if value.dtype == torch.int8 and value.dim() == 2 and key.endswith("weight"):
            out[key] = pack_weight.convert_ref_int2_to_w2t(value.to(device))
        else:
            out[key] = value.clone()
    return out


def unpack_offline_uint8(packed: torch.Tensor) -> torch.Tensor:
    """The offline-quantised form of the published checkpoints: uint8 [N/4, K], byte (r, k)
    holds rows r, r + N/4, r + 2N/4, r + 3N/4 of column k in bit pairs 0-1, 2-3, 4-5, 6-7 as
    code = weight + 1 (utils/convert-hf-to-gguf-bitnet.py:1097-1108).  Returns ternary int8 [N, K]."""
    assert packed.dtype == torch.uint8 and packed.dim() == 2
    shift = torch.tensor([0, 2, 4, 6], dtype=torch.uint8, device=packed.device).view(4, 1, 1)
    codes = (packed.unsqueeze(0) >> shift) & 3
    return (codes.to(torch.int8) - 1).reshape(packed.shape[0] * 4, packed.shape[1])


def load_int2_state(model, state: Dict[str, torch.Tensor]):
    """Loads an int2 state dict (convert_ts_checkpoint / convert_reference_int2_state) into a
    bitnet_b200.model.Transformer built with use_kernel=True."""
    from .model import BitLinearKernel

    dev = model.tok_embeddings.weight.device
    named = dict(model.named_modules())
    for key, value in state.items():
        if key.endswith("weight_scale"):
            continue
        mod_name, _, leaf = key.rpartition(".")
        mod = named.get(mod_name)
        if isinstance(mod, BitLinearKernel) and leaf == "weight":
            mod.weight.data = value.to(dev)
            ws = state[key.replace("weight", "weight_scale")].to(dev).to(torch.bfloat16)
            mod.weight_scale.data = ws
            mod.scale_f32 = ws[: len(mod.segments)].float().contiguous()
        elif mod is not None and hasattr(mod, leaf):
            getattr(mod, leaf).data = value.to(dev).to(getattr(mod, leaf).dtype)
    if model.args.tie_embeddings:
        model.output.weight = model.tok_embeddings.weight
    return model
