"""BitNet decoder built on the W2A8 BitLinear kernels.

Host-side mirror of the reference's gpu/model.py: the same module names (ModelArgs,
BitLinearKernel, BitLinear, Attention, FeedForward, TransformerBlock, Transformer,
make_cache) and the same arithmetic, with the xformers operators the reference imports
(RMSNorm, rope_padded, flash attention over a padded-keys bias; gpu/model.py:13-16)
replaced by plain PyTorch so that the module runs without xformers.  The BitLinear matmul
- the hot path - goes through libbitnet_b200.so; everything else is glue.

Differences from the reference that a caller sees:
* `forward(tokens, pos, cache)` takes token ids [B, T] and a device tensor `pos` [B] with
  the number of tokens already in the cache, instead of an xformers attention bias; with
  T == 1 the call has static shapes and can be captured in a CUDA graph.
* The RMSNorm in front of every BitLinear (attention_norm, attn_sub_norm, ffn_norm,
  ffn_sub_norm) is fused into the int8 quantisation kernel.
* Weight scales are applied per true row segment (q / k / v, gate / up), where the
  reference kernel splits the rows into equal parts (gpu/bitnet_kernels/bitnet_kernels.h:80-82).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn
from torch.nn import functional as F

from . import ops, pack_weight
from .config import PRESETS, ModelArgs, preset  # noqa: F401  (re-exported)


LayerCache = Tuple[torch.Tensor, torch.Tensor]


class RMSNorm(nn.Module):
    """(x * weight) * rsqrt(mean(x^2) + eps), computed in f32, returned in x's dtype (the
    operation order of the library's fused prologue)."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.bfloat16), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * self.weight.float() * r).to(x.dtype)


def quant_weight_int8(weight: torch.Tensor):
    """absmean ternarisation, gpu/convert_checkpoint.py:23-27."""
    s = 1.0 / weight.abs().mean().clamp_(min=1e-5)
    q = (weight * s).round().clamp(-1, 1).to(torch.int8)
    return q, (1.0 / s).to(torch.bfloat16).reshape(1)


class BitLinearKernel(nn.Module):
    """gpu/model.py:54-75.  `weight` is int8 [ceil16(N), ceil128(K)/4] in the W2T layout
    (pack_weight.convert_weight_int8_to_int2); `weight_scale` is the reference's bf16 [4]
    (one entry per fused sub-matrix, zero padded, gpu/convert_checkpoint.py:46-77);
    `segments` lists the row count of each sub-matrix."""

    def __init__(self, in_features: int, out_features: int, segments: Optional[Sequence[int]] = None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.segments = list(segments) if segments else [out_features]
        assert sum(self.segments) == out_features and len(self.segments) <= 4
        n_pad, k_pad = (out_features + 15) // 16 * 16, (in_features + 127) // 128 * 128
        self.weight = nn.Parameter(torch.zeros(n_pad, k_pad // 4, dtype=torch.int8), requires_grad=False)
        self.weight_scale = nn.Parameter(torch.zeros(4, dtype=torch.bfloat16), requires_grad=False)
        self.register_buffer("scale_f32", torch.zeros(len(self.segments), dtype=torch.float32), persistent=False)
        ends, acc = [], 0
        for n in self.segments:
            acc += n
            ends.append(acc)
        self.seg_end = ends

    @torch.no_grad()
    def load_ternary(self, parts: Sequence[torch.Tensor], scales: Sequence[torch.Tensor]):
        """parts[i]: ternary int8 [segments[i], K] on the GPU; scales[i]: bf16 scalar tensor."""
        q = torch.cat(list(parts), dim=0) if len(parts) > 1 else parts[0]
        self.weight.data = pack_weight.convert_weight_int8_to_int2(q)
        ws = torch.zeros(4, dtype=torch.bfloat16, device=q.device)
        for i, s in enumerate(scales):
            ws[i] = s.reshape(()).to(torch.bfloat16)
        self.weight_scale.data = ws
        self.scale_f32 = ws[: len(self.segments)].float().contiguous()

    def forward(self, x: torch.Tensor, norm: Optional[RMSNorm] = None) -> torch.Tensor:
        y, a, ysum = ops.quant_input(x, None if norm is None else norm.weight, 0.0 if norm is None else norm.eps)
        out = ops.linear_w2a8(y, a, ysum, self.weight, self.scale_f32, self.seg_end, self.out_features,
                              self.in_features)
        return out.view(*x.shape[:-1], self.out_features)

    def from_quantised(self, qa) -> torch.Tensor:
        """The matmul alone on already quantised activations (y, act_scale, ysum) -> bf16 [M, N]."""
        y, a, ysum = qa
        return ops.linear_w2a8(y, a, ysum, self.weight, self.scale_f32, self.seg_end, self.out_features, self.in_features)

    def add_into(self, qa, h: torch.Tensor, next_norm: Optional[RMSNorm]):
        """h += self(qa) in place, then quant_input(next_norm(h)) in the same launch (None without a
        next norm): ops.linear_w2a8_add_quant.  One row segment only (wo, w2)."""
        assert len(self.segments) == 1
        if getattr(self, "_host_scale", None) is None:       # read once, outside any stream capture
            self._host_scale = float(self.scale_f32[0])
        y, a, ysum = qa
        return ops.linear_w2a8_add_quant(y, a, ysum, self.weight, self._host_scale, self.out_features, self.in_features, h,
                                         None if next_norm is None else next_norm.weight,
                                         0.0 if next_norm is None else next_norm.eps)

    def forward_glu(self, x13: torch.Tensor, norm: Optional[RMSNorm] = None) -> torch.Tensor:
        """forward(squared_relu(x1) * x3, norm) for x13 = [x1 | x3], the gate fused into the
        quantisation kernel."""
        y, a, ysum = ops.quant_input_glu(x13, None if norm is None else norm.weight, 0.0 if norm is None else norm.eps)
        out = ops.linear_w2a8(y, a, ysum, self.weight, self.scale_f32, self.seg_end, self.out_features,
                              self.in_features)
        return out.view(*x13.shape[:-1], self.out_features)


class BitLinear(nn.Linear):
    """The BitLinear arithmetic in plain PyTorch: per-token absmax int8 quantisation
    (gpu/model.py:78-81), an exact integer product with the ternary weight, then the rescale
    in the order the reference's GPU kernel applies it (gpu/bitnet_kernels/bitnet_kernels.h:82:
    divide by the activation scale, multiply by the weight scale, round to bf16).  Library
    matmul in f32, exact because every partial sum is an integer below 2^24.  It is the
    floating-point reference that the kernel path is compared with; `weight` holds the
    dequantised ternary weight (as the reference's bf16 prefill model does), `ternary` and
    `row_scale` its two factors."""

    def __init__(self, in_features: int, out_features: int, segments: Optional[Sequence[int]] = None):
        super().__init__(in_features, out_features, bias=False, dtype=torch.bfloat16)
        self.weight.requires_grad_(False)
        self.register_buffer("ternary", torch.zeros(out_features, in_features, dtype=torch.float32), persistent=False)
        self.register_buffer("row_scale", torch.ones(out_features, dtype=torch.float32), persistent=False)

    def quant_input(self, x: torch.Tensor):
        xf = x.float()
        s = 127.0 / xf.abs().max(dim=-1, keepdim=True).values.clamp_(min=1e-5)
        return (xf * s).round().clamp(-128, 127), s

    def forward(self, x: torch.Tensor, norm: Optional[RMSNorm] = None) -> torch.Tensor:
        if norm is not None:
            x = norm(x)
        y, s = self.quant_input(x)
        assert self.in_features * 128 < (1 << 24)
        acc = F.linear(y, self.ternary)
        return (acc / s * self.row_scale).to(torch.bfloat16)


def rope_table(head_dim: int, max_len: int, theta: float, device) -> torch.Tensor:
    """[max_len, head_dim/2, 2] f32 cos/sin."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1)


def apply_rope(x: torch.Tensor, cs: torch.Tensor) -> torch.Tensor:
    """Rotates adjacent pairs (2i, 2i+1), as the interleaved rope the reference uses
    (gpu/model.py:144-152 with the row permutation of gpu/convert_safetensors.py:43-47).
    x: [B, T, H, D]; cs: [B, T, D/2, 2]."""
    xf = x.float().unflatten(-1, (-1, 2))
    c, s = cs[:, :, None, :, 0], cs[:, :, None, :, 1]
    out = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c], dim=-1)
    return out.flatten(-2).to(x.dtype)


class Attention(nn.Module):
    """gpu/model.py:87-162."""

    def __init__(self, dim, head_dim, n_heads, n_kv_heads, rope_theta, norm_eps, use_kernel):
        super().__init__()
        self.head_dim, self.rope_theta = head_dim, rope_theta
        self.n_local_heads, self.n_local_kv_heads = n_heads, n_kv_heads
        Linear = BitLinearKernel if use_kernel else BitLinear
        self.wqkv = Linear(dim, (n_heads + 2 * n_kv_heads) * head_dim,
                           segments=[n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim])
        self.wo = Linear(n_heads * head_dim, dim)
        self.attn_sub_norm = RMSNorm(dim, norm_eps)
        self.kernel_attention = True   # False: PyTorch attention for single-token steps too

    def forward(self, x, norm, cache: LayerCache, pos: torch.Tensor, rope: torch.Tensor,
                kv_len: Optional[int] = None) -> torch.Tensor:
        B, T, _ = x.shape
        H, Hkv, D = self.n_local_heads, self.n_local_kv_heads, self.head_dim
        xqkv = self.wqkv(x, norm)
        if T == 1 and kv_len is None and isinstance(self.wqkv, BitLinearKernel) and self.kernel_attention:
            # decode: the library's attention kernel (RoPE + cache append + split attention)
            out = ops.attention_decode(xqkv.view(B, -1), pos, rope, cache[0], cache[1], H, Hkv, D)
            return self.wo(out.view(B, 1, H * D), self.attn_sub_norm)
        xq = xqkv[..., : H * D].view(B, T, H, D)
        xk = xqkv[..., H * D: (H + Hkv) * D].view(B, T, Hkv, D)
        xv = xqkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
        p = pos[:, None] + torch.arange(T, device=x.device)[None, :]           # [B, T]
        cs = rope[p]
        xq, xk = apply_rope(xq, cs), apply_rope(xk, cs)
        cache_k, cache_v = cache
        bidx = torch.arange(B, device=x.device)[:, None].expand(B, T)
        cache_k.index_put_((bidx, p), xk)
        cache_v.index_put_((bidx, p), xv)
        L = cache_k.shape[1] if kv_len is None else kv_len
        keys, vals = cache_k[:, :L].transpose(1, 2), cache_v[:, :L].transpose(1, 2)
        mask = torch.arange(L, device=x.device)[None, None, None, :] <= p[:, None, :, None]
        out = F.scaled_dot_product_attention(xq.transpose(1, 2), keys, vals, attn_mask=mask, enable_gqa=True)
        out = out.transpose(1, 2).reshape(B, T, H * D)
        return self.wo(out, self.attn_sub_norm)


def squared_relu(x: torch.Tensor) -> torch.Tensor:
    return F.relu(x) ** 2


class FeedForward(nn.Module):
    """gpu/model.py:168-197."""

    def __init__(self, dim, hidden_dim, norm_eps, use_kernel):
        super().__init__()
        Linear = BitLinearKernel if use_kernel else BitLinear
        self.w13 = Linear(dim, 2 * hidden_dim, segments=[hidden_dim, hidden_dim])
        self.w2 = Linear(hidden_dim, dim)
        self.ffn_sub_norm = RMSNorm(hidden_dim, norm_eps)

    def forward(self, x: torch.Tensor, norm: RMSNorm) -> torch.Tensor:
        x13 = self.w13(x, norm)
        if isinstance(self.w2, BitLinearKernel):
            return self.w2.forward_glu(x13, self.ffn_sub_norm)
        x1, x3 = x13.chunk(2, -1)
        return self.w2(squared_relu(x1) * x3, self.ffn_sub_norm)


class TransformerBlock(nn.Module):
    """gpu/model.py:199-243."""

    def __init__(self, args: ModelArgs):
        super().__init__()
        self.attention = Attention(args.dim, args.head_dim, args.n_heads, args.n_kv_heads, args.rope_theta,
                                   args.norm_eps, args.use_kernel)
        self.feed_forward = FeedForward(args.dim, args.ffn_dim, args.norm_eps, args.use_kernel)
        self.attention_norm = RMSNorm(args.dim, args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, args.norm_eps)

    def forward(self, x, cache, pos, rope, kv_len=None):
        h = x + self.attention(x, self.attention_norm, cache, pos, rope, kv_len)
        return h + self.feed_forward(h, self.ffn_norm)

    def decode_fused(self, h: torch.Tensor, qa, cache, pos, rope, next_norm: Optional[RMSNorm]):
        """One decode step of the layer for 16 sequences or more on the kernel path, with the
        residual additions, the norms and the quantisations behind wo and w2 fused into their
        BitLinears: the same arithmetic as forward(), 10 launches instead of 15.
        h bf16 [B, dim] (updated in place); qa = quant_input(attention_norm(h)); returns the
        quantised input of the next layer (None behind the last one)."""
        att, ff = self.attention, self.feed_forward
        xqkv = att.wqkv.from_quantised(qa)
        out = ops.attention_decode(xqkv, pos, rope, cache[0], cache[1], att.n_local_heads, att.n_local_kv_heads, att.head_dim)
        qo = ops.quant_input(out, att.attn_sub_norm.weight, att.attn_sub_norm.eps)
        q13 = att.wo.add_into(qo, h, self.ffn_norm)
        x13 = ff.w13.from_quantised(q13)
        q2 = ops.quant_input_glu(x13, ff.ffn_sub_norm.weight, ff.ffn_sub_norm.eps)
        return ff.w2.add_into(q2, h, next_norm)


class Transformer(nn.Module):
    """gpu/model.py:246-296."""

    def __init__(self, args: ModelArgs, max_seq_len: int = 4096):
        super().__init__()
        self.args = args
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim, dtype=torch.bfloat16)
        self.tok_embeddings.weight.requires_grad_(False)
        self.layers = nn.ModuleList(TransformerBlock(args) for _ in range(args.n_layers))
        self.norm = RMSNorm(args.dim, args.norm_eps)
        self.output = nn.Linear(args.dim, args.vocab_size, bias=False, dtype=torch.bfloat16)
        self.output.weight.requires_grad_(False)
        if args.tie_embeddings:
            self.output.weight = self.tok_embeddings.weight
        self.max_seq_len = max_seq_len
        self.rope: Optional[torch.Tensor] = None
        self.fused_decode = True      # False: batched decode through the plain per-module path (for comparisons)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, cache: List[LayerCache],
                kv_len: Optional[int] = None, last_only: bool = False) -> torch.Tensor:
        """tokens int64 [B, T]; pos int64 [B] (tokens already cached); returns f32 logits
        [B, T, vocab], or [B, 1, vocab] for the last position only."""
        if self.rope is None or self.rope.device != tokens.device:
            self.rope = rope_table(self.args.head_dim, self.max_seq_len, self.args.rope_theta, tokens.device)
        h = self.tok_embeddings(tokens)
        B, T = tokens.shape
        if (self.fused_decode and T == 1 and kv_len is None and B >= 16 and self.args.use_kernel and self.args.dim % 8 == 0
                and all(l.attention.kernel_attention for l in self.layers)):
            # batched decode on the kernel path: residual, norm and quantisation fused behind wo and w2
            h = h.view(B, self.args.dim).contiguous()
            first = self.layers[0].attention_norm
            qa = ops.quant_input(h, first.weight, first.eps)
            for i, (layer, c) in enumerate(zip(self.layers, cache)):
                nxt = self.layers[i + 1].attention_norm if i + 1 < len(self.layers) else None
                qa = layer.decode_fused(h, qa, c, pos, self.rope, nxt)
            return self.output(self.norm(h.view(B, 1, self.args.dim))).float()
        for layer, c in zip(self.layers, cache):
            h = layer(h, c, pos, self.rope, kv_len)
        if last_only:
            h = h[:, -1:]
        return self.output(self.norm(h)).float()


def make_cache(args: ModelArgs, batch: int, length: int, device=None, dtype=torch.bfloat16) -> List[LayerCache]:
    """bf16 KV cache, one (k, v) pair per layer, each [batch, length, n_kv_heads, head_dim]
    (the reference's flat [1, batch*length, n_kv, 1, head_dim] of gpu/model.py:299-343 with
    the batch dimension split out)."""
    shape = (batch, length, args.n_kv_heads, args.head_dim)
    return [(torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype))
            for _ in range(args.n_layers)]


@torch.no_grad()
def build_synthetic(args: ModelArgs, seed: int = 0, device="cuda", max_seq_len: int = 4096) -> Transformer:
    """Random-initialised model of the given architecture: every BitLinear sub-matrix is
    drawn N(0,1) from a seeded generator and absmean-ternarised with a bf16 scale
    (gpu/convert_checkpoint.py:23-27,41-83); embeddings and norm weights are bf16."""
    with torch.device("meta"):
        model = Transformer(args, max_seq_len)
    model = model.to_empty(device=device)
    gen = torch.Generator(device=device)

    def ternary(n, k, s):
        gen.manual_seed(s)
        w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32)
        return quant_weight_int8(w)

    def fill(lin, tag):
        parts, scales = [], []
        for j, n in enumerate(lin.segments if isinstance(lin, BitLinearKernel) else getattr(lin, "_segments")):
            q, s = ternary(n, lin.in_features, seed * 1000003 + tag * 8 + j)
            parts.append(q)
            scales.append(s)
        if isinstance(lin, BitLinearKernel):
            lin.load_ternary(parts, scales)
        else:
            lin.weight.data = torch.cat([p.to(torch.bfloat16) * s for p, s in zip(parts, scales)], dim=0)
            lin.ternary = torch.cat(parts, dim=0).float()
            lin.row_scale = torch.cat([s.float().expand(p.shape[0]) for p, s in zip(parts, scales)])

    gen.manual_seed(seed * 1000003 + 1)
    model.tok_embeddings.weight.data = torch.randn((args.vocab_size, args.dim), generator=gen, device=device,
                                                   dtype=torch.float32).to(torch.bfloat16)
    if args.tie_embeddings:
        model.output.weight = model.tok_embeddings.weight
    else:
        gen.manual_seed(seed * 1000003 + 2)
        model.output.weight.data = torch.randn((args.vocab_size, args.dim), generator=gen, device=device,
                                               dtype=torch.float32).to(torch.bfloat16)
    model.norm.weight.data = torch.ones(args.dim, dtype=torch.bfloat16, device=device)
    D = args.head_dim
    for i, layer in enumerate(model.layers):
        att, ff = layer.attention, layer.feed_forward
        if not args.use_kernel:
            att.wqkv._segments = [args.n_heads * D, args.n_kv_heads * D, args.n_kv_heads * D]
            att.wo._segments = [args.dim]
            ff.w13._segments = [args.ffn_dim, args.ffn_dim]
            ff.w2._segments = [args.dim]
        fill(att.wqkv, 100 + i * 4 + 0)
        fill(att.wo, 100 + i * 4 + 1)
        fill(ff.w13, 100 + i * 4 + 2)
        fill(ff.w2, 100 + i * 4 + 3)
        for nrm, nd in ((layer.attention_norm, args.dim), (layer.ffn_norm, args.dim),
                        (att.attn_sub_norm, args.dim), (ff.ffn_sub_norm, args.ffn_dim)):
            gen.manual_seed(seed * 1000003 + 7 + i)
            nrm.weight.data = (1.0 + 0.1 * torch.randn(nd, generator=gen, device=device)).to(torch.bfloat16)
    model.rope = rope_table(D, max_seq_len, args.rope_theta, device)
    return model
