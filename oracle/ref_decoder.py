"""A CPU decoder made only of the checkers in this folder.  Test infrastructure only.

It restates one decode step of the reference's GPU model (gpu/model.py:269-282 through
TransformerBlock :231-243, Attention :121-162 and FeedForward :192-197) on NumPy arrays,
with every BitLinear running the reference's CPU arithmetic: per-token absmax int8
activations (gpu/model.py:68-71), the I2_S code sums of the reference's compiled kernel
(``RefLib.gemm``; the plain-C port where that library is absent) on I2_S bytes packed from
the same ternary weights, the ``- sum(y)`` offset, and the rescale in the order of
gpu/bitnet_kernels/bitnet_kernels.h:82.  Tensors that the reference keeps in bf16 are
rounded to bf16 after every operation that produces them.

The CUDA path is compared with it end to end (tests/test_gpu_e2e_oracle.py); nothing in the
product imports it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import np_oracle as O


@dataclass
class OracleLinear:
    """One BitLinear: ternary weights as I2_S bytes, one scale per row segment."""

    i2s: np.ndarray              # I2_S bytes (np_oracle.i2s_pack)
    q: np.ndarray                # the same weights as ternary int8 [N, K]
    n: int
    k: int
    scales: np.ndarray           # f32 [n_seg]
    seg_end: Sequence[int]

    @classmethod
    def from_ternary(cls, q: np.ndarray, scales, seg_end):
        q = np.ascontiguousarray(q, dtype=np.int8)
        n, k = q.shape
        buf = O.i2s_pack(q, 1.0) if (k % 128 == 0 and (n * k) % 128 == 0) else None
        return cls(buf, q, n, k, np.asarray(scales, dtype=np.float32), list(seg_end))


class OracleDecoder:
    """Holds the weights of a decoder as NumPy arrays and decodes one token per call."""

    def __init__(self, dim, n_heads, n_kv_heads, ffn_dim, vocab, eps, rope_theta, max_seq, gemm_lib=None):
        self.dim, self.H, self.Hkv, self.F, self.V = dim, n_heads, n_kv_heads, ffn_dim, vocab
        self.D = dim // n_heads
        self.eps = np.float32(eps)
        self.max_seq = max_seq
        self.lib = gemm_lib                  # RefLib or PortLib; None = exact NumPy integer product
        self.layers: List[dict] = []
        self.emb: Optional[np.ndarray] = None        # f32 values of the bf16 table [V, dim]
        self.out_w: Optional[np.ndarray] = None
        self.final_norm: Optional[np.ndarray] = None
        inv = (1.0 / (np.float32(rope_theta) ** (np.arange(0, self.D, 2, dtype=np.float32) / np.float32(self.D)))).astype(np.float32)
        ang = np.arange(max_seq, dtype=np.float32)[:, None] * inv[None, :]
        self.cos, self.sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        self.cache: List[tuple] = []
        self.trace: Optional[list] = None    # when a list: (name, y int8, acc int32, out f32) per BitLinear

    def add_layer(self, wqkv: OracleLinear, wo: OracleLinear, w13: OracleLinear, w2: OracleLinear, attention_norm,
                  attn_sub_norm, ffn_norm, ffn_sub_norm):
        f32 = lambda a: np.asarray(a, dtype=np.float32)
        self.layers.append(dict(wqkv=wqkv, wo=wo, w13=w13, w2=w2, attention_norm=f32(attention_norm),
                                attn_sub_norm=f32(attn_sub_norm), ffn_norm=f32(ffn_norm), ffn_sub_norm=f32(ffn_sub_norm)))

    def set_rope(self, table: np.ndarray):
        """Takes cos/sin from a [max_seq, D/2, 2] table (so that both sides of a comparison
        rotate by the same f32 values)."""
        table = np.asarray(table, dtype=np.float32)
        self.cos, self.sin = np.ascontiguousarray(table[..., 0]), np.ascontiguousarray(table[..., 1])

    def reset(self, batch: int):
        self.cache = [(np.zeros((batch, self.max_seq, self.Hkv, self.D), dtype=np.float32),
                       np.zeros((batch, self.max_seq, self.Hkv, self.D), dtype=np.float32)) for _ in self.layers]

    # ---- one BitLinear -------------------------------------------------------------------
    def code_sums(self, lin: OracleLinear, y: np.ndarray) -> np.ndarray:
        """sum_k (q+1) * y through the compiled I2_S kernel when the shape allows it."""
        if self.lib is not None and lin.i2s is not None:
            return np.asarray(self.lib.gemm(lin.i2s, y, lin.n, lin.k)).astype(np.int64).astype(np.int32)
        return O.matmul_i32(y, lin.q + 1)

    def bitlinear(self, lin: OracleLinear, x: np.ndarray, norm_w: Optional[np.ndarray], name: str = "") -> np.ndarray:
        """x f32 [M, K] (bf16 values) -> bf16-valued f32 [M, N]."""
        if norm_w is not None:
            x = O.to_bf16(O.rmsnorm(x, norm_w, float(self.eps)))
        y, a, ysum = O.act_quant(x)
        acc = self.code_sums(lin, y) - ysum[:, None]
        out = O.to_bf16(O.rescale(acc, a, lin.scales, lin.seg_end))
        if self.trace is not None:
            self.trace.append((name, y, acc, out))
        return out

    # ---- attention of one new token (gpu/model.py:121-158) --------------------------------
    def attention(self, li: int, xqkv: np.ndarray, pos: np.ndarray) -> np.ndarray:
        B = xqkv.shape[0]
        H, Hkv, D = self.H, self.Hkv, self.D
        q = xqkv[:, : H * D].reshape(B, H, D)
        k = xqkv[:, H * D: (H + Hkv) * D].reshape(B, Hkv, D)
        v = xqkv[:, (H + Hkv) * D:].reshape(B, Hkv, D)

        def rope(t, p):  # adjacent pairs rotate together; products rounded separately, result to bf16
            c, s = self.cos[p][None, :], self.sin[p][None, :]
            t0, t1 = t[..., 0::2], t[..., 1::2]
            r0 = O.to_bf16((t0 * c).astype(np.float32) - (t1 * s).astype(np.float32))
            r1 = O.to_bf16((t0 * s).astype(np.float32) + (t1 * c).astype(np.float32))
            out = np.empty_like(t)
            out[..., 0::2], out[..., 1::2] = r0, r1
            return out

        ck, cv = self.cache[li]
        out = np.zeros((B, H * D), dtype=np.float32)
        G = H // Hkv
        scale = np.float32(1.0) / np.sqrt(np.float32(D))
        for b in range(B):
            p = int(pos[b])
            qb, kb = rope(q[b], p), rope(k[b], p)
            ck[b, p], cv[b, p] = kb, v[b]
            keys, vals = ck[b, : p + 1], cv[b, : p + 1]              # [P+1, Hkv, D]
            for h in range(H):
                kvh = h // G
                s = (keys[:, kvh, :].astype(np.float64) @ qb[h].astype(np.float64)) * float(scale)
                w = np.exp(s - s.max())
                w /= w.sum()
                out[b, h * D:(h + 1) * D] = (w @ vals[:, kvh, :].astype(np.float64)).astype(np.float32)
        return O.to_bf16(out)

    # ---- one decoder layer, one decode step ------------------------------------------------
    def layer_forward(self, li: int, h: np.ndarray, pos: np.ndarray, att_given: Optional[np.ndarray] = None) -> np.ndarray:
        """h f32 [B, dim] (bf16 values) -> the layer's output, TransformerBlock.forward of
        gpu/model.py:231-243 for one new token per sequence.  att_given: take this as the
        attention output instead of computing it (the cache is still updated), so that a
        comparison of the BitLinear path does not hinge on two softmax implementations
        rounding alike."""
        L = self.layers[li]
        xqkv = self.bitlinear(L["wqkv"], h, L["attention_norm"], f"l{li}.wqkv")
        att = self.attention(li, xqkv, pos)
        self.last_attention = att
        if att_given is not None:
            att = np.asarray(att_given, dtype=np.float32)
        h = O.to_bf16(h + self.bitlinear(L["wo"], att, L["attn_sub_norm"], f"l{li}.wo"))
        x13 = self.bitlinear(L["w13"], h, L["ffn_norm"], f"l{li}.w13")
        x1, x3 = x13[:, : self.F], x13[:, self.F:]
        r = np.maximum(x1, np.float32(0))
        glu = O.to_bf16(O.to_bf16(r * r) * x3)                         # gpu/model.py:193-195 in bf16
        return O.to_bf16(h + self.bitlinear(L["w2"], glu, L["ffn_sub_norm"], f"l{li}.w2"))

    def head(self, h: np.ndarray) -> np.ndarray:
        """Final norm and output projection (gpu/model.py:280-281): bf16-valued f32 logits."""
        xn = O.to_bf16(O.rmsnorm(h, self.final_norm, float(self.eps)))
        return O.to_bf16((xn.astype(np.float64) @ self.out_w.astype(np.float64).T).astype(np.float32))

    def step(self, tokens: np.ndarray, pos: np.ndarray, att_given: Optional[Sequence[np.ndarray]] = None) -> np.ndarray:
        """tokens int [B], pos int [B] (keys already cached).  Returns logits [B, V].
        att_given[l]: attention output to use in layer l (see layer_forward); the oracle's own
        attention outputs of the step are kept in self.attention_outputs."""
        h = self.emb[np.asarray(tokens).reshape(-1)]
        self.attention_outputs = []
        for li in range(len(self.layers)):
            h = self.layer_forward(li, h, pos, None if att_given is None else att_given[li])
            self.attention_outputs.append(self.last_attention)
        return self.head(h)
