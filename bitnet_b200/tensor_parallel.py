"""Tensor-parallel BitNet decoder: one process per GPU, `torch.distributed` for the exchange.

The reference has no multi-GPU path (gpu/generate.py:324-326 fixes local_rank = 0); this is
the partition its fused layout invites (gpu/model.py:103-118 names the per-rank head counts
`n_local_heads` / `n_local_kv_heads`):

* column-parallel `wqkv` (each rank owns n_heads/tp query heads and n_kv_heads/tp key/value
  heads, with their slice of the KV cache) and `w13` (each rank owns ffn/tp gate rows and the
  matching up rows): no exchange, the input is replicated;
* row-parallel `wo` and `w2` (each rank owns a K slice of the weight).  The input of a
  row-parallel BitLinear passes through an RMSNorm and an absmax over the *whole* vector
  (gpu/model.py:159-160, 195-196), so the local slices are first **all-gathered** (a few KB
  per token) and every rank quantises the whole vector, exactly as a single GPU would; it
  then multiplies only its K slice and the exact int32 partial sums are **all-reduced**.
  Integer sums do not depend on the order of addition, so the result is bit-identical to
  the single-GPU result for every tp.
* the output projection is split over the vocabulary; the greedy choice is an all-gather of
  one (value, index) pair per rank.

Per layer: 2 all-gathers + 2 all-reduces.  `backend="torch"` runs the same algebra with
plain PyTorch BitLinear arithmetic (for CPU tests under gloo); `backend="kernel"` uses the
library's kernels.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch.nn import functional as F

from .model import ModelArgs, RMSNorm, apply_rope, quant_weight_int8, rope_table, squared_relu


def _seed(seed: int, layer: int, which: int, part: int) -> int:
    """The seed build_synthetic uses for sub-matrix `part` of BitLinear `which` of `layer`."""
    return seed * 1000003 + (100 + layer * 4 + which) * 8 + part


def _ternary_rows(n: int, k: int, s: int, device, rows: slice, cols: slice = slice(None)):
    """Rows/columns of the ternarised N(0,1) matrix with seed s.  The whole matrix is drawn and
    ternarised first: its scale is the scale of the full tensor (gpu/convert_checkpoint.py:23-27)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(s)
    q, scale = quant_weight_int8(torch.randn((n, k), generator=gen, device=device, dtype=torch.float32))
    return q[rows, cols].contiguous(), scale


class _Linear:
    """One BitLinear shard.  `cols` = (k0, k1) for a row-parallel shard (it multiplies columns
    k0..k1 of the quantised input), None for a column-parallel one."""

    def __init__(self, parts, scales, in_features: int, backend: str, cols: Optional[Tuple[int, int]] = None):
        self.backend, self.cols, self.in_features = backend, cols, in_features
        self.segments = [p.shape[0] for p in parts]
        self.n = sum(self.segments)
        self.k_local = parts[0].shape[1]
        ends, acc = [], 0
        for s in self.segments:
            acc += s
            ends.append(acc)
        self.seg_end = ends
        dev = parts[0].device
        self.scale = torch.stack([s.reshape(()).float() for s in scales]).to(dev)          # f32 [n_seg]
        self.row_scale = torch.cat([s.float().reshape(1).expand(p.shape[0]) for p, s in zip(parts, scales)]).to(dev)
        q = torch.cat(list(parts), dim=0)
        if backend == "kernel":
            from . import pack_weight
            self.weight = pack_weight.convert_weight_int8_to_int2(q)
        else:
            self.ternary = q.float()

    def quantize(self, x: torch.Tensor, norm: Optional[RMSNorm]):
        """x bf16 [M, K] over the full K.  Returns the backend's quantised activations."""
        if self.backend == "kernel":
            from . import ops
            return ops.quant_input(x, None if norm is None else norm.weight, 0.0 if norm is None else norm.eps)
        xf = (norm(x) if norm is not None else x).float()
        a = 127.0 / xf.abs().amax(dim=-1).clamp_(min=1e-5)
        return (xf * a[:, None]).round().clamp(-128, 127), a, None

    def accumulate(self, quantised) -> torch.Tensor:
        """Exact sum_k y[m,k] * w[n,k] over this shard's columns: int32 (kernel) or f32 holding
        exact integers (torch)."""
        y, a, ysum = quantised
        k0, k1 = self.cols if self.cols is not None else (0, self.in_features)
        if self.backend == "kernel":
            from . import ops
            ys = y[:, k0:] if self.cols is not None else y
            return ops.linear_w2a8(ys, None, ysum if self.cols is None else None, self.weight, None, [self.n], self.n,
                                   k1 - k0, want_acc=True, want_out=False)
        assert (k1 - k0) * 128 < (1 << 24)
        return F.linear(y[:, k0:k1], self.ternary)

    def rescale(self, acc: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
        """bf16(acc / a * ws), the order of gpu/bitnet_kernels/bitnet_kernels.h:82."""
        return (acc.float() / a[:, None] * self.row_scale).to(torch.bfloat16)

    def __call__(self, x: torch.Tensor, norm: Optional[RMSNorm]) -> torch.Tensor:
        qz = self.quantize(x, norm)
        return self.rescale(self.accumulate(qz), qz[1])


class TPDecoder:
    """The decoder of `model.Transformer`, sharded over `world` ranks.  With world == 1 it
    computes exactly what `model.build_synthetic(args, seed)` computes."""

    def __init__(self, args: ModelArgs, seed: int, rank: int, world: int, device, backend: str = "kernel",
                 max_seq_len: int = 4096, group=None, fast_random: bool = False):
        """fast_random=True (for benchmarks of large models): every shard is drawn directly as
        uniform ternary values with a fixed scale, seeded by (seed, layer, tensor, rank), instead
        of being cut out of the ternarised whole matrix; the shards of different tp degrees then
        do not make up the same model, which a throughput measurement does not need."""
        assert args.n_heads % world == 0 and args.n_kv_heads % world == 0, "heads must divide by the tp degree"
        assert args.ffn_dim % world == 0 and args.vocab_size % world == 0
        D = args.head_dim
        self.args, self.rank, self.world, self.device, self.group, self.backend = args, rank, world, device, group, backend
        self.Hl, self.Hkvl = args.n_heads // world, args.n_kv_heads // world
        Fl = args.ffn_dim // world
        if backend == "kernel":
            assert (self.Hl * D) % 128 == 0 and Fl % 128 == 0, "K slices must be multiples of the 128-column tile"
        gen = torch.Generator(device=device)

        def bf16_randn(shape, s):
            gen.manual_seed(s)
            return torch.randn(shape, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)

        self.emb = bf16_randn((args.vocab_size, args.dim), seed * 1000003 + 1)
        out_w = self.emb if args.tie_embeddings else bf16_randn((args.vocab_size, args.dim), seed * 1000003 + 2)
        Vl = args.vocab_size // world
        self.out_w = out_w[rank * Vl:(rank + 1) * Vl].contiguous()
        self.vocab_lo = rank * Vl
        self.final_norm = RMSNorm(args.dim, args.norm_eps).to(device)
        self.layers = []
        r = rank

        def _rows(n, k, s, device, rows, cols=slice(None)):
            if not fast_random:
                return _ternary_rows(n, k, s, device, rows, cols)
            nl = len(range(*rows.indices(n)))
            kl = len(range(*cols.indices(k)))
            g2 = torch.Generator(device=device)
            g2.manual_seed(s * 131 + rank)
            return (torch.randint(-1, 2, (nl, kl), generator=g2, device=device, dtype=torch.int8),
                    torch.tensor([0.8], dtype=torch.bfloat16, device=device))

        for i in range(args.n_layers):
            qs, ks = slice(r * self.Hl * D, (r + 1) * self.Hl * D), slice(r * self.Hkvl * D, (r + 1) * self.Hkvl * D)
            q_p, s_q = _rows(args.n_heads * D, args.dim, _seed(seed, i, 0, 0), device, qs)
            k_p, s_k = _rows(args.n_kv_heads * D, args.dim, _seed(seed, i, 0, 1), device, ks)
            v_p, s_v = _rows(args.n_kv_heads * D, args.dim, _seed(seed, i, 0, 2), device, ks)
            wo_p, s_o = _rows(args.dim, args.n_heads * D, _seed(seed, i, 1, 0), device, slice(None), qs)
            fs = slice(r * Fl, (r + 1) * Fl)
            g_p, s_1 = _rows(args.ffn_dim, args.dim, _seed(seed, i, 2, 0), device, fs)
            u_p, s_3 = _rows(args.ffn_dim, args.dim, _seed(seed, i, 2, 1), device, fs)
            w2_p, s_2 = _rows(args.dim, args.ffn_dim, _seed(seed, i, 3, 0), device, slice(None), fs)
            norms = {}
            for name, nd in (("attention_norm", args.dim), ("ffn_norm", args.dim), ("attn_sub_norm", args.dim),
                             ("ffn_sub_norm", args.ffn_dim)):
                gen.manual_seed(seed * 1000003 + 7 + i)
                nrm = RMSNorm(nd, args.norm_eps).to(device)
                nrm.weight.data = (1.0 + 0.1 * torch.randn(nd, generator=gen, device=device)).to(torch.bfloat16)
                norms[name] = nrm
            self.layers.append(dict(
                wqkv=_Linear([q_p, k_p, v_p], [s_q, s_k, s_v], args.dim, backend),
                wo=_Linear([wo_p], [s_o], args.n_heads * D, backend, cols=(qs.start, qs.stop)),
                w13=_Linear([g_p, u_p], [s_1, s_3], args.dim, backend),
                w2=_Linear([w2_p], [s_2], args.ffn_dim, backend, cols=(fs.start, fs.stop)), **norms))
        self.rope = rope_table(D, max_seq_len, args.rope_theta, device)
        self.max_seq_len = max_seq_len
        self.fused_one_rank = True      # False: batched decode on one rank through the per-op path as well (for comparisons)

    # ---- collectives --------------------------------------------------------------------
    def _all_gather_cols(self, x: torch.Tensor) -> torch.Tensor:
        """[M, n_local] per rank -> [M, world * n_local], rank-major columns."""
        if self.world == 1:
            return x
        out = torch.empty((self.world * x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out.view(self.world, x.shape[0], x.shape[1]).permute(1, 0, 2).reshape(x.shape[0], -1)

    def _all_reduce(self, acc: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return acc

    # ---- model ----------------------------------------------------------------------------
    def make_cache(self, batch: int, length: int):
        shape = (batch, length, self.Hkvl, self.args.head_dim)
        return [(torch.zeros(shape, device=self.device, dtype=torch.bfloat16),
                 torch.zeros(shape, device=self.device, dtype=torch.bfloat16)) for _ in self.layers]

    def _attention(self, xqkv, cache, pos, T, B, kv_len):
        Hl, Hkvl, D = self.Hl, self.Hkvl, self.args.head_dim
        if T == 1 and kv_len is None and self.backend == "kernel":
            from . import ops
            return ops.attention_decode(xqkv, pos, self.rope, cache[0], cache[1], Hl, Hkvl, D)
        xq = xqkv[:, : Hl * D].view(B, T, Hl, D)
        xk = xqkv[:, Hl * D: (Hl + Hkvl) * D].view(B, T, Hkvl, D)
        xv = xqkv[:, (Hl + Hkvl) * D:].view(B, T, Hkvl, D)
        p = pos[:, None] + torch.arange(T, device=xqkv.device)[None, :]
        cs = self.rope[p]
        xq, xk = apply_rope(xq, cs), apply_rope(xk, cs)
        bidx = torch.arange(B, device=xqkv.device)[:, None].expand(B, T)
        cache[0].index_put_((bidx, p), xk)
        cache[1].index_put_((bidx, p), xv)
        L = cache[0].shape[1] if kv_len is None else kv_len
        mask = torch.arange(L, device=xqkv.device)[None, None, None, :] <= p[:, None, :, None]
        keys, vals = cache[0][:, :L].transpose(1, 2), cache[1][:, :L].transpose(1, 2)
        if xq.device.type == "cpu":     # CPU SDPA has no bf16 GQA path everywhere: do it in f32
            rep = Hl // Hkvl
            out = F.scaled_dot_product_attention(xq.transpose(1, 2).float(), keys.float().repeat_interleave(rep, 1),
                                                 vals.float().repeat_interleave(rep, 1), attn_mask=mask)
            out = out.to(torch.bfloat16)
        else:
            out = F.scaled_dot_product_attention(xq.transpose(1, 2), keys, vals, attn_mask=mask, enable_gqa=True)
        return out.transpose(1, 2).reshape(B * T, Hl * D)

    @torch.no_grad()
    def _hidden_one_rank(self, tokens: torch.Tensor, pos: torch.Tensor, cache) -> torch.Tensor:
        """Batched decode on one rank: the same arithmetic as `hidden`, with the library's fused calls
        (matmul + rescale in one call; residual, norm and next quantisation behind wo and w2 in one
        kernel, as model.TransformerBlock.decode_fused)."""
        from . import ops

        a, B = self.args, tokens.shape[0]
        h = self.emb[tokens.reshape(-1)].contiguous()
        first = self.layers[0]["attention_norm"]
        qa = ops.quant_input(h, first.weight, first.eps)

        def mm(lin, q):
            return ops.linear_w2a8(q[0], q[1], q[2], lin.weight, lin.scale, lin.seg_end, lin.n, lin.in_features)

        def add_into(lin, q, nxt):
            if getattr(lin, "_host_scale", None) is None:       # read once, outside any stream capture
                lin._host_scale = float(lin.scale[0])
            return ops.linear_w2a8_add_quant(q[0], q[1], q[2], lin.weight, lin._host_scale, lin.n, lin.in_features, h,
                                             None if nxt is None else nxt.weight, 0.0 if nxt is None else nxt.eps)

        for i, (L, c) in enumerate(zip(self.layers, cache)):
            xqkv = mm(L["wqkv"], qa)
            att = ops.attention_decode(xqkv, pos, self.rope, c[0], c[1], self.Hl, self.Hkvl, a.head_dim)
            qo = ops.quant_input(att, L["attn_sub_norm"].weight, L["attn_sub_norm"].eps)
            q13 = add_into(L["wo"], qo, L["ffn_norm"])
            x13 = mm(L["w13"], q13)
            q2 = ops.quant_input_glu(x13, L["ffn_sub_norm"].weight, L["ffn_sub_norm"].eps)
            nxt = self.layers[i + 1]["attention_norm"] if i + 1 < len(self.layers) else None
            qa = add_into(L["w2"], q2, nxt)
        return h

    @torch.no_grad()
    def hidden(self, tokens: torch.Tensor, pos: torch.Tensor, cache, kv_len: Optional[int] = None) -> torch.Tensor:
        """tokens int64 [B, T] -> final hidden state bf16 [B*T, dim] (identical on every rank)."""
        B, T = tokens.shape
        if (self.world == 1 and self.backend == "kernel" and T == 1 and kv_len is None and B >= 16
                and self.args.dim % 8 == 0 and self.fused_one_rank):
            return self._hidden_one_rank(tokens, pos, cache)
        h = self.emb[tokens.reshape(-1)]
        for L, c in zip(self.layers, cache):
            xqkv = L["wqkv"](h, L["attention_norm"])
            att = self._all_gather_cols(self._attention(xqkv, c, pos, T, B, kv_len))
            qz = L["wo"].quantize(att, L["attn_sub_norm"])
            h = h + L["wo"].rescale(self._all_reduce(L["wo"].accumulate(qz)), qz[1])
            x13 = L["w13"](h, L["ffn_norm"])
            x1, x3 = x13.chunk(2, -1)
            inner = self._all_gather_cols(squared_relu(x1) * x3)
            qz = L["w2"].quantize(inner, L["ffn_sub_norm"])
            h = h + L["w2"].rescale(self._all_reduce(L["w2"].accumulate(qz)), qz[1])
        return h

    @torch.no_grad()
    def logits_local(self, h: torch.Tensor) -> torch.Tensor:
        x = self.final_norm(h)
        if x.device.type == "cpu":
            return F.linear(x.float(), self.out_w.float()).to(torch.bfloat16).float()
        return F.linear(x, self.out_w).float()

    @torch.no_grad()
    def logits(self, h: torch.Tensor) -> torch.Tensor:
        """Full-vocabulary logits f32 [M, vocab] (gathers the shards; for tests)."""
        return self._all_gather_cols(self.logits_local(h))

    @torch.no_grad()
    def greedy(self, h: torch.Tensor) -> torch.Tensor:
        """Greedy token per row: one (value, index) pair per rank is exchanged."""
        lg = self.logits_local(h)
        val, idx = lg.max(dim=-1)
        if self.world == 1:
            return idx + self.vocab_lo
        pair = torch.stack([val, (idx + self.vocab_lo).float()], dim=-1)                # [M, 2]; indices < 2^24
        allp = torch.empty((self.world * pair.shape[0], 2), dtype=pair.dtype, device=pair.device)
        dist.all_gather_into_tensor(allp, pair.contiguous(), group=self.group)
        allp = allp.view(self.world, pair.shape[0], 2)
        best = allp[..., 0].argmax(dim=0)                                               # first maximum: lowest rank
        return allp[best, torch.arange(pair.shape[0], device=pair.device), 1].long()

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, pos: torch.Tensor, cache) -> torch.Tensor:
        """tokens int64 [B, 1] -> next tokens int64 [B]."""
        return self.greedy(self.hidden(tokens, pos, cache))


class GraphedStep:
    """One greedy decode step of a TPDecoder captured in a CUDA graph (collectives included:
    NCCL work enqueued on the capturing stream becomes graph nodes).  The step feeds itself:
    `tokens` [B, 1] is overwritten with the chosen ids and `pos` [B] advances by one, so a
    decode loop is a sequence of `replay()` calls.  Every rank must build and replay it
    in step with the others."""

    def __init__(self, dec: "TPDecoder", tokens: torch.Tensor, pos: torch.Tensor, cache, warmup: int = 2):
        assert tokens.is_cuda and tokens.dim() == 2 and tokens.shape[1] == 1
        self.dec, self.tokens, self.pos, self.cache = dec, tokens, pos, cache
        self.out = torch.zeros((tokens.shape[0],), dtype=torch.int64, device=tokens.device)
        self.stream = torch.cuda.Stream(device=tokens.device)
        saved = tokens.clone()
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):      # allocations, lazy initialisation, NCCL connections
                self._body()
                self.tokens.copy_(saved)
                self.pos.sub_(1)
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
                self._body()
        torch.cuda.synchronize()

    def _body(self):
        nxt = self.dec.decode_step(self.tokens, self.pos, self.cache)
        self.out.copy_(nxt)
        self.tokens.copy_(nxt.view(-1, 1))
        self.pos.add_(1)

    def replay(self):
        self.graph.replay()


class TPFusedStep:
    """The tensor-parallel decode step inside the library (`bitnet_decoder_create_tp`): the
    chain of fused kernels of `generate.FusedDecoder`, with the shards of a `TPDecoder`
    (backend "kernel").  The ranks exchange through device memory mapped with CUDA IPC - the
    statistics of the row-parallel BitLinears' inputs and their exact int32 partial sums - inside
    the kernels; no collective library call is part of a step.  `group` is only used to hand
    the IPC handles round when the step is built.  Bit-identical to the same class with one rank.

    tokens int64 [B, 1] and pos int64 [B] live on the device and are advanced by the step;
    `out` holds the chosen ids.  Every rank must build it and call `step()` in step."""

    def __init__(self, dec: "TPDecoder", batch: int, max_seq_len: int, group=None, wait_limit_ms: Optional[float] = None,
                 absent_peers: bool = False, local_only: bool = False):
        """absent_peers=True (for tests of the bounded waits): the other ranks' exchange areas are
        plain buffers of this process that nobody ever writes to, and no process group is used.
        local_only=True (for timing): this rank's shards run as a model of their own, with no
        exchange at all - the same weight bytes and kernels minus the peer traffic and the waits,
        so that the difference to the real step is the cost of the exchange."""
        import ctypes

        from . import _lib
        from .generate import _DecoderConfig, _DecoderLayer

        assert dec.backend == "kernel" and 1 <= batch <= 8
        a, dev = dec.args, dec.device
        self.dec, self.batch, self.max_seq_len = dec, batch, max_seq_len
        self.cache = dec.make_cache(batch, max_seq_len)
        self.tokens = torch.zeros((batch, 1), dtype=torch.int64, device=dev)
        self.pos = torch.zeros((batch,), dtype=torch.int64, device=dev)
        self.out = torch.zeros((batch,), dtype=torch.int64, device=dev)
        cfg = _DecoderConfig(a.dim, a.n_layers, a.n_heads, a.n_kv_heads, a.head_dim, a.ffn_dim, a.vocab_size,
                             a.norm_eps, batch, max_seq_len)
        L = _lib.lib
        world, rank = dec.world, dec.rank
        if local_only:
            cfg = _DecoderConfig(a.dim, a.n_layers, dec.Hl, dec.Hkvl, a.head_dim, a.ffn_dim // world,
                                 a.vocab_size // world, a.norm_eps, batch, max_seq_len)
            world, rank = 1, 0
        self._area, self._peers = None, []
        areas = (ctypes.c_void_p * max(world, 1))()
        if world > 1:
            nbytes = L.bitnet_tp_area_bytes(ctypes.byref(cfg), world)
            area, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _lib.check(L.bitnet_tp_area_create(nbytes, ctypes.byref(area), handle))
            self._area = area
            handles = [None] * world
            if not absent_peers:
                dist.all_gather_object(handles, handle.raw, group=group)
            self._stand_ins = []
            for r in range(world):
                if r == rank:
                    areas[r] = area.value
                elif absent_peers:
                    p, h2 = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                    _lib.check(L.bitnet_tp_area_create(nbytes, ctypes.byref(p), h2))
                    self._stand_ins.append(p)
                    areas[r] = p.value
                else:
                    p = ctypes.c_void_p()
                    _lib.check(L.bitnet_tp_area_open(handles[r], ctypes.byref(p)))
                    self._peers.append(p)
                    areas[r] = p.value
        layers = (_DecoderLayer * a.n_layers)()
        self.rope = dec.rope[:max_seq_len].contiguous()
        for i, (lay, (ck, cv)) in enumerate(zip(dec.layers, self.cache)):
            S = layers[i]
            S.wqkv, S.wo, S.w13, S.w2 = (lay["wqkv"].weight.data_ptr(), lay["wo"].weight.data_ptr(),
                                         lay["w13"].weight.data_ptr(), lay["w2"].weight.data_ptr())
            S.s_q, S.s_k, S.s_v = (float(x) for x in lay["wqkv"].scale.tolist())
            S.s_o = float(lay["wo"].scale[0])
            S.s_1, S.s_3 = (float(x) for x in lay["w13"].scale.tolist())
            S.s_2 = float(lay["w2"].scale[0])
            S.attention_norm = lay["attention_norm"].weight.data_ptr()
            S.attn_sub_norm = lay["attn_sub_norm"].weight.data_ptr()
            S.ffn_norm = lay["ffn_norm"].weight.data_ptr()
            S.ffn_sub_norm = lay["ffn_sub_norm"].weight.data_ptr()
            S.cache_k, S.cache_v = ck.data_ptr(), cv.data_ptr()
        self.handle = L.bitnet_decoder_create_tp(ctypes.byref(cfg), layers, dec.emb.data_ptr(),
                                                 dec.final_norm.weight.data_ptr(), dec.out_w.data_ptr(),
                                                 self.rope.data_ptr(), rank, world, areas)
        if not self.handle:
            _lib.check()
            raise _lib.BitnetError("bitnet_decoder_create_tp failed")
        if wait_limit_ms is not None:
            _lib.check(L.bitnet_decoder_set_wait_limit(self.handle, float(wait_limit_ms)))
        if world > 1 and not absent_peers:
            dist.barrier(group=group)       # every rank has mapped every area before anybody steps
        self.world = world
        self._lib = _lib
        self.kernels_per_step = L.bitnet_decoder_kernels_per_step(self.handle)

    def step(self, logits: Optional[torch.Tensor] = None):
        """Enqueues one decode step on the current stream (may be captured in a CUDA graph)."""
        _lib = self._lib
        _lib.check(_lib.lib.bitnet_decoder_step(self.handle, _lib.ptr(self.tokens), _lib.ptr(self.pos), _lib.ptr(self.out),
                                                _lib.ptr(logits), _lib.stream_ptr()))

    def error_flag(self) -> int:
        return self._lib.lib.bitnet_decoder_error_flag(self.handle)

    def close(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            self._lib.lib.bitnet_decoder_destroy(h)
        for p in getattr(self, "_peers", []):
            self._lib.lib.bitnet_tp_area_close(p)
        self._peers = []
        for p in getattr(self, "_stand_ins", []):
            self._lib.lib.bitnet_tp_area_free(p)
        self._stand_ins = []
        if getattr(self, "_area", None):
            self._lib.lib.bitnet_tp_area_free(self._area)
            self._area = None

    def __del__(self):
        if getattr(self, "_lib", None) is not None and getattr(self._lib, "lib", None) is not None:
            self.close()
