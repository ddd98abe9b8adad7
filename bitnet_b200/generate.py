"""Greedy generation loop over the decoder, with the decode step captured in a CUDA graph.

Thin counterpart of the reference's gpu/generate.py (FastGen, :36-304): a prefill pass over
the prompt, then one graph replay per generated token.  The reference keeps two models
(bf16 prefill, int2 decode); here both phases run the same W2A8 kernels.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _lib, ops
from .model import BitLinearKernel, Transformer, make_cache


class _DecoderConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("dim", "n_layers", "n_heads", "n_kv_heads", "head_dim", "ffn_dim",
                                            "vocab_size")] + [("norm_eps", ctypes.c_float), ("batch", ctypes.c_int),
                                                              ("max_seq_len", ctypes.c_int)]


class _DecoderLayer(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("wqkv", "wo", "w13", "w2")] +
                [(n, ctypes.c_float) for n in ("s_q", "s_k", "s_v", "s_o", "s_1", "s_3", "s_2")] +
                [(n, ctypes.c_void_p) for n in ("attention_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm",
                                                "cache_k", "cache_v")])


class FusedDecoder:
    """One decode step for a batch of at most 8 through `bitnet_decoder_step`: the whole
    step runs inside the library (see include/bitnet_b200.h) as a chain of fused kernels."""

    MAX_BATCH = 8

    def __init__(self, model: Transformer, cache, batch: int, max_seq_len: int):
        a = model.args
        assert a.use_kernel and 1 <= batch <= self.MAX_BATCH
        assert model.rope is not None and model.rope.shape[0] >= max_seq_len
        cfg = _DecoderConfig(a.dim, a.n_layers, a.n_heads, a.n_kv_heads, a.head_dim, a.ffn_dim, a.vocab_size,
                             a.norm_eps, batch, max_seq_len)
        layers = (_DecoderLayer * a.n_layers)()
        self._keep = [model, cache]
        for i, (layer, (ck, cv)) in enumerate(zip(model.layers, cache)):
            att, ff = layer.attention, layer.feed_forward
            for lin in (att.wqkv, att.wo, ff.w13, ff.w2):
                assert isinstance(lin, BitLinearKernel)
            assert ck.is_contiguous() and cv.is_contiguous() and tuple(ck.shape) == (batch, max_seq_len, a.n_kv_heads,
                                                                                   a.head_dim)
            sq, sk, sv = (float(x) for x in att.wqkv.scale_f32.tolist())
            s1, s3 = (float(x) for x in ff.w13.scale_f32.tolist())
            L = layers[i]
            L.wqkv, L.wo, L.w13, L.w2 = (att.wqkv.weight.data_ptr(), att.wo.weight.data_ptr(),
                                         ff.w13.weight.data_ptr(), ff.w2.weight.data_ptr())
            L.s_q, L.s_k, L.s_v, L.s_o, L.s_1, L.s_3, L.s_2 = (sq, sk, sv, float(att.wo.scale_f32[0]), s1, s3,
                                                                float(ff.w2.scale_f32[0]))
            L.attention_norm = layer.attention_norm.weight.data_ptr()
            L.attn_sub_norm = att.attn_sub_norm.weight.data_ptr()
            L.ffn_norm = layer.ffn_norm.weight.data_ptr()
            L.ffn_sub_norm = ff.ffn_sub_norm.weight.data_ptr()
            L.cache_k, L.cache_v = ck.data_ptr(), cv.data_ptr()
        self.rope = model.rope[:max_seq_len].contiguous()
        self.handle = _lib.lib.bitnet_decoder_create(ctypes.byref(cfg), layers, model.tok_embeddings.weight.data_ptr(),
                                                     model.norm.weight.data_ptr(), model.output.weight.data_ptr(),
                                                     self.rope.data_ptr())
        if not self.handle:
            _lib.check()
            raise _lib.BitnetError("bitnet_decoder_create failed")
        self.kernels_per_step = _lib.lib.bitnet_decoder_kernels_per_step(self.handle)

    def step(self, tokens: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, logits: Optional[torch.Tensor] = None):
        """tokens int64 [B] (or [B,1]), pos int64 [B], out int64 [B] on the device; enqueued on the current stream."""
        _lib.check(_lib.lib.bitnet_decoder_step(self.handle, _lib.ptr(tokens), _lib.ptr(pos), _lib.ptr(out),
                                                _lib.ptr(logits), _lib.stream_ptr()))

    def step_sync(self, tokens: torch.Tensor, pos: torch.Tensor, out: torch.Tensor):
        """`step` and a wait for the current stream in one library call; tokens and out may be
        pinned host tensors (the kernels read and write them in place)."""
        _lib.check(_lib.lib.bitnet_decoder_step_sync(self.handle, _lib.ptr(tokens), _lib.ptr(pos), _lib.ptr(out), None,
                                                     _lib.stream_ptr()))

    def bench_linears(self, tokens: torch.Tensor):
        """Enqueues only the fused BitLinear kernels of every layer (a measurement aid)."""
        _lib.check(_lib.lib.bitnet_decoder_bench_linears(self.handle, _lib.ptr(tokens), _lib.stream_ptr()))

    def error_flag(self) -> int:
        return _lib.lib.bitnet_decoder_error_flag(self.handle)

    def clear_error(self):
        _lib.check(_lib.lib.bitnet_decoder_clear_error(self.handle))

    def set_attention_tap(self, buffer: Optional[torch.Tensor]):
        """bf16 [n_layers, batch, dim] that every attention kernel of later steps also writes
        its output to (None switches it off): lets a checker follow the step layer by layer."""
        self._tap = buffer
        _lib.check(_lib.lib.bitnet_decoder_set_attention_tap(self.handle, _lib.ptr(buffer)))

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and _lib is not None and getattr(_lib, "lib", None) is not None:   # may run at interpreter exit
            _lib.lib.bitnet_decoder_destroy(h)


class Generator:
    AUTO_FUSED_MAX_BATCH = 4

    def __init__(self, model: Transformer, batch: int, max_seq_len: int, use_cuda_graph: bool = True,
                 fused: Optional[bool] = None, temperature: float = 0.0, top_p: float = 1.0, seed: int = 0):
        """fused=None picks the in-library decode step where it is the faster path (kernel model,
        batch <= AUTO_FUSED_MAX_BATCH); fused=True asks for it up to batch 8.
        temperature > 0 draws every next token from softmax(logits / temperature) cut at top_p
        (gpu/generate.py:250-257) on the device, reproducibly for a given seed; 0 is greedy."""
        self.model, self.batch, self.max_seq_len = model, batch, max_seq_len
        dev = model.tok_embeddings.weight.device
        self.device = dev
        self.temperature, self.top_p, self.seed = float(temperature), float(top_p), int(seed)
        self.sampling = self.temperature > 0.0
        self.logits = (torch.zeros((batch, model.args.vocab_size), dtype=torch.float32, device=dev)
                       if self.sampling else None)
        self.cache = make_cache(model.args, batch, max_seq_len, device=dev)
        self.tokens = torch.zeros((batch, 1), dtype=torch.int64, device=dev)     # input of the next step
        self.pos = torch.zeros((batch,), dtype=torch.int64, device=dev)         # tokens already cached
        self.out = torch.zeros((batch,), dtype=torch.int64, device=dev)         # result of the last step
        self.host_in = torch.zeros((batch, 1), dtype=torch.int64).pin_memory()
        self.host_out = torch.zeros((batch,), dtype=torch.int64).pin_memory()
        self.use_cuda_graph = use_cuda_graph
        self._pos_host = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_host: Optional[torch.cuda.CUDAGraph] = None
        self._host_state = False
        self.stream = torch.cuda.Stream(device=dev)
        can_fuse = model.args.use_kernel and batch <= FusedDecoder.MAX_BATCH
        if fused and not can_fuse:
            raise ValueError("the fused decode chain needs the kernel model and batch <= 8")
        self.fused: Optional[FusedDecoder] = None
        # fused=None: the in-library step where it is the faster path.  Its kernels repeat the
        # activation prologue of every token in every CTA, so at eight sequences one launch per
        # operation wins (measured on B200, 2B architecture, ms per step in-library vs per
        # operation: batch 1: 0.82 vs 1.69; 2: 1.12 vs 1.71; 4: 1.55 vs 1.79; 8: 2.42 vs 1.92).
        if can_fuse and (fused or (fused is None and batch <= self.AUTO_FUSED_MAX_BATCH)):
            if model.rope is None or model.rope.shape[0] < max_seq_len:
                from .model import rope_table
                model.rope = rope_table(model.args.head_dim, max(max_seq_len, model.max_seq_len),
                                        model.args.rope_theta, dev)
            try:
                self.fused = FusedDecoder(model, self.cache, batch, max_seq_len)
            except _lib.BitnetError:
                # e.g. batch x hidden size beyond the fused kernels' shared memory: the
                # op-by-op path (same kernels, one launch per operation) takes over
                if fused:
                    raise

    def _draw(self, logits: torch.Tensor, out: torch.Tensor, tokens: Optional[torch.Tensor]):
        """The sampled ids for f32 logits [B, V]; the random numbers are a function of the seed,
        the sequence and self.pos (already advanced), so a replayed graph draws afresh each step."""
        ops.sample_top_p(logits, self.temperature, self.top_p, self.seed, pos=self.pos, out=out, tokens=tokens)

    def _step(self):
        if self.fused is not None:
            self.fused.step(self.tokens, self.pos, self.out, self.logits)
            if self.sampling:
                self._draw(self.logits, self.out, self.tokens)
            return
        logits = self.model(self.tokens, self.pos, self.cache)
        self.pos.add_(1)
        if self.sampling:
            self.logits.copy_(logits[:, -1])
            self._draw(self.logits, self.out, self.tokens)
            return
        nxt = logits[:, -1].argmax(-1)
        self.out.copy_(nxt)
        self.tokens.copy_(nxt[:, None])

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor):
        """prompt int64 [B, T] on the device.  Fills the cache and leaves the first generated
        token as the input of the next decode step."""
        B, T = prompt.shape
        assert B == self.batch and T < self.max_seq_len
        self._pos_host = T                      # host mirror of the positions (all sequences advance together)
        self.pos.zero_()
        logits = self.model(prompt, self.pos, self.cache, kv_len=T, last_only=True)
        self.pos.fill_(T)
        if self.sampling:
            self.logits.copy_(logits[:, -1])
            self._draw(self.logits, self.out, self.tokens)
            return self.out.clone()
        nxt = logits[:, -1].argmax(-1)
        self.out.copy_(nxt)
        self.tokens.copy_(nxt[:, None])
        return nxt

    @torch.no_grad()
    def capture(self):
        """Warms the decode step up on a side stream, then captures it (the order the
        reference uses, gpu/generate.py:181-203).  State is restored afterwards."""
        if not self.use_cuda_graph or self.graph is not None:
            return
        saved = (self.tokens.clone(), self.pos.clone(), self.out.clone())
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            self._step()
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self._step()
            # The same step for callers that hand over and read back ids in host memory.  The
            # in-library step reads the ids from, and writes the chosen ids to, the pinned host
            # buffers directly (they are addressable from the device), so no copy engine sits
            # between the host and the kernel; otherwise the two copies are part of the graph.
            self.graph_host = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_host, stream=self.stream):
                if self.fused is not None:
                    self.fused.step(self.host_in, self.pos, self.host_out, self.logits)
                    if self.sampling:
                        self._draw(self.logits, self.host_out, self.host_in)
                else:
                    self.tokens.copy_(self.host_in, non_blocking=True)
                    self._step()
                    self.host_out.copy_(self.out, non_blocking=True)
        torch.cuda.synchronize()
        self.tokens.copy_(saved[0]); self.pos.copy_(saved[1]); self.out.copy_(saved[2])
        torch.cuda.synchronize()

    def _advance(self):
        """Refuses a step that would write beyond the KV cache (the kernels would flag it and
        skip the append; the host knows earlier)."""
        if self._pos_host >= self.max_seq_len:
            raise ValueError(f"decode step at position {self._pos_host} exceeds max_seq_len {self.max_seq_len}")
        self._pos_host += 1

    @torch.no_grad()
    def decode_step(self):
        """One token for every sequence, device resident (input = previous output)."""
        self._advance()
        if self._host_state:   # the last steps ran on the host buffers: take their state over
            self.tokens.copy_(self.host_in)
            self.out.copy_(self.host_out)
            self._host_state = False
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step()

    @torch.no_grad()
    def decode_step_host(self, tokens_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token with host buffers on both sides: takes the input ids from pinned host
        memory (tokens_host, or the ids the previous step chose), runs the step, and returns
        the chosen ids in pinned host memory once they have arrived."""
        self._advance()
        with torch.cuda.stream(self.stream):
            if tokens_host is not None:
                self.host_in.copy_(tokens_host)
            elif not self._host_state:
                self.host_in.copy_(self.tokens)
            if self.graph_host is not None:
                self.graph_host.replay()
                self._host_state = self.fused is not None   # next input and result live in host_in / host_out
            else:
                self.tokens.copy_(self.host_in, non_blocking=True)
                self._pos_host -= 1             # decode_step counts the step itself
                self.decode_step()
                self.host_out.copy_(self.out, non_blocking=True)
            self.stream.synchronize()
        return self.host_out

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int) -> torch.Tensor:
        """Greedy (or, with a temperature, sampled) decode; returns int64 [B, n_new] (first column =
        the token the prefill chose)."""
        first = self.prefill(prompt)
        self.capture()
        outs: List[torch.Tensor] = [first.clone()]
        with torch.cuda.stream(self.stream):
            self.stream.wait_stream(torch.cuda.current_stream())
            for _ in range(n_new - 1):
                self.decode_step()
                outs.append(self.out.clone())
            self.stream.synchronize()
        return torch.stack(outs, dim=1)
