"""Greedy generation loop over the decoder, with the decode step captured in a CUDA graph.

Thin counterpart of the reference's gpu/generate.py (FastGen, :36-304): a prefill pass over
the prompt, then one graph replay per generated token.  The reference keeps two models
(bf16 prefill, int2 decode); here both phases run the same W2A8 kernels.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .model import Transformer, make_cache


class Generator:
    def __init__(self, model: Transformer, batch: int, max_seq_len: int, use_cuda_graph: bool = True):
        self.model, self.batch, self.max_seq_len = model, batch, max_seq_len
        dev = model.tok_embeddings.weight.device
        self.device = dev
        self.cache = make_cache(model.args, batch, max_seq_len, device=dev)
        self.tokens = torch.zeros((batch, 1), dtype=torch.int64, device=dev)     # input of the next step
        self.pos = torch.zeros((batch,), dtype=torch.int64, device=dev)         # tokens already cached
        self.out = torch.zeros((batch,), dtype=torch.int64, device=dev)         # result of the last step
        self.host_in = torch.zeros((batch, 1), dtype=torch.int64).pin_memory()
        self.host_out = torch.zeros((batch,), dtype=torch.int64).pin_memory()
        self.use_cuda_graph = use_cuda_graph
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.stream = torch.cuda.Stream(device=dev)

    def _step(self):
        logits = self.model(self.tokens, self.pos, self.cache)
        nxt = logits[:, -1].argmax(-1)
        self.out.copy_(nxt)
        self.tokens.copy_(nxt[:, None])
        self.pos.add_(1)

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor):
        """prompt int64 [B, T] on the device.  Fills the cache and leaves the first generated
        token as the input of the next decode step."""
        B, T = prompt.shape
        assert B == self.batch and T < self.max_seq_len
        self.pos.zero_()
        logits = self.model(prompt, self.pos, self.cache, kv_len=T)
        nxt = logits[:, -1].argmax(-1)
        self.out.copy_(nxt)
        self.tokens.copy_(nxt[:, None])
        self.pos.fill_(T)
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
        torch.cuda.synchronize()
        self.tokens.copy_(saved[0]); self.pos.copy_(saved[1]); self.out.copy_(saved[2])
        torch.cuda.synchronize()

    @torch.no_grad()
    def decode_step(self):
        """One token for every sequence, device resident (input = previous output)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step()

    @torch.no_grad()
    def decode_step_host(self, tokens_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token with host buffers on both sides: copies the input ids from pinned host
        memory, runs the step, copies the chosen ids back and waits for them."""
        with torch.cuda.stream(self.stream):
            if tokens_host is not None:
                self.host_in.copy_(tokens_host)
            self.tokens.copy_(self.host_in, non_blocking=True)
            self.decode_step()
            self.host_out.copy_(self.out, non_blocking=True)
            self.stream.synchronize()
        return self.host_out

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int) -> torch.Tensor:
        """Greedy decode; returns int64 [B, n_new] (first column = the token the prefill chose)."""
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
