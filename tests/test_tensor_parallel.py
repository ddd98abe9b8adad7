"""Tensor-parallel decoder: tp=2 over gloo on CPU must equal tp=1 bit for bit (the partial
sums that cross ranks are exact integers), and tp=1 on the GPU must equal the plain model."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from bitnet_b200.model import preset

ARGS = dict(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=512, ffn_dim=384)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_tp1(backend, device, seed=3, steps=3):
    from bitnet_b200.tensor_parallel import TPDecoder

    args = preset("tiny", **ARGS)
    dec = TPDecoder(args, seed, 0, 1, device, backend=backend, max_seq_len=32)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, args.vocab_size, (2, 6), generator=g).to(device)
    cache = dec.make_cache(2, 32)
    pos = torch.zeros(2, dtype=torch.int64, device=device)
    h = dec.hidden(prompt, pos, cache, kv_len=6)
    outs = [h.float().cpu(), dec.logits(h).cpu()]
    tok = dec.greedy(h).view(2, 6)[:, -1:]
    toks = [tok.cpu()]
    for s in range(steps):
        tok = dec.decode_step(tok, pos + 6 + s, cache).view(2, 1)
        toks.append(tok.cpu())
    return outs, torch.cat(toks, dim=1)


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from bitnet_b200.tensor_parallel import TPDecoder

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        args = preset("tiny", **ARGS)
        dec = TPDecoder(args, 3, rank, world, "cpu", backend="torch", max_seq_len=32)
        g = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, args.vocab_size, (2, 6), generator=g)
        cache = dec.make_cache(2, 32)
        pos = torch.zeros(2, dtype=torch.int64)
        h = dec.hidden(prompt, pos, cache, kv_len=6)
        lg = dec.logits(h)
        tok = dec.greedy(h).view(2, 6)[:, -1:]
        toks = [tok]
        for s in range(3):
            tok = dec.decode_step(tok, pos + 6 + s, cache).view(2, 1)
            toks.append(tok)
        if rank == 0:
            q.put((h.float(), lg, torch.cat(toks, dim=1)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tp2_gloo_equals_tp1_bit_for_bit():
    (h1, lg1), toks1 = _run_tp1("torch", "cpu")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    import queue
    import time

    deadline, result = time.time() + 240, None
    while result is None and time.time() < deadline:
        try:
            result = q.get(timeout=2)
        except queue.Empty:
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    assert result is not None and all(p.exitcode == 0 for p in procs)
    h2, lg2, toks2 = result
    assert torch.equal(h1, h2)            # hidden states: identical bits
    assert torch.equal(lg1, lg2)
    assert torch.equal(toks1, toks2)


@pytest.mark.gpu
def test_tp1_kernel_backend_equals_plain_model():
    from bitnet_b200.model import build_synthetic, make_cache
    from bitnet_b200.tensor_parallel import TPDecoder

    args = preset("tiny", **ARGS)
    model = build_synthetic(args, seed=3, device="cuda", max_seq_len=32)
    dec = TPDecoder(args, 3, 0, 1, "cuda", backend="kernel", max_seq_len=32)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, args.vocab_size, (2, 6), generator=g).cuda()
    pos = torch.zeros(2, dtype=torch.int64, device="cuda")
    c1, c2 = make_cache(args, 2, 32, "cuda"), dec.make_cache(2, 32)
    want = model(prompt, pos, c1, kv_len=6)
    got = dec.logits(dec.hidden(prompt, pos, c2, kv_len=6)).view(2, 6, -1)
    assert torch.equal(got, want)
    tok = want[:, -1].argmax(-1)[:, None]
    for s in range(4):                    # single-token steps go through the attention kernel
        p = pos + 6 + s
        w = model(tok, p, c1)[:, -1]
        h = dec.hidden(tok, p, c2)
        assert torch.equal(dec.logits(h), w)
        tok = w.argmax(-1)[:, None]
        assert torch.equal(dec.greedy(h), tok[:, 0])
