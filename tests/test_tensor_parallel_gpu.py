"""Tensor parallel on real GPUs: two ranks over NCCL must reproduce the single-GPU logits bit
for bit (needs two B200s; skipped otherwise)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["BITNET_ROOT"])
from bitnet_b200.model import preset
from bitnet_b200.tensor_parallel import TPDecoder
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
args = preset("8b", n_layers=2, vocab_size=4096)
def run(dec):
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, args.vocab_size, (2, 9), generator=g).cuda()
    cache = dec.make_cache(2, 64)
    pos = torch.zeros(2, dtype=torch.int64, device="cuda")
    h = dec.hidden(prompt, pos, cache, kv_len=9)
    outs = [dec.logits(h)]
    tok = dec.greedy(h).view(2, 9)[:, -1:]
    for s in range(5):
        h = dec.hidden(tok, pos + 9 + s, cache)
        outs.append(dec.logits(h))
        tok = dec.greedy(h).view(2, 1)
    return torch.cat([o.reshape(-1) for o in outs]), tok
dec_tp = TPDecoder(args, 7, rank, world, "cuda", backend="kernel", max_seq_len=64)
tp = run(dec_tp)
# the same decode steps replayed from a CUDA graph (collectives captured) give the same tokens
from bitnet_b200.tensor_parallel import GraphedStep
def greedy_loop(graph):
    g = torch.Generator().manual_seed(6)
    tok = torch.randint(0, args.vocab_size, (2, 1), generator=g).cuda()
    pos = torch.full((2,), 3, dtype=torch.int64, device="cuda")
    cache = dec_tp.make_cache(2, 64)
    outs = []
    step = GraphedStep(dec_tp, tok, pos, cache) if graph else None
    for s in range(6):
        if graph:
            step.replay()
            torch.cuda.synchronize()
            outs.append(step.out.clone())
        else:
            nxt = dec_tp.decode_step(tok, pos, cache)
            tok = nxt.view(2, 1)
            pos += 1
            outs.append(nxt.clone())
    return torch.stack(outs)
assert torch.equal(greedy_loop(True), greedy_loop(False))

# the in-library step (peer-memory exchange inside the kernels, no collective call in the step):
# logits and tokens bit-identical to the same step on one rank, eagerly and replayed from a graph
from bitnet_b200.tensor_parallel import TPFusedStep
def fused_loop(dec, graph, steps=12):
    st = TPFusedStep(dec, 2, 64)
    g = torch.Generator().manual_seed(8)
    st.tokens.copy_(torch.randint(0, args.vocab_size, (2, 1), generator=g).cuda())
    st.pos.zero_()
    Vl = args.vocab_size // dec.world
    logits = torch.zeros((2, Vl), dtype=torch.float32, device="cuda")
    toks, lgs = [], []
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        if graph:
            st.step(logits); stream.synchronize()
            st.tokens.copy_(torch.randint(0, args.vocab_size, (2, 1), generator=torch.Generator().manual_seed(8)).cuda()); st.pos.zero_()
            for c in st.cache:
                c[0].zero_(); c[1].zero_()
            cg = torch.cuda.CUDAGraph()
            stream.synchronize()
            if dec.world > 1: dist.barrier()
            with torch.cuda.graph(cg, stream=stream):
                st.step(logits)
        for s in range(steps):
            if graph: cg.replay()
            else: st.step(logits)
            stream.synchronize()
            toks.append(st.out.clone()); lgs.append(logits.clone())
    assert st.error_flag() == 0
    out = torch.stack(toks), torch.stack(lgs)
    if dec.world > 1: dist.barrier()
    st.close()
    return out
t2, l2 = fused_loop(dec_tp, False)
t2g, l2g = fused_loop(dec_tp, True)
assert torch.equal(t2, t2g) and torch.equal(l2, l2g)
gathered = [torch.zeros_like(l2) for _ in range(world)]
dist.all_gather(gathered, l2)
if rank == 0:
    t1, l1 = fused_loop(TPDecoder(args, 7, 0, 1, "cuda", backend="kernel", max_seq_len=64), False)
    assert torch.equal(t2, t1), (t2, t1)
    assert torch.equal(torch.cat(gathered, dim=-1), l1), float((torch.cat(gathered, dim=-1) - l1).abs().max())
    print("TP_FUSED_OK")
if rank == 0:
    one = run(TPDecoder(args, 7, 0, 1, "cuda", backend="kernel", max_seq_len=64))
    assert torch.equal(tp[0], one[0]), float((tp[0] - one[0]).abs().max())
    assert torch.equal(tp[1], one[1])
    print("TP_OK")
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_nccl_equals_single_gpu(tmp_path):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, BITNET_ROOT=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "TP_OK" in r.stdout and "TP_FUSED_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_bounded_wait_for_an_absent_rank_returns_an_error_status():
    """A tensor-parallel step whose peer never contributes must end by itself: the kernels' waits
    for the other rank run out (here after 2 ms each), the decoder's error word holds code 6, the
    call returns, and the GPU keeps working (a single-GPU decoder gives its usual bits)."""
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import build_synthetic, preset
    from bitnet_b200.tensor_parallel import TPDecoder, TPFusedStep

    args = preset("tiny", n_heads=4, n_kv_heads=2, ffn_dim=512)
    dec = TPDecoder(args, 3, 0, 2, "cuda", backend="kernel", max_seq_len=32)    # rank 0 of 2; rank 1 does not exist
    st = TPFusedStep(dec, 1, 32, wait_limit_ms=2.0, absent_peers=True)
    st.tokens.fill_(5)
    st.step()
    torch.cuda.synchronize()
    assert st.error_flag() == 6
    st.close()
    model = build_synthetic(preset("tiny"), seed=5, device="cuda", max_seq_len=32)
    prompt = torch.randint(0, 512, (1, 6), device="cuda", generator=torch.Generator("cuda").manual_seed(2))
    a = Generator(model, 1, 32, use_cuda_graph=False, fused=True).generate(prompt, 8)
    b = Generator(model, 1, 32, use_cuda_graph=True, fused=True).generate(prompt, 8)
    assert torch.equal(a, b)


def test_one_rank_batched_decode_fused_calls_equal_per_op_path():
    """On one rank, batches of 16 or more take the library's fused calls (matmul + rescale,
    residual + norm + quantisation behind wo and w2): same hidden states and tokens, bit for bit,
    as the per-op path that the multi-rank decoder uses."""
    from bitnet_b200.model import preset
    from bitnet_b200.tensor_parallel import TPDecoder

    args = preset("tiny", n_heads=4, n_kv_heads=2, ffn_dim=512, n_layers=3)
    dec = TPDecoder(args, 9, 0, 1, "cuda", backend="kernel", max_seq_len=64)
    outs = []
    for fused in (True, False):
        dec.fused_one_rank = fused
        cache = dec.make_cache(24, 64)
        g = torch.Generator("cuda").manual_seed(4)
        tok = torch.randint(0, args.vocab_size, (24, 1), device="cuda", generator=g)
        pos = torch.zeros(24, dtype=torch.int64, device="cuda")
        hs = []
        for s in range(5):
            h = dec.hidden(tok, pos + s, cache)
            hs.append(h.clone())
            tok = dec.greedy(h).view(24, 1)
        outs.append(torch.stack(hs))
    dec.fused_one_rank = True
    assert torch.equal(outs[0], outs[1])
