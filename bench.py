#!/usr/bin/env python
"""Benchmark of the W2A8 BitLinear decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the BitNet-b1.58-2B-4T architecture, random-init from a seed, batch 1,
128 uniform-random prompt tokens, then greedy decode; a "step" is one decode step (one new
token per sequence) through the whole model.  One JSON line is printed by rank 0.

* `value`    - decode tokens/s with everything resident on the device (the step is a CUDA
               graph that feeds its own output back as the next input).
* `e2e`      - the same through the public API with host buffers: every step copies the
               input token ids from pinned host memory and copies the chosen ids back.
* `roofline` - the BitLinear matmul kernel alone: all of the model's BitLinear launches of
               one step (distinct weights, larger than L2) timed back to back with CUDA
               events; achieved = packed weight bytes per launch / mean launch time.
* `cpu_baseline` - the reference's own I2_S CPU kernel (compiled from its source, or the C
               port when that is absent) on this machine's host cores, BitLinear layers only.

With N > 1 every rank runs an independent replica of the same workload (weak scaling; the
2B architecture has 5 KV heads, which no tensor-parallel degree of 2, 4 or 8 divides) and
the time is the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 128
SEED = 20240611


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="2b", help="architecture preset (2b, 3b, 8b, 100b)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--engine", choices=["auto", "chain", "ops"], default="auto",
                    help="decode step (batch <= 8) as the in-library chain of fused kernels, or whichever path the "
                         "generator picks for the batch (auto); ops = one launch per operation (the path of batches above 8)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the kernel sweep and the batch-64 decode")
    ap.add_argument("--sweep-only", default="", metavar="N,K,M",
                    help="run only the isolated BitLinear call for one shape and token count (for profilers) and exit")
    ap.add_argument("--tp", action="store_true",
                    help="shard one model tensor-parallel over the ranks (strong scaling) instead of replicas; "
                         "needs head counts divisible by the rank count (8b, 100b presets)")
    ap.add_argument("--no-graph", action="store_true", help="with --tp: issue the step op by op instead of replaying a graph")
    ap.add_argument("--graph", action="store_true",
                    help="with --tp on several ranks: replay the step (collectives included) from a CUDA graph; the "
                         "default there is op by op")
    ap.add_argument("--layers", type=int, default=0, help="use only the first LAYERS layers (0 = all): a small case for profilers, or with --tp")
    ap.add_argument("--context", type=int, default=PROMPT_LEN, help="tokens in the KV cache when decode starts (with --tp)")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = [r.strip().split(", ") for r in open(self.tmp.name).read().splitlines() if r.strip()]
        os.unlink(self.tmp.name)
        rows = [r for r in rows if len(r) >= 9]
        if not rows:
            return out
        sm = [float(r[1]) for r in rows]
        power = [float(r[3]) for r in rows if r[3].replace(".", "").isdigit()]
        # samples under load: the upper half by power draw (idle samples bracket the timed region)
        if power and len(power) == len(sm):
            thr = statistics.median(power)
            loaded = [c for c, p in zip(sm, power) if p >= thr] or sm
        else:
            loaded = sm
        reasons = []
        for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                          ("sw_power_cap", 8)):
            if any(r[col].strip().lower() == "active" for r in rows):
                reasons.append(name)
        out.update(sm_mhz=statistics.median(loaded), sm_max_mhz=float(rows[0][2]), reasons=reasons,
                   samples=len(rows), power_w_max=max(power) if power else None)
        return out


# ----------------------------------------------------------------------------------------
# the reference's CPU kernel on the host cores
# ----------------------------------------------------------------------------------------
def bitlinear_shapes(args_model):
    d, f, hd = args_model.dim, args_model.ffn_dim, args_model.head_dim
    return [((args_model.n_heads + 2 * args_model.n_kv_heads) * hd, d), (d, args_model.n_heads * hd), (2 * f, d),
            (d, f)]


def cpu_i2s_tokens_per_s(args_model, batch: int, steps: int, warmup: int, layers_sampled: int):
    """Times the BitLinear layers of `layers_sampled` layers (distinct I2_S weights, so they
    stream from DRAM as they would in a full model) with the reference's compiled kernel on
    all host threads; returns (tokens/s extrapolated to all layers, info dict)."""
    import numpy as np

    from oracle import build_oracle
    from oracle import np_oracle as O

    ref_path = build_oracle.build_ref()
    if ref_path:
        lib, kind = O.RefLib(ref_path), "reference"
    else:
        lib, kind = O.PortLib(build_oracle.build_port()), "port"
    # every core this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    rng = np.random.default_rng(SEED)
    # bytes whose four 2-bit fields are all in {0,1,2}: valid I2_S codes, ternary weights
    valid = np.array([a << 6 | b << 4 | c << 2 | d for a in range(3) for b in range(3) for c in range(3)
                      for d in range(3)], dtype=np.uint8)
    shapes = [s for s in bitlinear_shapes(args_model) if s[1] % 128 == 0]
    mats = []
    for _ in range(layers_sampled):
        for n, k in shapes:
            mats.append((valid[rng.integers(0, 81, size=n * k // 4 + 32)], n, k))
    acts = {k: rng.integers(-127, 128, size=(batch, k), dtype=np.int8) for _, k in shapes}

    def one_pass():
        t = 0.0
        for buf, n, k in mats:
            t += lib.gemm_time(buf, acts[k], n, k, threads, 1)
        return t

    for _ in range(warmup):
        one_pass()
    times = [one_pass() for _ in range(steps)]
    per_layer = (sum(times) / len(times)) / layers_sampled
    tok_s = batch / (per_layer * args_model.n_layers)
    info = {"kind": kind, "cores": threads,
            "sample": f"BitLinear layers only: {layers_sampled} of {args_model.n_layers} layers x {len(shapes)} "
                      f"I2_S matmuls at M={batch}, distinct weights, {steps} passes, extrapolated to all layers; "
                      "attention, norms and the bf16 output projection are not included (the reference's "
                      "llama.cpp runtime is not vendored)"}
    return tok_s, info, sum(times) / len(times)


def run_reference(a, args_model):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = min(args_model.n_layers, 8)
    t0 = time.time()
    tok_s, info, step_s = cpu_i2s_tokens_per_s(args_model, a.batch, a.steps, a.warmup, layers)
    line = {
        "impl": "reference", "metric": f"BitNet-{a.workload.upper()} decode tok/s (bs{a.batch})", "value": tok_s,
        "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": 1e3 * a.batch / tok_s, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x 2-bit ternary -> int32", "data": "synthetic",
        "config": {"workload": f"{a.workload} architecture, random ternary weights, batch {a.batch}, decode step",
                   "batch": a.batch},
        "cpu_baseline": dict(info, value=tok_s, unit="tok/s"),
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.time() - t0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
# extra measurements reported beside the headline (rank 0, one GPU)
# ----------------------------------------------------------------------------------------
def kernel_sweep(dev, peak_gbs, shapes=None, ms=None):
    """The isolated BitLinear call over the 2B shapes and M in {1..2048}: quantised
    activations in, bf16 out, through bitnet_linear_w2a8; distinct weight buffers (> 2 x L2)
    cycled inside a CUDA graph, time per launch from CUDA events."""
    import ctypes

    import torch

    from bitnet_b200 import _lib

    L = _lib.lib
    rows = []
    g = torch.Generator(device=dev).manual_seed(1)
    stream = torch.cuda.Stream(device=dev)
    for n, k in (shapes or [(3840, 2560), (2560, 2560), (13824, 2560), (2560, 6912)]):
        nbytes = n * k // 4
        copies = max(2, int(300e6 // nbytes))
        ws = [torch.randint(-128, 127, (n, k // 4), dtype=torch.int8, device=dev, generator=g) for _ in range(copies)]
        for m in (ms or (1, 8, 32, 128, 512, 2048)):
            y = torch.randint(-127, 127, (m, k), dtype=torch.int8, device=dev, generator=g)
            a = torch.ones(m, device=dev)
            ysum = y.int().sum(-1).int()
            wsc = torch.ones(1, device=dev)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            seg = (ctypes.c_int * 1)(n)
            reps = copies if m <= 128 else max(2, copies // 8)

            def run():
                st = _lib.stream_ptr()
                for w in ws[:reps]:
                    L.bitnet_linear_w2a8(_lib.ptr(y), k, _lib.ptr(w), _lib.ptr(out), n, None, _lib.ptr(a), _lib.ptr(ysum),
                                         _lib.ptr(wsc), seg, 1, m, n, k, st)

            with torch.cuda.stream(stream):
                run()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    run()
                for _ in range(3):
                    graph.replay()
                stream.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(3):
                    graph.replay()
                e1.record(stream)
                stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (3 * reps)
            rows.append({"N": n, "K": k, "M": m, "us": round(us, 2), "weight_gbs": round(nbytes / us / 1e3, 1),
                         "hbm_frac": round(nbytes / us / 1e3 / peak_gbs, 4), "tops": round(2.0 * m * n * k / us / 1e6, 1)})
        del ws
    return rows


def decode_batch(model, args_model, dev, batch, steps, warmup):
    """Decode tokens/s at a larger batch through the op-by-op path (tcgen05 BitLinear kernel,
    library attention), captured in a CUDA graph; device-resident."""
    import torch

    from bitnet_b200.generate import Generator

    max_seq = (PROMPT_LEN + steps + warmup + 64 + 127) // 128 * 128
    gen = Generator(model, batch, max_seq)
    g = torch.Generator(device=dev).manual_seed(SEED + 5)
    prompt = torch.randint(0, args_model.vocab_size, (batch, PROMPT_LEN), generator=g, device=dev)
    gen.prefill(prompt)
    gen.capture()
    with torch.cuda.stream(gen.stream):
        for _ in range(warmup):
            gen.decode_step()
        gen.stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(gen.stream)
        for _ in range(steps):
            gen.decode_step()
        e1.record(gen.stream)
        gen.stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"batch": batch, "value": batch / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms, "steps": steps}


# ----------------------------------------------------------------------------------------
# this library on the GPU
# ----------------------------------------------------------------------------------------
def run_ours(a, args_model):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from bitnet_b200 import ops
    from bitnet_b200.generate import Generator
    from bitnet_b200.model import BitLinearKernel, build_synthetic

    dev = torch.device("cuda", local_rank)
    B, K, W = a.batch, a.steps, a.warmup
    max_seq = (PROMPT_LEN + 2 * (K + W) + 3 * W + 64 + 127) // 128 * 128
    model = build_synthetic(args_model, seed=SEED + rank, device=dev, max_seq_len=max_seq)
    if a.engine == "ops":
        gen = Generator(model, B, max_seq, fused=False)
    else:
        gen = Generator(model, B, max_seq, fused=True if (a.engine == "chain" and B <= 8) else None)
    g = torch.Generator(device=dev)
    g.manual_seed(SEED + 17 * rank)
    prompt = torch.randint(0, args_model.vocab_size, (B, PROMPT_LEN), generator=g, device=dev)
    gen.prefill(prompt)
    gen.capture()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    stream = gen.stream

    # ---- device-resident decode ---------------------------------------------------------
    with torch.cuda.stream(stream):
        for _ in range(W):
            gen.decode_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.nvtx.range_push("timed_decode")   # lets a profiler pick out the timed steps
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(K):
            gen.decode_step()
        e1.record(stream)
    barrier()
    torch.cuda.nvtx.range_pop()
    ms = max_over_ranks(e0.elapsed_time(e1))

    # ---- host in, host out --------------------------------------------------------------
    host_tok = gen.host_out.clone()
    for _ in range(W):
        host_tok = gen.decode_step_host(host_tok[:, None]).clone()
    barrier()
    with torch.cuda.stream(stream):
        e0.record(stream)
    for _ in range(K):
        host_tok = gen.decode_step_host(host_tok[:, None]).clone()
    with torch.cuda.stream(stream):
        e1.record(stream)
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))

    # ---- the BitLinear kernel alone: every BitLinear of the model, once per step ----------
    lins = [m for m in model.modules() if isinstance(m, BitLinearKernel)]
    fused = gen.fused is not None
    inputs = {}
    for lin in lins:
        if lin.in_features not in inputs:
            x = torch.randn((B, lin.in_features), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            inputs[lin.in_features] = ops.quant_input(x)
    outs = {lin.out_features: torch.empty((B, lin.out_features), dtype=torch.bfloat16, device=dev) for lin in lins}
    weight_bytes = sum(l.out_features * l.in_features // 4 for l in lins)

    def linears_once():
        if fused:                      # the fused BitLinear kernels (prologue + matmul), chained
            gen.fused.bench_linears(gen.tokens)
            return
        for lin in lins:
            y, sc, ys = inputs[lin.in_features]
            ops.linear_w2a8(y, sc, ys, lin.weight, lin.scale_f32, lin.seg_end, lin.out_features, lin.in_features)

    with torch.cuda.stream(stream):
        for _ in range(max(W, 3)):
            linears_once()
        stream.synchronize()
        gl = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gl, stream=stream):
            linears_once()
        gl.replay()
    barrier()
    reps = max(3, min(K, 20))
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            gl.replay()
        e1.record(stream)
    barrier()
    ms_lin = e0.elapsed_time(e1) / reps
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = weight_bytes / (ms_lin * 1e-3) / 1e9
    cpu = None
    if world == 1 and not a.no_cpu_baseline:
        tok_s, info, _ = cpu_i2s_tokens_per_s(args_model, B, steps=3, warmup=1, layers_sampled=min(args_model.n_layers, 4))
        cpu = dict(info, value=tok_s, unit="tok/s")
    extras = {}
    if world == 1 and not a.no_extras:
        try:
            extras["decode_bs64"] = decode_batch(model, args_model, dev, 64, steps=min(K, 16), warmup=3)
            extras["kernel_sweep"] = kernel_sweep(dev, peak)
        except Exception as exc:   # the headline stands on its own
            extras["extras_error"] = repr(exc)[:300]
    n_lin = len(lins)
    # every byte a decode step must read: packed BitLinear weights + the bf16 output projection
    step_bytes = weight_bytes + 2 * args_model.vocab_size * args_model.dim
    step_gbs = step_bytes / (ms / K * 1e-3) / 1e9
    # the BitLinear kernels of the chain on their own (prologue + matmul, no attention, no head)
    chain_linears = {"kernel": "chain_linear_kernel (prologue + W2A8 matmul + epilogue, PDL chain)" if fused else "w2a8_gemv_kernel",
                     "launches_per_step": n_lin, "bytes_per_launch": weight_bytes / n_lin,
                     "us_per_launch": 1e3 * ms_lin / n_lin, "achieved": achieved, "frac": achieved / peak,
                     # dram__bytes_read + write per launch from one ncu capture of the four 2B shapes
                     # (profiles/fused_linear_kernel_2b_m1.md), averaged as the launches are mixed
                     "traffic": 4.50e6 if (fused and a.workload == "2b" and B == 1) else None}
    roofline = dict(chain_linears, bound="hbm", peak=peak, unit="GB/s", peak_source="measured" if peaks else "fallback",
                    step_bytes=step_bytes, step_gbs=step_gbs, step_frac=step_gbs / peak)
    line = {
        "metric": f"BitNet-{a.workload.upper()} decode tok/s (bs{B})", "value": world * B * K / (ms * 1e-3),
        "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x 2-bit ternary -> int32 (bf16 elsewhere)", "data": "synthetic",
        "config": {"workload": f"{a.workload} architecture random-init (seed {SEED}), batch {B}, {PROMPT_LEN} random "
                               f"prompt tokens then greedy decode; replicas x{world}",
                   "batch": B, "prompt_len": PROMPT_LEN,
                   "engine": "kernel chain" if fused else "op by op",
                   "l2": "weights read per step (%.0f MB packed + bf16 output projection) exceed the 126 MB L2"
                         % (weight_bytes / 1e6)},
        "e2e": {"value": world * B * K / (ms_e2e * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8 * B,
                "d2h_bytes_per_step": 8 * B},
        "gpu_launches": (gen.fused.kernels_per_step if fused else 2 * n_lin) * K,
        "roofline": roofline,
        "cpu_baseline": cpu, "clocks": clocks, **extras,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_tp(a, args_model):
    """One model sharded over the ranks (bitnet_b200.tensor_parallel): column-parallel wqkv/w13,
    row-parallel wo/w2 with an all-gather and an exact int32 all-reduce each; the decode step
    (kernels and collectives) is captured in a CUDA graph (--no-graph: issued op by op), timed
    with CUDA events, maximum over ranks."""
    import torch
    import torch.distributed as dist

    from bitnet_b200.tensor_parallel import GraphedStep, TPDecoder

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # One rank: the step is replayed from a CUDA graph.  Several ranks: op by op unless --graph
    # (a two-rank graph of 2 layers replays correctly in tests/test_tensor_parallel_gpu.py, but the
    # 8-layer bench configuration did not finish on this pool, cause not found: left off by default).
    if world > 1 and not a.graph:
        a.no_graph = True
    if world > 1:
        if not a.no_graph:
            # collectives replayed from a CUDA graph: plain ring/tree algorithms (no NVLink SHARP
            # multicast objects bound to graph nodes)
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    B, K, W = a.batch, a.steps, a.warmup
    max_seq = (a.context + K + W + 8 + 127) // 128 * 128
    dec = TPDecoder(args_model, SEED, rank, world, dev, backend="kernel", max_seq_len=max_seq)
    cache = dec.make_cache(B, max_seq)
    g = torch.Generator(device=dev).manual_seed(SEED)
    for ck, cv in cache:     # a context of random keys and values stands in for a prefill
        ck[:, : a.context].copy_(torch.randn(ck[:, : a.context].shape, generator=g, device=dev).to(torch.bfloat16))
        cv[:, : a.context].copy_(torch.randn(cv[:, : a.context].shape, generator=g, device=dev).to(torch.bfloat16))
    tok = torch.randint(0, args_model.vocab_size, (B, 1), generator=g, device=dev)
    pos = torch.full((B,), a.context, dtype=torch.int64, device=dev)
    step = None if a.no_graph else GraphedStep(dec, tok, pos, cache)
    stream = step.stream if step else torch.cuda.current_stream()

    def one_step():
        nonlocal tok
        if step:
            step.replay()
        else:
            tok = dec.decode_step(tok, pos, cache).view(B, 1)
            pos.add_(1)

    with torch.cuda.stream(stream):
        for _ in range(W):
            one_step()
    # The barrier's collective runs on another stream than the step's: the device is drained
    # first, so that collectives of one communicator never overlap on two streams (their order
    # on the GPUs could then differ between the ranks).
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(K):
            one_step()
        e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        D = args_model.head_dim
        per_layer = ((args_model.n_heads + 2 * args_model.n_kv_heads) * D * args_model.dim + args_model.dim * args_model.dim
                     + 3 * args_model.ffn_dim * args_model.dim) // 4
        step_bytes = per_layer * args_model.n_layers + 2 * args_model.vocab_size * args_model.dim
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        gbs = step_bytes / (ms / K * 1e-3) / 1e9
        print(json.dumps({
            "metric": f"BitNet-{a.workload.upper()} decode tok/s (bs{B}, tp{world})", "value": B * K / (ms * 1e-3),
            "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 x 2-bit ternary -> int32 (bf16 elsewhere)",
            "data": "synthetic",
            "config": {"workload": f"{a.workload} architecture ({args_model.n_layers} layers) random-init, batch {B}, "
                                   f"context {a.context}, tensor parallel x{world}, "
                                   f"{'op by op' if a.no_graph else 'CUDA graph'}", "batch": B},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak * world, "unit": "GB/s",
                         "frac": gbs / (peak * world), "traffic": None,
                         "note": "whole step: packed weights + bf16 output projection over aggregate HBM bandwidth"},
            "gpu_launches": None}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    a = parse_args()
    from bitnet_b200.config import preset   # no torch, no CUDA library: the reference arm loads neither

    args_model = preset(a.workload, n_layers=a.layers) if a.layers else preset(a.workload)
    if a.sweep_only:
        import torch

        n, k, m = (int(v) for v in a.sweep_only.split(","))
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        try:
            peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6650.0))
        except (OSError, ValueError):
            peak = 6650.0
        print(json.dumps({"kernel_sweep": kernel_sweep(dev, peak, shapes=[(n, k)], ms=[m])}), flush=True)
        return
    if a.tp:
        return run_tp(a, args_model)
    if a.impl == "reference":
        run_reference(a, args_model)
    else:
        run_ours(a, args_model)


if __name__ == "__main__":
    main()
