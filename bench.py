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
the time is the maximum over ranks.  The line then also carries a `tp` object: the 8B and the
~100B architectures decoded tensor-parallel over the N GPUs by the in-library step (peer-memory
exchange inside the kernels), with their fraction of the aggregate HBM roofline.
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
                    help="only the tensor-parallel measurement of --workload (8b, 100b) over the ranks, as its own line")
    ap.add_argument("--tp-engine", choices=["fused", "nccl"], default="fused",
                    help="with --tp: the in-library step (peer-memory exchange inside the kernels) or the op-by-op "
                         "decoder with NCCL collectives (the bring-up arm)")
    ap.add_argument("--no-tp", action="store_true", help="skip the tp object of a multi-GPU run")
    ap.add_argument("--layers", type=int, default=0, help="use only the first LAYERS layers (0 = all): a small case for profilers, or with --tp")
    ap.add_argument("--context", type=int, default=PROMPT_LEN, help="tokens in the KV cache when decode starts (with --tp)")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (0 = the preset's): a small case for profilers")
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


def reference_gpu_kernel_us(dev):
    """The reference's own GPU kernel (its gpu/bitnet_kernels source built with its own command
    line as compute_80 PTX, compiled for this GPU by the driver when the library loads) on the
    four 2B shapes at M = 1: distinct weight buffers (> 2 x L2) cycled inside a CUDA graph, time
    per launch from CUDA events.  A baseline beside the sweep; nothing of it is on the product path."""
    import ctypes

    import torch

    from bitnet_b200 import _lib
    from oracle import build_oracle

    path = build_oracle.build_ref_gpu()
    if not path:
        return {"unavailable": "the reference's GPU kernel library was not built"}
    try:
        ref = ctypes.CDLL(path)
    except OSError as exc:
        return {"unavailable": f"load failed: {exc}"[:200]}
    ref.bitlinear_int8xint2.restype = None
    ref.bitlinear_int8xint2.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    g = torch.Generator(device=dev).manual_seed(2)
    stream = torch.cuda.Stream(device=dev)
    rows = []
    for n, k in [(3840, 2560), (2560, 2560), (13824, 2560), (2560, 6912)]:
        nbytes = n * k // 4
        copies = max(2, int(300e6 // nbytes))
        ws = [torch.randint(-128, 127, (n, k // 4), dtype=torch.int8, device=dev, generator=g) for _ in range(copies)]
        y = torch.randint(-127, 127, (1, k), dtype=torch.int8, device=dev, generator=g)
        s = torch.ones(1, dtype=torch.bfloat16, device=dev)
        wsc = torch.ones(4, dtype=torch.bfloat16, device=dev)
        out = torch.zeros((1, n), dtype=torch.bfloat16, device=dev)

        def run():
            st = _lib.stream_ptr()
            for w in ws:
                ref.bitlinear_int8xint2(_lib.ptr(y), _lib.ptr(w), _lib.ptr(out), _lib.ptr(s), _lib.ptr(wsc), 1, n, k, st)

        with torch.cuda.stream(stream):
            run()
            stream.synchronize()
            if not out.any():
                return {"unavailable": "the reference kernel's PTX produced no output on this GPU"}
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
        us = e0.elapsed_time(e1) * 1e3 / (3 * copies)
        rows.append({"N": n, "K": k, "M": 1, "us": round(us, 2), "weight_gbs": round(nbytes / us / 1e3, 1)})
        del ws
    return {"kernel": "ladder_int8xint2_kernel (reference, compute_80 PTX)", "rows": rows}


def decode_batch(model, args_model, dev, batch, steps, warmup, peak, prompt_len=PROMPT_LEN, want_e2e=True):
    """Prefill `prompt_len` random tokens for `batch` sequences, then greedy decode steps from a
    CUDA graph: device-resident tokens/s, the same with host buffers (ids copied in from pinned
    memory and copied back every step), prefill tokens/s, and the step's bytes (packed weights +
    bf16 output projection + the keys and values read) over the HBM peak."""
    import torch

    from bitnet_b200.generate import Generator

    max_seq = (prompt_len + 2 * (steps + warmup) + 64 + 127) // 128 * 128
    gen = Generator(model, batch, max_seq)
    g = torch.Generator(device=dev).manual_seed(SEED + 5)
    prompt = torch.randint(0, args_model.vocab_size, (batch, prompt_len), generator=g, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gen.prefill(prompt)                       # warm-up of the prefill kernels
    torch.cuda.synchronize()
    e0.record()
    gen.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    ms_prefill = e0.elapsed_time(e1)
    gen.capture()
    with torch.cuda.stream(gen.stream):
        for _ in range(warmup):
            gen.decode_step()
        gen.stream.synchronize()
        e0.record(gen.stream)
        for _ in range(steps):
            gen.decode_step()
        e1.record(gen.stream)
        gen.stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    weights, kv = arch_step_bytes(args_model, batch, prompt_len + warmup + steps // 2)
    gbs = (weights + kv) / (ms * 1e-3) / 1e9
    out = {"batch": batch, "value": batch / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms, "steps": steps,
           "prompt_len": prompt_len, "prefill_tok_s": batch * prompt_len / (ms_prefill * 1e-3),
           "engine": "kernel chain" if gen.fused is not None else "op by op (tcgen05 BitLinear, library attention)",
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "bytes_per_step": weights + kv, "traffic": None}}
    if want_e2e:
        host_tok = gen.host_out.clone()
        for _ in range(warmup):
            host_tok = gen.decode_step_host(host_tok[:, None]).clone()
        torch.cuda.synchronize()
        with torch.cuda.stream(gen.stream):
            e0.record(gen.stream)
        for _ in range(steps):
            host_tok = gen.decode_step_host(host_tok[:, None]).clone()
        with torch.cuda.stream(gen.stream):
            e1.record(gen.stream)
        torch.cuda.synchronize()
        out["e2e"] = {"value": batch * steps / (e0.elapsed_time(e1) * 1e-3), "unit": "tok/s",
                      "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch}
    return out


def config3_report(dev, peak, steps):
    """The 3B architecture (hidden 3200, FFN 8640, head_dim 100: K is padded to the 128-column
    tile): prefill of 512 random tokens, then decode, at batch 1, 16 and 64."""
    import torch

    from bitnet_b200.config import preset
    from bitnet_b200.model import build_synthetic

    am = preset("3b")
    model = build_synthetic(am, seed=SEED + 3, device=dev, max_seq_len=1024)
    rows = []
    for batch in (1, 16, 64):
        try:
            rows.append(decode_batch(model, am, dev, batch, steps, 3, peak, prompt_len=512, want_e2e=False))
        except Exception as exc:
            rows.append({"batch": batch, "error": repr(exc)[:300]})
    del model
    torch.cuda.empty_cache()
    return rows


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

        # the ranks share exchange areas through CUDA IPC; collectives are used for set-up, barriers and
        # the maximum over ranks only, and need no NVLink multicast objects
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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
    n_lin = len(lins)

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
    peak, measured = hbm_peak()
    n_launches = (gen.fused.kernels_per_step if fused else 2 * len(lins)) * K

    # ---- several GPUs: the 8B and ~100B architectures sharded tensor-parallel over them --------
    tp_rows = None
    if world > 1 and not a.no_tp:
        del gl, gen, model, lins
        torch.cuda.empty_cache()
        tp_rows = sharded_report(rank, world, dev, peak, steps=min(K, 32))
        lins = []

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    achieved = weight_bytes / (ms_lin * 1e-3) / 1e9
    cpu = None
    extras = {}
    if world == 1 and not a.no_cpu_baseline:
        tok_s, info, _ = cpu_i2s_tokens_per_s(args_model, B, steps=3, warmup=1, layers_sampled=min(args_model.n_layers, 4))
        cpu = dict(info, value=tok_s, unit="tok/s")
        try:       # the other baseline: the reference's GPU kernel on this GPU
            extras["reference_gpu_kernel"] = reference_gpu_kernel_us(dev)
        except Exception as exc:
            extras["reference_gpu_kernel"] = {"unavailable": repr(exc)[:200]}
    if world == 1 and not a.no_extras:
        try:
            extras["decode_bs64"] = decode_batch(model, args_model, dev, 64, steps=min(K, 16), warmup=3, peak=peak)
            extras["kernel_sweep"] = kernel_sweep(dev, peak)
            del gen, model
            torch.cuda.empty_cache()
            # the other architectures the benchmark configurations name, on this one GPU
            extras["config3_3b"] = config3_report(dev, peak, steps=min(K, 16))
            extras["tp"] = sharded_report(0, 1, dev, peak, steps=min(K, 32))
        except Exception as exc:   # the headline stands on its own
            extras["extras_error"] = repr(exc)[:300]
    if tp_rows is not None:
        extras["tp"] = tp_rows
    # every byte a decode step must read: packed BitLinear weights + the bf16 output projection
    step_bytes = weight_bytes + 2 * args_model.vocab_size * args_model.dim
    step_gbs = step_bytes / (ms / K * 1e-3) / 1e9
    # the BitLinear kernels of the chain on their own (prologue + matmul, no attention, no head)
    chain_linears = {"kernel": "chain_linear_kernel (prologue + W2A8 matmul + epilogue, PDL chain)" if fused else "w2a8_gemv_kernel",
                     "launches_per_step": n_lin, "bytes_per_launch": weight_bytes / n_lin,
                     "us_per_launch": 1e3 * ms_lin / n_lin, "achieved": achieved, "frac": achieved / peak,
                     # dram__bytes_read + write per launch from one ncu capture of the four 2B shapes
                     # (profiles/chain_linear_kernel_2b_m1.md), averaged as the launches are mixed
                     "traffic": 4.41e6 if (fused and a.workload == "2b" and B == 1) else None}
    roofline = dict(chain_linears, bound="hbm", peak=peak, unit="GB/s", peak_source="measured" if measured else "fallback",
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
        "gpu_launches": n_launches,
        "roofline": roofline,
        "cpu_baseline": cpu, "clocks": clocks, **extras,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def arch_step_bytes(args_model, batch, context):
    """Bytes one decode step must read: packed BitLinear weights, the bf16 output projection and
    the bf16 keys and values of `context` positions for every sequence."""
    D = args_model.head_dim
    per_layer = ((args_model.n_heads + 2 * args_model.n_kv_heads) * D * args_model.dim
                 + args_model.n_heads * D * args_model.dim + 3 * args_model.ffn_dim * args_model.dim) // 4
    weights = per_layer * args_model.n_layers + 2 * args_model.vocab_size * args_model.dim
    kv = 2 * 2 * args_model.n_kv_heads * D * context * batch * args_model.n_layers
    return weights, kv


def measure_sharded_decode(name, args_model, batch, context, steps, warmup, rank, world, dev, peak, want_local=True,
                           dec=None):
    """Decode steps of one model sharded tensor-parallel over the ranks (one rank: the whole
    model), at a KV cache already holding `context` positions per sequence.

    Batches up to 8 run the in-library step (`TPFusedStep`: the chain of fused kernels, the
    exchange between ranks inside the kernels through peer memory), replayed from a CUDA graph.
    Larger batches run the op-by-op decoder (`TPDecoder.decode_step`; with several ranks its NCCL
    collectives are issued eagerly, never from a graph).  Time from CUDA events, maximum over
    ranks.  `exchange_share` = 1 - (the same shards stepped with no exchange) / (the real step)."""
    import torch
    import torch.distributed as dist

    from bitnet_b200.tensor_parallel import GraphedStep, TPDecoder, TPFusedStep

    max_seq = (context + 2 * (steps + warmup) + 16 + 127) // 128 * 128
    if dec is None:
        dec = TPDecoder(args_model, SEED, rank, world, dev, backend="kernel", max_seq_len=max_seq, fast_random=True)
    assert dec.max_seq_len >= max_seq
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    fused = batch <= 8

    def fill(cache):
        for ck, cv in cache:     # a context of random keys and values stands in for a prefill
            ck[:, :context].copy_(torch.randn(ck[:, :context].shape, generator=g, device=dev, dtype=torch.bfloat16))
            cv[:, :context].copy_(torch.randn(cv[:, :context].shape, generator=g, device=dev, dtype=torch.bfloat16))

    def max_ms(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, stream):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
        barrier()
        return max_ms(e0.elapsed_time(e1)) / steps

    out = {"model": name, "batch": batch, "context": context, "tp": world, "steps": steps}
    if fused:
        def fused_ms(local_only):
            st = TPFusedStep(dec, batch, max_seq, local_only=local_only)
            fill(st.cache)
            st.tokens.copy_(torch.randint(0, args_model.vocab_size, (batch, 1), generator=g, device=dev))
            st.pos.fill_(context)
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                st.step()
                stream.synchronize()
                barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    st.step()
            ms = timed(graph.replay, stream)
            err, launches = st.error_flag(), st.kernels_per_step
            barrier()
            del graph
            st.close()
            return ms, err, launches

        from bitnet_b200._lib import BitnetError

        try:
            ms, err, launches = fused_ms(False)
            out.update(engine="in-library chain, peer-memory exchange inside the kernels, CUDA graph",
                       kernels_per_step=launches, error_flag=err)
            if world > 1 and want_local:
                try:
                    ms_local, _, _ = fused_ms(True)
                    out.update(ms_per_step_no_exchange=ms_local, exchange_share=max(0.0, 1.0 - ms_local / ms))
                except BitnetError as exc:
                    out["no_exchange_error"] = str(exc)[:160]
        except BitnetError as exc:
            # refused when the step is built (the same on every rank), e.g. batch x K of a BitLinear beyond
            # the shared memory that holds a CTA's quantised activations: the op-by-op decoder takes the case
            out["chain_refused"] = str(exc)[:160]
            fused = False
    if not fused:
        cache = dec.make_cache(batch, max_seq)
        fill(cache)
        tok = torch.randint(0, args_model.vocab_size, (batch, 1), generator=g, device=dev)
        pos = torch.full((batch,), context, dtype=torch.int64, device=dev)
        if world == 1:
            step = GraphedStep(dec, tok, pos, cache)
            ms = timed(step.replay, step.stream)
            out.update(engine="op by op (tcgen05 BitLinear, library attention), CUDA graph")
        else:
            def one():
                nonlocal tok
                tok = dec.decode_step(tok, pos, cache).view(batch, 1)
                pos.add_(1)

            ms = timed(one, torch.cuda.current_stream())
            out.update(engine="op by op with NCCL all-gather / all-reduce, issued eagerly")
        del cache
    weights, kv = arch_step_bytes(args_model, batch, context)
    gbs = (weights + kv) / (ms * 1e-3) / 1e9
    out.update(ms_per_step=ms, value=batch / (ms * 1e-3), unit="tok/s", step_bytes=weights + kv,
               achieved_gbs=gbs, peak_gbs=peak * world, frac=gbs / (peak * world))
    torch.cuda.empty_cache()
    return out


# (model, batch, context): the 8B architecture at a 2048-token context and the ~100B architecture
# at a 4096-token context; batches above 8 take the op-by-op decoder
SHARDED_CASES = [("8b", 1, 2048), ("8b", 8, 2048), ("8b", 64, 2048), ("100b", 1, 4096), ("100b", 8, 4096),
                 ("100b", 32, 4096)]


def sharded_report(rank, world, dev, peak, steps, cases=None):
    """The cases of SHARDED_CASES that the rank count divides; one decoder per model."""
    import torch

    from bitnet_b200.config import preset
    from bitnet_b200.tensor_parallel import TPDecoder

    rows, dec, dec_name = [], None, None
    for name, batch, context in (cases or SHARDED_CASES):
        am = preset(name)
        if am.n_heads % world or am.n_kv_heads % world:
            continue
        k = steps if batch <= 8 else max(2, steps // 4)
        try:
            if dec_name != name:
                dec = None
                torch.cuda.empty_cache()
                dec = TPDecoder(am, SEED, rank, world, dev, backend="kernel", max_seq_len=context + 2 * steps + 256,
                                fast_random=True)
                dec_name = name
            rows.append(measure_sharded_decode(name, am, batch, context, k, 3, rank, world, dev, peak, dec=dec))
        except Exception as exc:      # one case must not take the line with it
            rows.append({"model": name, "batch": batch, "context": context, "tp": world, "error": repr(exc)[:300]})
            break                     # the ranks may no longer be in step: stop here
    dec = None
    torch.cuda.empty_cache()
    return rows


def run_tp(a, args_model):
    """Only the tensor-parallel measurement of --workload, as a line of its own."""
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    peak, measured = hbm_peak()
    r = measure_sharded_decode(a.workload, args_model, a.batch, a.context, a.steps, max(a.warmup, 3), rank, world, dev, peak)
    if rank == 0:
        print(json.dumps({
            "metric": f"BitNet-{a.workload.upper()} decode tok/s (bs{a.batch}, tp{world})", "value": r["value"],
            "unit": "tok/s", "n_gpus": world, "steps": r["steps"], "warmup": max(a.warmup, 3), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x 2-bit ternary -> int32 (bf16 elsewhere)", "data": "synthetic",
            "config": {"workload": f"{a.workload} architecture ({args_model.n_layers} layers) random ternary shards, batch "
                                   f"{a.batch}, context {a.context}, tensor parallel x{world}; {r['engine']}",
                       "batch": a.batch},
            "roofline": {"bound": "hbm", "achieved": r["achieved_gbs"], "peak": r["peak_gbs"], "unit": "GB/s",
                         "frac": r["frac"], "traffic": None, "peak_source": "measured" if measured else "fallback",
                         "note": "whole step: packed weights + bf16 output projection + KV cache over aggregate HBM bandwidth"},
            "tp": r, "gpu_launches": r.get("kernels_per_step", 0) * r["steps"]}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def hbm_peak():
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(peaks["hbm_gbs"]), True
    except (OSError, ValueError, KeyError):
        return 6650.0, False


def main():
    a = parse_args()
    from bitnet_b200.config import preset   # no torch, no CUDA library: the reference arm loads neither

    over = {}
    if a.layers:
        over["n_layers"] = a.layers
    if a.vocab:
        over["vocab_size"] = a.vocab
    args_model = preset(a.workload, **over)
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
