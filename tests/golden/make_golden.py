"""Generates the golden vectors under tests/golden/ from the reference's own code.

Run it where a microsoft/BitNet checkout is available (it cannot run on a machine without
one; the vectors it writes are committed so that the tests need no checkout):

    python tests/golden/make_golden.py --ref /path/to/BitNet

What it records (all inputs come from numpy's seeded PCG64 generator, seeds in the file):

* ``ref_gpu_pack.npz``  - gpu/pack_weight.py:convert_weight_int8_to_int2 imported from the
  checkout and run on small ternary matrices.
* ``ref_i2s.npz``       - src/ggml-bitnet-mad.cpp compiled in place (oracle/build_oracle.py):
  quantize_i2_s bytes and ggml_vec_dot_i2_i8_s results, including a ragged row count, a
  non-multiple-of-32 block count, and raw random bytes (so that code 3 occurs).
* ``ref_converters.npz`` - utils/convert-hf-to-gguf-bitnet.py:quantize_to_i2_s (with and
  without override_scale) and gpu/convert_safetensors.py:invert_convert_q, taken from their
  files by name and run on small inputs.
* ``ref_gpu_test_kat.npz`` - the inputs and expected bf16 outputs of the procedural
  known-answer test gpu/test.py:42-61 (ternary weights, int8 activations in [-128,126],
  all scales 1, expected = int32 matmul cast to bf16) on reduced shapes plus one real
  shape, with the reference's packed weights for those inputs.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BITNET_REFERENCE_DIR", "/root/reference"))
    a = ap.parse_args()

    from oracle import build_oracle
    from oracle import np_oracle as O

    ref_so = build_oracle.build_ref(a.ref, force=True)
    assert ref_so, "reference checkout not found"
    R = O.RefLib(ref_so)

    # ---- the reference's GPU packer, imported from the checkout --------------------------
    import torch

    sys.path.insert(0, os.path.join(a.ref, "gpu"))
    import pack_weight as ref_pack  # noqa: E402  (the reference's module)

    out = {}
    for i, (n, k) in enumerate([(16, 32), (32, 128), (48, 256), (64, 384)]):
        rng = np.random.default_rng(1000 + i)
        q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
        packed = ref_pack.convert_weight_int8_to_int2(torch.from_numpy(q.copy())).numpy()
        out[f"q_{i}"] = q
        out[f"packed_{i}"] = packed
    np.savez_compressed(os.path.join(HERE, "ref_gpu_pack.npz"), **out)

    # ---- the reference's compiled I2_S quantiser and dot kernel ---------------------------
    out = {}
    cases = [(8, 128, 1), (8, 256, 4), (5, 640, 3), (16, 2560, 8), (4, 4224, 1), (4, 6912, 4)]
    for i, (n, k, m) in enumerate(cases):
        rng = np.random.default_rng(2000 + i)
        q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
        scale = np.float32(0.5 + 0.25 * i)
        w = (q.astype(np.float32) * scale).astype(np.float32)
        buf = R.quantize_i2_s(w)
        y = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
        s = np.stack([R.vec_dot(buf[r * k // 4:], y[j:j + 1], k)[0] for r in range(n) for j in range(m)])
        out[f"w_{i}"] = w
        out[f"i2s_{i}"] = buf
        out[f"y_{i}"] = y
        out[f"dot_{i}"] = s.reshape(n, m).T.copy()          # [M, N] float code sums
        out[f"gemm_{i}"] = R.gemm(buf, y, n, k, threads=2)   # through the blocked driver
    # raw random bytes (code 3 present), as the reference's kernel timer feeds it
    # (utils/test_gemm_kernel.sh:183-197)
    rng = np.random.default_rng(2999)
    n, k, m = 8, 512, 4
    raw = rng.integers(0, 256, size=n * k // 4 + 32, dtype=np.uint8)
    y = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
    out["raw_bytes"] = raw
    out["raw_y"] = y
    out["raw_gemm"] = R.gemm(raw, y, n, k, threads=1)
    np.savez_compressed(os.path.join(HERE, "ref_i2s.npz"), **out)

    # ---- gpu/test.py's known-answer test, restated on the CPU ----------------------------
    out = {}
    for i, (n, k) in enumerate([(32, 256), (64, 1024), (2560, 2560)]):
        rng = np.random.default_rng(3000 + i)
        q = rng.integers(-1, 2, size=(n, k), dtype=np.int8)           # torch.randint(-1, 2)
        y = rng.integers(-128, 127, size=(1, k), dtype=np.int8)       # torch.randint(-128, 127)
        expect = torch.from_numpy(O.matmul_i32(y, q)).to(torch.bfloat16).view(torch.int16).numpy()
        out[f"shape_{i}"] = np.array([n, k, 3000 + i])
        out[f"expect_bf16_bits_{i}"] = expect
        if n * k <= 65536:                      # the large case is regenerated from its seed
            out[f"q_{i}"] = q
            out[f"y_{i}"] = y
            out[f"ref_packed_{i}"] = ref_pack.convert_weight_int8_to_int2(torch.from_numpy(q.copy())).numpy()
    np.savez_compressed(os.path.join(HERE, "ref_gpu_test_kat.npz"), **out)
    # ---- the reference's Python converters (functions taken from their files by name: the
    # modules themselves import the llama.cpp fork's gguf package, which is not in the checkout)
    import ast

    def ref_function(rel_path, name, env):
        src = open(os.path.join(a.ref, rel_path)).read()
        for node in ast.parse(src).body:
            if isinstance(node, ast.FunctionDef) and node.name == name:
                exec(compile(ast.Module([node], []), rel_path, "exec"), env)
                return env[name]
        raise KeyError(name)

    env = {"np": np}
    ref_quantize_to_i2_s = ref_function("utils/convert-hf-to-gguf-bitnet.py", "quantize_to_i2_s", env)
    from einops import rearrange

    env2 = {"torch": torch, "rearrange": rearrange}
    ref_invert_q = ref_function("gpu/convert_safetensors.py", "invert_convert_q", env2)
    out = {}
    for i, (n, k) in enumerate([(4, 128), (16, 256), (24, 640)]):
        rng = np.random.default_rng(4000 + i)
        w = rng.standard_normal((n, k)).astype(np.float32)
        s = np.float32(1.0) / max(np.abs(w).mean(dtype=np.float32), np.float32(1e-5))
        wq = (np.clip(np.rint(w * s), -1, 1) / s).astype(np.float32)           # weight_quant, :1055-1060
        out[f"wq_{i}"] = wq
        out[f"i2s_{i}"] = ref_quantize_to_i2_s(wq)
        tern = rng.integers(-1, 2, size=(n, k)).astype(np.float32)
        out[f"tern_{i}"] = tern
        out[f"i2s_override_{i}"] = ref_quantize_to_i2_s(tern, override_scale=0.625 + i)

    class Cfg:
        n_head = 4
    wq = torch.arange(4 * 8 * 3, dtype=torch.float32).view(32, 3)
    out["rope_in"] = wq.numpy()
    out["rope_out"] = ref_invert_q(wq, Cfg()).numpy()
    np.savez_compressed(os.path.join(HERE, "ref_converters.npz"), **out)

    for f in ("ref_gpu_pack.npz", "ref_i2s.npz", "ref_gpu_test_kat.npz", "ref_converters.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
