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
    for f in ("ref_gpu_pack.npz", "ref_i2s.npz", "ref_gpu_test_kat.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
