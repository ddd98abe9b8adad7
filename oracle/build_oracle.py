"""Builds the two CPU checkers.  Test infrastructure only.

* ``oracle/liboracle_port.so``  - the plain-C restatement (``i2s_port.c``).
* ``oracle/_ref/libref_i2s.so`` - the reference's own ``src/ggml-bitnet-mad.cpp`` compiled
  where it lies in the reference checkout (never copied), against the four stand-in
  headers in ``oracle/shim``, together with ``ref_driver.cpp``.  Built only when a
  reference checkout is present; a machine without one uses the prebuilt file.
* ``oracle/_ref/libbitnet_ref_gpu.so`` - the reference's own GPU kernel
  ``gpu/bitnet_kernels/bitnet_kernels.cu`` compiled where it lies with the reference's own
  command line (``gpu/bitnet_kernels/compile.sh:1``: PTX for compute_80, which the driver
  compiles for the GPU it finds at load time).  A second checker on a GPU machine and the
  "kernel to beat" in the benchmark's kernel sweep.

Usage: ``python oracle/build_oracle.py [--ref /path/to/BitNet]``
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REF = os.environ.get("BITNET_REFERENCE_DIR", "/root/reference")
PORT_SO = os.path.join(HERE, "liboracle_port.so")
REF_SO = os.path.join(HERE, "_ref", "libref_i2s.so")
REF_GPU_SO = os.path.join(HERE, "_ref", "libbitnet_ref_gpu.so")
# AVX2 only (no -march=native): the library is built on one machine and run on another.
SIMD = ["-mavx2", "-mfma"]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_port(force=False):
    src = os.path.join(HERE, "i2s_port.c")
    if force or _stale(PORT_SO, [src]):
        _run(["gcc", "-O3", "-fPIC", "-shared", "-fopenmp", "-std=c11", *SIMD, src, "-lm", "-o", PORT_SO])
    return PORT_SO


def build_ref(ref_dir=DEFAULT_REF, force=False):
    """Returns the path of the compiled reference, or None when it cannot be had."""
    mad = os.path.join(ref_dir, "src", "ggml-bitnet-mad.cpp")
    drv = os.path.join(HERE, "ref_driver.cpp")
    if not os.path.exists(mad):
        return REF_SO if os.path.exists(REF_SO) else None
    shims = [os.path.join(HERE, "shim", f) for f in os.listdir(os.path.join(HERE, "shim"))]
    if force or _stale(REF_SO, [mad, drv, *shims]):
        os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
        _run(["g++", "-O3", "-fPIC", "-shared", "-fopenmp", "-std=c++17", "-fpermissive", "-w", *SIMD,
              "-I", os.path.join(HERE, "shim"), "-I", os.path.join(ref_dir, "include"),
              mad, drv, "-o", REF_SO])
    return REF_SO


def build_ref_gpu(ref_dir=DEFAULT_REF, force=False):
    """The reference's GPU kernel library, or None when it cannot be had (no checkout and
    no prebuilt file, or no nvcc)."""
    src = os.path.join(ref_dir, "gpu", "bitnet_kernels", "bitnet_kernels.cu")
    hdr = os.path.join(ref_dir, "gpu", "bitnet_kernels", "bitnet_kernels.h")
    if not os.path.exists(src):
        return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
    if force or _stale(REF_GPU_SO, [src, hdr]):
        import shutil

        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        if not os.path.exists(nvcc):
            return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
        os.makedirs(os.path.dirname(REF_GPU_SO), exist_ok=True)
        # the reference's own line (gpu/bitnet_kernels/compile.sh:1), output redirected
        _run([nvcc, "-std=c++17", "-Xcudafe", "--diag_suppress=177", "--compiler-options", "-fPIC", "-lineinfo",
              "--shared", src, "-lcuda", "-gencode=arch=compute_80,code=compute_80", "-o", REF_GPU_SO])
    return REF_GPU_SO


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print("port:", build_port(a.force))
    print("ref: ", build_ref(a.ref, a.force))
    print("ref gpu:", build_ref_gpu(a.ref, a.force))


if __name__ == "__main__":
    sys.exit(main())
