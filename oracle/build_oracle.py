"""Builds the two CPU checkers.  Test infrastructure only.

* ``oracle/liboracle_port.so``  - the plain-C restatement (``i2s_port.c``).
* ``oracle/_ref/libref_i2s.so`` - the reference's own ``src/ggml-bitnet-mad.cpp`` compiled
  where it lies in the reference checkout (never copied), against the four stand-in
  headers in ``oracle/shim``, together with ``ref_driver.cpp``.  Built only when a
  reference checkout is present; a machine without one uses the prebuilt file.

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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print("port:", build_port(a.force))
    print("ref: ", build_ref(a.ref, a.force))


if __name__ == "__main__":
    sys.exit(main())
