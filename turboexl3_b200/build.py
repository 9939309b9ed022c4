"""Builds libt3.so (the C-ABI library) in-tree with nvcc for sm_100a. No torch, no JIT cache: the .so sits next to the
sources so it travels with the tree.

    python -m turboexl3_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libt3.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]

# (source, object stem, extra flags)
UNITS = [
    ("t3_noalloc.cu", "t3_noalloc", []),
    ("t3_table.cu", "t3_table", []),
    ("t3_prefill.cu", "t3_prefill", []),
    ("t3_api.cu", "t3_api", []),
    ("t3_dequant.cu", "t3_dequant", []),
    ("t3_decode_rows.cu", "t3_decode_rows_cb0", ["-DT3_CB=0"]),
    ("t3_decode_rows.cu", "t3_decode_rows_cb1", ["-DT3_CB=1"]),
    ("t3_decode_rows.cu", "t3_decode_rows_probe2", ["-DT3_CB=2"]),  # the dense GEMV's timing probes
    ("t3_decode_rows.cu", "t3_decode_rows_probe3", ["-DT3_CB=3"]),
    ("t3_decode_rows.cu", "t3_decode_rows_probe4", ["-DT3_CB=4"]),
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libt3.so cannot be built")


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    for header in ("t3.h", "t3_table.h"):
        with open(os.path.join(os.path.dirname(HERE), "include", header), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(repr(UNITS).encode())
    return h.hexdigest()


def sources_digest() -> str:
    """A digest of the kernel sources alone (what a captured profile is a profile of)."""
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()[:16]


def _compile(unit, verbose: bool) -> str:
    src, stem, extra = unit
    obj = os.path.join(OBJ, stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src} ({stem}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        with open(os.path.join(OBJ, stem + ".ptxas.txt"), "w") as f:
            f.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every translation unit for sm_100a and link libt3.so; returns its path. Skips when up to date."""
    os.makedirs(OBJ, exist_ok=True)
    stamp = os.path.join(OBJ, "digest.txt")
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda u: _compile(u, verbose), UNITS))
    res = subprocess.run([_nvcc(), "-shared", "-o", LIB, *objs], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
