"""In-tree build of ``libquashkv_b200.so`` (nvcc, sm_100a only).

``python -m quashkv_b200._build`` or ``build()``; the library lands in
``quashkv_b200/lib/`` next to the sources so that it travels with the tree.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libquashkv_b200.so")
SOURCES = ["rotate_quant.cu", "rotate_mma.cu", "rotate_umma.cu", "packing.cu", "attention.cu", "attention_mma.cu", "index_scan.cu", "index_scan_mma.cu", "index_scan_umma.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = _sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "quashkv_b200.h"))
    return any(os.path.getmtime(p) > built for p in deps if os.path.exists(p))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources when the library is missing or older than a source."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("quashkv_b200: nvcc not found; cannot build libquashkv_b200.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, *_sources()]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("quashkv_b200: nvcc failed\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
