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
SOURCES = ["rotate_quant.cu", "rotate_mma.cu", "rotate_umma.cu", "decompress_umma.cu", "packing.cu", "attention.cu", "attention_mma.cu", "attention_tiled.cu", "tiling.cu", "index_scan.cu", "index_scan_mma.cu", "index_scan_umma.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _headers() -> list[str]:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "quashkv_b200.h"))
    return [p for p in deps if os.path.exists(p)]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(p) > built for p in deps)


def _stale() -> bool:
    return _newer(LIB_PATH, _sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources when the library is missing or older than a source.  Every source becomes an
    object file of its own (compiled side by side, kept under lib/obj so that a change rebuilds one file),
    then the objects are linked into the shared library."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("quashkv_b200: nvcc not found; cannot build libquashkv_b200.so")
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    headers = _headers()
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src: str):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        if not force and not _newer(obj, [src] + headers):
            return obj, ""
        cmd = [nvcc, *compile_flags, "-c", src, "-o", obj]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"quashkv_b200: nvcc failed on {os.path.basename(src)}\n" + proc.stdout + proc.stderr)
        return obj, proc.stderr

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, _sources()))
    if verbose:
        sys.stderr.write("".join(log for _, log in results))
    proc = subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *[obj for obj, _ in results]], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("quashkv_b200: link failed\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
