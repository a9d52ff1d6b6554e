"""Builds libb200ops.so (sm_100a) from the CUDA sources beside this file.

nvcc cross-compiles without a GPU. The cubins target sm_100a only; the CUDA
runtime is linked statically and the driver entry point the library needs
(cuTensorMapEncodeTiled) is resolved at run time, so the library loads on a
machine without a driver (its compute entry points then refuse).
"""

from __future__ import annotations

import hashlib
import os
from pathlib import Path
import shutil
import subprocess
import sys

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
LIB_DIR = ROOT / "lib"
LIB = LIB_DIR / "libb200ops.so"
SOURCES = [
    "core.cu",
    "pool.cu",
    "rowwise.cu",
    "reduce.cu",
    "eltwise.cu",
    "pack.cu",
    "gemm.cu",
    "gemm_simt.cu",
    "gemm_umma.cu",
    "host_rows.cu",
    "attention.cu",
    "peer.cu",
]
HEADERS = ["common.cuh", "gemm_common.cuh", "umma_ptx.cuh", "../../include/b200ops.h"]
FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return found


def _stamp() -> str:
    digest = hashlib.sha256()
    for name in SOURCES + HEADERS:
        digest.update((HERE / name).read_bytes())
    digest.update(" ".join(FLAGS).encode())
    return digest.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source to an object (in parallel) and link the shared library.
    Up-to-date builds (same sources and flags) are skipped."""
    LIB_DIR.mkdir(exist_ok=True)
    stamp_file = LIB_DIR / "libb200ops.stamp"
    stamp = _stamp()
    if not force and LIB.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    compiler = nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    procs = []
    for name in SOURCES:
        obj = obj_dir / (Path(name).stem + ".o")
        cmd = [compiler, *FLAGS, *extra, "-c", str(HERE / name), "-o", str(obj)]
        procs.append((name, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objects = []
    failed = []
    for name, obj, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(f"--- {name}\n{out}\n")
        if proc.returncode != 0:
            failed.append(name)
        objects.append(str(obj))
    if failed:
        raise RuntimeError(f"nvcc failed for: {', '.join(failed)}")
    link = [compiler, "-shared", "-o", str(LIB), *objects, "-cudart", "static", "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    stamp_file.write_text(stamp)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
