"""Build recipe for libwinnow_tq.so (nvcc, sm_100a only, in-tree output)."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libwinnow_tq.so"
SOURCES = ["wtq_pack.cu", "wtq_append.cu", "wtq_decode.cu", "wtq_decode_mma.cu", "wtq_api.cu", "wtq_dequant.cu", "wtq_dequant_umma.cu", "wtq_prefill.cu", "wtq_rows_mma.cu",
           "wtq_decode_static.cu", "wtq_dense.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str | None:
    return shutil.which("nvcc") or (
        "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES]


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "winnow_tq.h"]
    return all(d.stat().st_mtime <= built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel into one shared library next to this file."""
    if not force and up_to_date():
        return LIB
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libwinnow_tq.so")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB),
           *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB
