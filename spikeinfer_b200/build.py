"""Build the C-ABI CUDA library in-tree with nvcc for sm_100a.

``python -m spikeinfer_b200.build`` compiles ``csrc/*.cu`` into
``spikeinfer_b200/libspikeinfer_b200.so``.  nvcc cross-compiles without a GPU, so this
also runs on a CPU-only build machine.  The library is rebuilt only when a source or
header is newer than it (``force=True`` overrides).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libspikeinfer_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
]
# Translation units whose arithmetic contract forbids contracting a multiply and an add into one rounding: the LIF
# recurrence (every product and sum is rounded on its own, as the reference does) and the RMSNorm's mean + eps.
NO_FMA_CONTRACTION = {"spk_lif.cu", "spk_norm.cu"}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    if not force and not is_stale():
        return LIB_PATH
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        if src.name in NO_FMA_CONTRACTION:
            cmd.insert(1, "--fmad=false")
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = []
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed.append(f"--- {src.name} ---\n{out}")
        elif (verbose or ptxas_info) and out.strip():
            print(f"--- {src.name} ---\n{out}", flush=True)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp),
            *map(str, objs), "-lcudart", "-ldl"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
