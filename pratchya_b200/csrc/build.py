"""Builds the shared libraries in this directory with nvcc for sm_100a.

    python -m pratchya_b200.csrc.build [--force] [-v]

libpratchya_b200.so is the product.  libpratchya_b200_diag.so is the same sources compiled with
-DPB_DIAGNOSTICS plus selftest.cu: cycle counters, timing experiments, environment switches, the
fault injection of the abort-path test and the device self-checks live there only, and only the
tests load it.  Both are kept in-tree next to their sources; nothing is installed anywhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
INCLUDE = HERE.parent.parent / "include"
LIB = HERE / "libpratchya_b200.so"
DIAG_LIB = HERE / "libpratchya_b200_diag.so"
SOURCES = ["api.cu", "quantize.cu", "dequantize.cu", "transpose_quantize.cu", "optimizer.cu", "gemm_sm100.cu", "wkv7.cu", "rwkv_glue.cu", "rwkv_norms.cu", "loss.cu"]
DIAG_SOURCES = SOURCES + ["selftest.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, diagnostics: bool = False) -> Path:
    """Compiles what is stale and links the product library (or, with `diagnostics`, the diagnostics one)."""
    names = DIAG_SOURCES if diagnostics else SOURCES
    lib = DIAG_LIB if diagnostics else LIB
    extra = ["-DPB_DIAGNOSTICS"] if diagnostics else []
    srcs = [HERE / s for s in names if (HERE / s).exists()]
    headers = list(HERE.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    objdir = HERE / ("build_diag" if diagnostics else "build")
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in srcs:
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, f"-I{INCLUDE}", f"-I{HERE}", "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    if force or procs or _stale(lib, objs):
        cmd = [nvcc, "-shared", "--cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(lib), *map(str, objs), "-ldl", "-lpthread"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return lib


def build_all(force: bool = False, verbose: bool = False):
    return build(force, verbose), build(force, verbose, diagnostics=True)


if __name__ == "__main__":
    print(*build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
