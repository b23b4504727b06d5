"""Builds libnumr_b200.so in-tree with nvcc for sm_100a.

Usage: python -m numr_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and resolves cuTensorMapEncodeTiled
through the runtime's driver entry-point query, so it loads on a machine without
a GPU driver (its compute entry points then return NUMR_B200_ECUDA).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libnumr_b200.so"
TRACE_LIB_PATH = PKG_DIR / "libnumr_b200_trace.so"

# (source, object stem, extra defines). The tcgen05 GEMM kernel is instantiated once per
# (MMA kind, output kind) pair, each in its own object, so the instantiations compile in parallel.
GEMM_INSTANCES = [(0, 1), (0, 2), (1, 0), (2, 0), (2, 1), (2, 2), (2, 3), (2, 4), (3, 5)]
SOURCES = [("gemm_inst.cu", f"gemm_inst_k{k}_o{o}", [f"-DNB_INST_KIND={k}", f"-DNB_INST_OUT={o}"])
           for k, o in GEMM_INSTANCES]
SOURCES += [(s, s.rsplit(".", 1)[0], []) for s in
            ["gemm_sm100.cu", "gemv_sm100.cu", "matmul_int_sm100.cu", "prepass.cu", "conv_sm100.cu", "capi.cu",
             "ops.cpp"]]
HEADERS = ["sm100_ptx.cuh", "epilogue_math.cuh", "gemm_internal.h", "gemm_params.h", "gemm_kernel.cuh",
           "../../include/numr_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build numr_b200")
    return nvcc


def _deps_mtime() -> float:
    deps = [CSRC / h for h in HEADERS] + [Path(__file__)]
    return max(d.stat().st_mtime for d in deps)


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    newest = max(_deps_mtime(), max((CSRC / s).stat().st_mtime for s, _, _ in SOURCES))
    return newest > built


def build(force: bool = False, verbose: bool = False, jobs: int | None = None, trace: bool = False) -> Path:
    """Compiles every source for sm_100a and links the shared library.

    Objects are rebuilt only when their source or a header is newer (all of them with force=True);
    up to `jobs` compilations run at once (default: the CPU count). `trace=True` builds a second
    library, libnumr_b200_trace.so, whose GEMM kernel records timeline marks (NUMR_B200_TRACE_PTR);
    load it by naming it in NUMR_B200_LIBRARY. The normal library carries no trace code."""
    lib_path = TRACE_LIB_PATH if trace else LIB_PATH
    if not force and not trace and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    objdir = PKG_DIR / ("build_trace" if trace else "build")
    objdir.mkdir(exist_ok=True)
    hdr_time = _deps_mtime()
    jobs = jobs or max(1, os.cpu_count() or 1)
    objs, todo = [], []
    for src, stem, defines in SOURCES:
        obj = objdir / (stem + ".o")
        objs.append(str(obj))
        fresh = (not force and obj.exists()
                 and obj.stat().st_mtime >= max(hdr_time, (CSRC / src).stat().st_mtime))
        if not fresh:
            cmd = [nvcc, *NVCC_FLAGS, *defines, *(["-DNUMR_B200_TRACE"] if trace else []),
                   "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            todo.append((stem, cmd))
    failed = False
    running = []

    def reap(block_until_below: int):
        nonlocal failed
        while len(running) > block_until_below:
            stem, p = running.pop(0)
            out, _ = p.communicate()
            if p.returncode != 0:
                failed = True
                sys.stderr.write(f"--- nvcc failed on {stem} ---\n{out}\n")
            elif verbose or out.strip():
                sys.stderr.write(f"--- {stem} ---\n{out}")

    for stem, cmd in todo:
        reap(jobs - 1)
        if verbose:
            print(" ".join(cmd), flush=True)
        running.append((stem, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    reap(0)
    if failed:
        raise RuntimeError("numr_b200: compilation failed")
    link = [nvcc, "-shared", "-o", str(lib_path), *objs, "-cudart", "static",
            "-Xlinker", "--exclude-libs,ALL"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"numr_b200: link failed\n{r.stdout}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv)
    print(path)
