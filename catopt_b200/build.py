"""Build libcatopt_b200.so in-tree with nvcc for sm_100a.

Run as ``python -m catopt_b200.build`` (or call :func:`build`).  nvcc
cross-compiles without a GPU, so this also works on a CPU-only machine.  The
library lands beside this file so that it travels with the source tree and the
ctypes loader in ``_lib.py`` finds it without any install step.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libcatopt_b200.so"

SOURCES = [
    "verify_reduce.cu",
    "diag_scan.cu",
    "diag_compose.cu",
    "diag_scan_seg.cu",
    "linear_f32.cu",
    "linear_tf32x3.cu",
    "decayed_chunk_ffma.cu",
    "decayed_chunk_small.cu",
    "decayed_chunk_tc.cu",
    "decayed_chunk_tf32.cu",
    "decayed_seg_state.cu",
    "decayed_chunk.cu",
    "gated_contract.cu",
    "gated_contract_tc.cu",
    "om_causal.cu",
    "om_causal_tc.cu",
    "device_wait.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(
        [src.stat().st_mtime]
        + [h.stat().st_mtime for h in CSRC.glob("*.cuh")]
        + [(HERE.parent / "include" / "catopt_b200.h").stat().st_mtime]
    )
    return obj.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source and link the shared library."""
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for name in SOURCES:
        src = CSRC / name
        obj = objdir / (name + ".o")
        objs.append(obj)
        if force or _stale(obj, src):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for name, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {name}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not LIB.exists():
        cmd = [_nvcc(), "-Wno-deprecated-gpu-targets", "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
