"""Build the CUDA library in-tree with nvcc for sm_100a.

Mirrors the role of the reference's ``flashloop-build-kernels`` console script
(flashloop/build_kernels.py:12-32): compile the extension next to the package.
Here the product is a plain C-ABI shared library, ``csrc/libflashloop_b200.so``;
no torch headers are involved and nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIBRARY = CSRC / "libflashloop_b200.so"
SOURCES = ("fl_capi.cu", "fl_pack.cu", "fl_reader.cu", "fl_selected.cu", "fl_select.cu", "fl_append.cu", "fl_compact.cu",
           "fl_step.cu", "fl_encode.cu", "fl_comm.cu", "fl_linear.cu")
FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr")


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build flashloop_b200")
    return found


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source and link the shared library; returns its path."""

    nvcc = _nvcc()
    headers = list(CSRC.glob("*.cuh")) + [CSRC.parents[1] / "include" / "flashloop_b200.h"]
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    objects = []
    jobs = []
    for src in sources:
        obj = src.with_suffix(".o")
        objects.append(obj)
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in jobs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(out)
        if proc.returncode != 0:
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    if force or jobs or _stale(LIBRARY, objects):
        subprocess.run([nvcc, "-arch=sm_100a", "-shared", "-o", str(LIBRARY), *map(str, objects), "-lcudart"],
                       check=True)
    return LIBRARY


def main() -> None:
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)


if __name__ == "__main__":
    main()
