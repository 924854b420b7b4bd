"""Test infrastructure: builds the reference's own CUDA readers for the timing arm of bench.py.

Compiles the reference's extension ``flashloop_kivi_gemv`` (flashloop/csrc/kivi_outer_gemv_binding.cpp and
kivi_outer_gemv_cuda.cu, the files flashloop/csrc/setup.py lists, with its flags ``-O3 --use_fast_math
-lineinfo``) for sm_100a straight from the reference checkout, without copying a source file, into
``oracle/_ref/`` (git-ignored).  The result is the baseline "the reference's kernels on the same GPU":
``bench.py --impl reference --workload kernels`` loads it; nothing in the product path does.

    python oracle/build_ref.py [path of the reference checkout]
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "flashloop_kivi_gemv"


def build(reference: Path, *, verbose: bool = True) -> Path | None:
    """Returns the built module's path, or None when the reference checkout is not there."""

    csrc = Path(reference) / "flashloop" / "csrc"
    sources = [csrc / "kivi_outer_gemv_binding.cpp", csrc / "kivi_outer_gemv_cuda.cu"]
    if not all(s.exists() for s in sources):
        return None
    from torch.utils import cpp_extension

    target = OUT / f"{NAME}.so"
    if target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources):
        return target
    OUT.mkdir(exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"]]
    libs = cpp_extension.library_paths()
    cmd = [nvcc, "-O3", "--use_fast_math", "-lineinfo", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-shared", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "--expt-relaxed-constexpr", "-diag-suppress", "20012,20013,20014,20015",
           *[f"-I{i}" for i in includes], *[str(s) for s in sources], *[f"-L{l}" for l in libs],
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           *[f"-Xlinker=-rpath={l}" for l in libs], "-o", str(target)]
    if verbose:
        print("building", target, "from", csrc, flush=True)
    done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"the reference's CUDA extension did not build:\n{done.stdout[-4000:]}")
    return target


if __name__ == "__main__":
    path = build(Path(sys.argv[1]) if len(sys.argv) > 1 else Path("/root/reference"))
    print(path if path else "reference checkout not found: nothing built")
