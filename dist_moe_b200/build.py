"""Build the C-ABI shared library ``_lib/libdist_moe_b200.so`` with nvcc for sm_100a.

The library is built in-tree so that it travels with the source tree; nothing is
installed into site-packages.  ``python -m dist_moe_b200.build`` rebuilds it.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
LIB_DIR = _PKG / "_lib"
LIB_PATH = LIB_DIR / "libdist_moe_b200.so"
_STAMP = LIB_DIR / "build.stamp"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
# extra compiler flags for experiments, e.g. DIST_MOE_NVCC_EXTRA="-DDM_PAIR_TRACE"
NVCC_FLAGS += os.environ.get("DIST_MOE_NVCC_EXTRA", "").split()


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [_PKG.parent / "include" / "dist_moe_b200.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; dist_moe_b200 needs the CUDA toolkit to build its kernels")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` into one shared library (skipped when up to date)."""
    digest = _digest()
    if not force and LIB_PATH.exists() and _STAMP.exists() and _STAMP.read_text().strip() == digest:
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    nvcc = find_nvcc()
    common = NVCC_FLAGS
    log_lines = []
    procs = []
    for src in _sources():
        obj = LIB_DIR / (src.stem + ".o")
        cmd = [nvcc, *common, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        log_lines.append(f"== {src.name}\n{out}")
        if proc.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src.name}")
        objs.append(str(obj))
    (LIB_DIR / "ptxas.log").write_text("\n".join(log_lines))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link failed")
    _STAMP.write_text(digest)
    if verbose:
        print("\n".join(log_lines))
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
