"""Compile the reference's own CUDA kernels (rust/kernels/asca.cu, unmodified, included from
where it lies) together with the host launchers of oracle/ref_kernels.cu into
oracle/_ref/libasca_ref.so. TEST INFRASTRUCTURE: it lets GPU tests pin the CPU oracle against
outputs of the reference's own code. Runs only where the reference tree is present; the built
library travels with the repository snapshot to the GPU machine.

    python oracle/build_ref.py <path-to-reference-root>

The reference root comes from the argument or from the environment variable ASCA_REFERENCE_ROOT; without either
nothing is built and an already built library is used as it is.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

DIR = Path(__file__).resolve().parent
OUT = DIR / "_ref" / "libasca_ref.so"


def build(reference_root: str | None = None, force: bool = False) -> Path | None:
    where = reference_root or os.environ.get("ASCA_REFERENCE_ROOT")
    src = Path(where) / "rust" / "kernels" / "asca.cu" if where else None
    if src is None or not src.exists():
        return OUT if OUT.exists() else None
    wrap = DIR / "ref_kernels.cu"
    if not force and OUT.exists() and OUT.stat().st_mtime >= max(src.stat().st_mtime, wrap.stat().st_mtime):
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    # the reference's own nvcc flags (rust/build.rs:28-37: -O3 -std=c++17), arch set to sm_100a
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           "-cudart", "static", f'-DASCA_REF_CU="{src}"', str(wrap), "-o", str(OUT)]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
