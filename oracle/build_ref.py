"""Builds oracle/_ref/libref_cuda.so: the REFERENCE's own CUDA decode kernels, compiled for sm_100a, behind the small
host harness of ref_harness.cu. Test infrastructure only (a GPU-side oracle and baseline for the MLX-4 matrix-vector
product); nothing of the reference is copied into the repository: the kernel text is read from the reference's tree
where it lies, written to oracle/_ref/ (git-ignored) and compiled there.

The reference builds its NVRTC module from the KERNEL_SRC string of src/cuda.rs followed by src/cuda_decode.cu
(src/cuda.rs:477); this script does the same concatenation. It runs only where the reference's tree is present; on a
machine without it the prebuilt library (if any) is used as it is.
"""
from __future__ import annotations

import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libref_cuda.so"


def build(reference: Path | None = None, verbose: bool = False) -> Path | None:
    """``reference``: the root of the reference's source tree; by default the OXINFER_REFERENCE environment variable, else the
    ``reference`` folder beside this repository."""
    import os

    if reference is None:
        reference = Path(os.environ.get("OXINFER_REFERENCE", str(HERE.parent.parent / "reference")))
    rs, cu = reference / "src" / "cuda.rs", reference / "src" / "cuda_decode.cu"
    if not rs.exists() or not cu.exists():
        return LIB if LIB.exists() else None
    m = re.search(r'const KERNEL_SRC: &str = r#"(.*?)"#;', rs.read_text(), re.S)
    if not m:
        raise RuntimeError("KERNEL_SRC not found in the reference's src/cuda.rs")
    OUT.mkdir(exist_ok=True)
    (OUT / "ref_kernels.cuh").write_text("// generated from the reference's tree by oracle/build_ref.py; not part of this repository\n"
                                         + m.group(1) + "\n" + cu.read_text())
    cmd = ["/usr/local/cuda/bin/nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared", "-Xcompiler",
           "-fPIC,-fvisibility=hidden", "-cudart", "static", "-o", str(LIB), str(HERE / "ref_harness.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=str(HERE))
    if verbose or r.returncode != 0:
        print(r.stdout[-3000:], r.stderr[-3000:])
    if r.returncode != 0:
        raise RuntimeError("building oracle/_ref/libref_cuda.so failed")
    return LIB


if __name__ == "__main__":
    p = build(verbose=True)
    print(p if p else "reference tree not present and no prebuilt library")
    sys.exit(0)
