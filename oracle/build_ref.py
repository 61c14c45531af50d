"""Builds the checker's native pieces (test infrastructure, never shipped):

  oracle/_ref/*.cubin   the reference's own CUDA translation units
                        (kernels/sm89/{linear,encoder,decoder,subsampling,frontend}.cu of the
                        reference checkout), compiled where they lie -- no source is
                        copied -- with the flags of the reference's build.rs:91-103
                        (--cubin --std=c++17 -O3 -lineinfo [--use_fast_math]) but for
                        sm_100a instead of sm_89.  Used as the GPU-side oracle.
  oracle/_ref/liboracle.so   the C restatement (oracle/pk_oracle.c).

The reference's Rust host cannot be built here (no cargo/rustc), so only its
kernels run; their launch sequences are restated in oracle/refkernels.py.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
UNITS = {"linear": True, "encoder": True, "decoder": True, "subsampling": True, "frontend": True}


def reference_root(root: str | os.PathLike | None = None) -> Path | None:
    """The reference checkout: the argument, else $PK_REFERENCE_ROOT, else a directory named
    `reference` beside this repository.  None when its kernels are not there."""
    if root is None:
        root = os.environ.get("PK_REFERENCE_ROOT") or HERE.parent.parent / "reference"
    root = Path(root)
    return root if (root / "kernels" / "sm89" / "encoder.cu").exists() else None


def build_reference_cubins(force: bool = False, root: str | os.PathLike | None = None) -> list[Path]:
    root = reference_root(root)
    if root is None:
        return sorted(OUT.glob("*.cubin"))          # prebuilt files travel with the tree
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT.mkdir(exist_ok=True)
    procs = []
    for unit, fast_math in UNITS.items():
        src = root / "kernels" / "sm89" / f"{unit}.cu"
        dst = OUT / f"{unit}.cubin"
        if dst.exists() and not force and dst.stat().st_mtime >= src.stat().st_mtime:
            continue
        cmd = [nvcc, "--cubin", "--std=c++17", "-O3", "-lineinfo",
               "--generate-code=arch=compute_100a,code=sm_100a"]
        if fast_math:
            cmd.append("--use_fast_math")
        cmd += [str(src), "-o", str(dst)]
        procs.append((unit, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for unit, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"reference unit {unit} failed to compile:\n{out}")
    return sorted(OUT.glob("*.cubin"))


def build_c_oracle(force: bool = False) -> Path:
    src = HERE / "pk_oracle.c"
    dst = OUT / "liboracle.so"
    OUT.mkdir(exist_ok=True)
    if dst.exists() and not force and dst.stat().st_mtime >= src.stat().st_mtime:
        return dst
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", str(src), "-o", str(dst), "-lm"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("C oracle failed to compile:\n" + res.stdout)
    return dst


if __name__ == "__main__":
    force = "--force" in sys.argv
    roots = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build_c_oracle(force))
    for p in build_reference_cubins(force, roots[0] if roots else None):
        print(p)
