"""Builds libgla_b200.so in-tree with nvcc for sm_100a.

    python -m gla_jax_b200.build [--force] [--verbose]

The library has no Python or torch dependency: it is plain CUDA behind the C ABI declared in
include/gla_b200.h.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libgla_b200.so"
SOURCES = ["gla_api.cu", "gla_scan.cu", "gla_simt.cu", "gla_recurrent.cu", "gla_chunk_sm100.cu", "gla_state_sm100.cu", "gla_static.cu", "gla_decode.cu", "gla_layer.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static",
]


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "gla_b200.h"]
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every translation unit to an object file and link the shared library."""
    if not force and not _stale():
        return LIB
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = objdir / (src[:-3] + ".o")
        cmd = [NVCC, *FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [NVCC, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "-Xlinker", "--exclude-libs,ALL", "-Xlinker", "-Bsymbolic",
            "-o", str(LIB), *objs, "-lcuda"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


def build_xla_ffi() -> Path:
    """Compile csrc/gla_xla_ffi.cc into libgla_b200_xla.so against jaxlib's XLA FFI headers.
    Needs an importable jax (jax.ffi.include_dir()); raises otherwise."""
    import jax  # noqa: F401  (ImportError here means: no jax in this environment)
    inc = jax.ffi.include_dir()
    out = PKG / "libgla_b200_xla.so"
    cmd = [NVCC, "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-I", inc, str(CSRC / "gla_xla_ffi.cc"),
           "-o", str(out), "-L", str(PKG), "-lgla_b200", "-Xlinker", "-rpath,$ORIGIN"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("building the XLA FFI handlers failed")
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--with-jax", action="store_true", help="also build the XLA FFI handler library")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    if a.with_jax:
        print(build_xla_ffi())
