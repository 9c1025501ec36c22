"""Build the C-ABI shared library with nvcc for sm_100a, in-tree.

The reference compiles its generated device source with CANN's `bisheng` and
links a `.so` per kernel (`src/backend/cann.py:28-172`); here a fixed set of
hand-written CUDA sources is compiled once into `ascendflow_b200/lib/`.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from pathlib import Path

from .diagnostics import ErrorKind, require

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
SOURCES = (PACKAGE / "csrc" / "sparse_mla_abi.cu", PACKAGE / "csrc" / "sparse_mla_neighbours.cu")
LIBRARY = PACKAGE / "lib" / "libsparse_mla_sm100a.so"
STAMP = LIBRARY.with_suffix(".stamp")
FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "--use_fast_math",
)


def _identity():
    digest = hashlib.sha256(" ".join(FLAGS).encode())
    for path in sorted((PACKAGE / "csrc").glob("*")) + [ROOT / "include" / "sparse_mla.h"]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def nvcc():
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    return None


def build_library(force=False, verbose=False):
    """Compile when sources changed; return the library path."""
    identity = _identity()
    if not force and LIBRARY.exists() and STAMP.exists() and STAMP.read_text() == identity:
        return LIBRARY
    compiler = nvcc()
    require(compiler is not None, "nvcc not found; cannot build the sm_100a library",
            kind=ErrorKind.RESOURCE)
    LIBRARY.parent.mkdir(parents=True, exist_ok=True)
    command = [compiler, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIBRARY),
               *map(str, SOURCES)]
    result = subprocess.run(command, capture_output=True, text=True)
    require(result.returncode == 0, "nvcc failed:\n" + result.stderr[-4000:], kind=ErrorKind.RESOURCE)
    STAMP.write_text(identity)
    if verbose:
        print(result.stderr)
    from . import gather_bench  # the isolated gather experiment is a second, small library

    gather_bench.build()
    return LIBRARY


def is_current():
    """True when the built library matches the sources and flags it would be built from now."""
    return LIBRARY.exists() and STAMP.exists() and STAMP.read_text() == _identity()


ATTENTION_KERNEL_SOURCES = ("sparse_mla_common.cuh", "tcgen05_ptx.cuh", "sparse_mla_tcgen05.cuh")


def attention_kernel_identity():
    """Hash of the files the tcgen05 attention kernel is compiled from (and of the flags): what a
    profile of that kernel is a profile of, whatever else in the library changes."""
    digest = hashlib.sha256(" ".join(FLAGS).encode())
    for name in ATTENTION_KERNEL_SOURCES:
        digest.update(name.encode())
        digest.update((PACKAGE / "csrc" / name).read_bytes())
    return digest.hexdigest()


def identity():
    """What the result records say about the binary: compiler flags and a hash of the sources."""
    return {"flags": " ".join(FLAGS), "source_sha256": _identity(),
            "attention_kernel_sha256": attention_kernel_identity(), "library": LIBRARY.name,
            "library_is_current": is_current()}


def library_path():
    """Path of the built library. A missing or stale library (sources or flags changed since it
    was built) is rebuilt if nvcc is here; otherwise this fails loudly: there is no other
    implementation to fall back to, and a stale binary must not be measured or shipped."""
    if not is_current() and nvcc() is not None:
        build_library()
    require(LIBRARY.exists(),
            f"{LIBRARY} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU fallback)", kind=ErrorKind.RESOURCE)
    require(is_current(),
            f"{LIBRARY} was built from other sources or flags than those present: rebuild it with "
            "`python -c 'import __graft_entry__ as g; g.build()'`", kind=ErrorKind.RESOURCE)
    return LIBRARY
