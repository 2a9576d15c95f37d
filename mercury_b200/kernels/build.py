"""Compile the CUDA sources under `csrc/` into one shared library for sm_100a.

No JIT framework and no Python headers: every source is a plain `.cu` with `extern "C"`
entry points, compiled by nvcc and loaded through ctypes, so a fresh checkout builds in
well under a minute. The library lands next to this file (`_lib/`), or, when that folder
cannot be written, under the system's temporary folder; it is rebuilt when a source or a
flag changes (the file name carries a hash of both). Progress goes to stderr, one line per
source, because the first call of a fresh checkout has to wait for it.

`build(bounds_check=True)` makes the checked variant (`-DMB_BOUNDS_CHECK`, see
csrc/common.cuh): every index a kernel takes from the step's device buffers is compared
with its limit and a bad one is recorded instead of used. It is a library of its own
(another file name) and is loaded instead of the ordinary one when the environment has
MERCURY_B200_BOUNDS_CHECK=1. It is the stand-in for a memory checker where none may run.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
SOURCES = ["elementwise.cu", "gemm_simt.cu", "gemm_skinny.cu", "gemm_tcgen05.cu", "gemm_pair.cu", "attention_simt.cu", "attention_mma.cu", "attention_tcgen05.cu", "sampling.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise BuildError("nvcc was not found (set NVCC or put it on PATH); the CUDA kernels "
                     "cannot be compiled and there is no fallback")


def _sources() -> list[Path]:
    listed = [CSRC / name for name in SOURCES]
    missing = [str(p) for p in listed if not p.exists()]
    if missing:
        raise BuildError(f"kernel sources are missing: {missing}")
    return listed


# the checked variant shares its status words between the sources: relocatable device code
CHECK_FLAGS = ["-DMB_BOUNDS_CHECK", "-rdc=true"]


def bounds_check_wanted() -> bool:
    return os.environ.get("MERCURY_B200_BOUNDS_CHECK", "") not in ("", "0")


def _fingerprint(bounds_check: bool = False) -> str:
    digest = hashlib.sha256()
    for path in sorted(CSRC.glob("*.cu*")) + sorted(CSRC.glob("*.h")):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + (CHECK_FLAGS if bounds_check else [])).encode())
    return digest.hexdigest()[:16]


def _writable_dir() -> Path:
    in_tree = Path(__file__).resolve().parent / "_lib"
    try:
        in_tree.mkdir(exist_ok=True)
        probe = in_tree / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return in_tree
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"mercury_b200_lib_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _say(message: str) -> None:
    print(f"[mercury_b200] {message}", file=sys.stderr, flush=True)


def library_path(bounds_check: bool = False) -> Path:
    stem = "libmercury_b200_checked_" if bounds_check else "libmercury_b200_"
    return _writable_dir() / f"{stem}{_fingerprint(bounds_check)}.so"


def build(force: bool = False, verbose: bool = True, bounds_check: bool = False) -> Path:
    """Build the library (or its checked variant) if it is not there yet; returns its path."""
    target = library_path(bounds_check)
    extra = CHECK_FLAGS if bounds_check else []
    if target.exists() and not force:
        return target
    nvcc = _nvcc()
    out_dir = target.parent
    work = Path(tempfile.mkdtemp(prefix="mercury_b200_build_", dir=str(out_dir)))
    started = time.time()
    if verbose:
        _say(f"compiling {len(SOURCES)} CUDA sources for sm_100a with {nvcc} (first call only"
             f"{', checked variant' if bounds_check else ''})")

    def compile_one(src: Path) -> Path:
        obj = work / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t0 = time.time()
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
        if verbose:
            _say(f"  {src.name} compiled in {time.time() - t0:.1f} s")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
            objects = list(pool.map(compile_one, _sources()))
        partial = work / target.name
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(partial), *map(str, objects)]
        done = subprocess.run(link, capture_output=True, text=True)
        if done.returncode != 0:
            raise BuildError(f"linking failed:\n{done.stdout}\n{done.stderr}")
        os.replace(partial, target)  # atomic: a concurrent builder sees all or nothing
    finally:
        shutil.rmtree(work, ignore_errors=True)
    for stale in out_dir.glob("libmercury_b200_*.so"):
        if stale != target and ("_checked_" in stale.name) == bounds_check:
            try:
                stale.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"built {target.name} in {time.time() - started:.1f} s")
    return target
