"""Compile the CUDA sources of ``csrc/`` for sm_100a into one shared library.

The sources are plain CUDA with C entry points (no torch headers), so a file
compiles in seconds; the files are compiled in parallel and linked once.  The
library's name carries a hash of the sources and flags, so an edited source is
rebuilt and a stale library is never loaded.  The build folder is
``csrc/_build`` inside the package when that is writable, else a per-user folder
under the system's temporary directory; no home directory is needed.  While nvcc
runs, a line is printed every few seconds.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
LIB_PREFIX = "libacvram_b200_"
if os.environ.get("ACVRAM_B200_TIMELINE", "0") not in ("", "0"):
    NVCC_FLAGS.append("-DACV_TIMELINE")      # diagnostic build: kernels log their CTAs' begin and end times
    LIB_PREFIX = "libacvram_b200tl_"         # a library of its own beside the serving one
    if os.environ["ACVRAM_B200_TIMELINE"] == "sums":
        NVCC_FLAGS.append("-DACV_TIMELINE_SUMS")     # and the matrix product sums up what its loops wait for


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("ACVRAM_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $ACVRAM_NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the engine has no path without its CUDA kernels")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        out = os.path.join(tempfile.gettempdir(), f"acvram_b200_build_{os.getuid()}")
        os.makedirs(out, exist_ok=True)
        return out


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of the compiled library; compiles it first if it is not there."""
    tag = source_hash()
    bdir = _build_dir()
    lib = os.path.join(bdir, f"{LIB_PREFIX}{tag}.so")
    if os.path.isfile(lib):
        return lib
    # a library built in-tree travels with the checkout even when the folder is read-only
    in_tree_lib = os.path.join(CSRC, "_build", f"{LIB_PREFIX}{tag}.so")
    if os.path.isfile(in_tree_lib):
        return in_tree_lib
    if not build:
        raise BuildError(f"{lib} is not built")
    _compile(bdir, lib, tag, verbose)
    return lib


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[acvram_b200] {msg}", file=sys.stderr, flush=True)


def _compile(bdir: str, lib: str, tag: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)", verbose)
    done = []
    stop = threading.Event()

    def heartbeat():
        while not stop.wait(5.0):
            _say(f"  ... still compiling, {len(done)}/{len(srcs)} files done, {time.time() - t0:.0f} s", verbose)

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()

    def one(src: str) -> str:
        obj = os.path.join(bdir, f"{os.path.basename(src)[:-3]}_{tag}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}")
        done.append(src)
        _say(f"  compiled {os.path.basename(src)} ({len(done)}/{len(srcs)})", verbose)
        return obj

    try:
        with ThreadPoolExecutor(max_workers=max(1, min(len(srcs), os.cpu_count() or 1))) as pool:
            objs = list(pool.map(one, srcs))
        tmp = f"{lib}.{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-lcudart"]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {lib} failed:\n{proc.stdout}")
        os.replace(tmp, lib)
        for name in os.listdir(bdir):       # libraries of earlier source states are never loaded again
            if name.startswith(LIB_PREFIX) and name.endswith(".so") and os.path.join(bdir, name) != lib:
                try:
                    os.remove(os.path.join(bdir, name))
                except OSError:
                    pass
        for obj in objs:
            try:
                os.remove(obj)
            except OSError:
                pass
    finally:
        stop.set()
    _say(f"built {os.path.basename(lib)} in {time.time() - t0:.0f} s", verbose)


def ptxas_report() -> str:
    """Registers, spills and shared memory of every kernel (``-Xptxas -v``), as text."""
    nvcc = find_nvcc()
    out = []
    for src in sources():
        cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", CSRC, "-c", src, "-o", os.devnull]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        out.append(f"== {os.path.basename(src)}\n{proc.stdout}")
    return "\n".join(out)
