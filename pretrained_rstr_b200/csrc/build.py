"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

``nvcc`` is called directly (no torch headers are involved, so a file compiles in
seconds); objects and the library go to ``csrc/_build`` inside the package when that
folder can be written, otherwise to a per-user folder under the system's temporary
directory.  A stamp of the sources and flags decides whether a rebuild is needed.
While compiling, a line is printed now and then so that a first call does not look
hung.  Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libprb200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math=false",
                           "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# --use_fast_math is deliberately off: expf/tanhf/erff/division stay IEEE-accurate.
NVCC_FLAGS = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
# extra flags for experiments (part of the stamp, so changing them rebuilds)
NVCC_FLAGS += os.environ.get("PRB200_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    """The CUDA files of the library: every .cu file of this folder."""
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set NVCC or put it on PATH); the CUDA extension of "
                     "pretrained_rstr_b200 cannot be built and there is no fallback")


def _stamp() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w") as fh:
            fh.write("x")
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("PRB200_BUILD_DIR")
    if override and _writable_dir(override):
        return override
    in_tree = os.path.join(HERE, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"prb200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable build folder ({in_tree} and {fallback} both failed)")


def _log(msg: str) -> None:
    print(f"[pretrained_rstr_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, verbose_ptxas: bool) -> str:
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + \
          ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Build if needed; returns the path of the shared library."""
    out_dir = build_dir()
    lib_name = LIB_NAME
    lib = os.path.join(out_dir, lib_name)
    stamp_file = os.path.join(out_dir, "stamp")
    stamp = _stamp()

    def fresh() -> bool:
        if not os.path.isfile(lib) or not os.path.isfile(stamp_file):
            return False
        with open(stamp_file) as fh:
            return fh.read().strip() == stamp

    if not force and fresh():
        return lib
    lock_path = os.path.join(out_dir, "lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return lib
            nvcc = find_nvcc()
            srcs = sources()
            _log(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} "
                 f"(first call only)")
            t0 = time.time()
            stop = threading.Event()

            def ticker():
                while not stop.wait(10.0):
                    _log(f"... still compiling ({time.time() - t0:.0f} s)")

            th = threading.Thread(target=ticker, daemon=True)
            th.start()
            try:
                objs = [os.path.join(out_dir, s[:-3] + ".o") for s in srcs]
                workers = max(1, min(len(srcs), os.cpu_count() or 1))
                with concurrent.futures.ThreadPoolExecutor(workers) as pool:
                    futs = {pool.submit(_compile_one, nvcc, s, o, verbose_ptxas): s
                            for s, o in zip(srcs, objs)}
                    for fut in concurrent.futures.as_completed(futs):
                        info = fut.result()
                        _log(f"compiled {futs[fut]} ({time.time() - t0:.0f} s)")
                        if verbose_ptxas and info:
                            print(info, file=sys.stderr)
                tmp = lib + f".tmp{os.getpid()}"
                cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs
                proc = subprocess.run(cmd, capture_output=True, text=True)
                if proc.returncode != 0:
                    raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
                os.replace(tmp, lib)
                with open(stamp_file, "w") as fh:
                    fh.write(stamp)
            finally:
                stop.set()
            _log(f"built {lib_name} in {time.time() - t0:.0f} s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv))
