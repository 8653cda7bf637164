"""Build the CUDA shared library in-tree (``ixrun_b200/libixb200.so``).

    python -m ixrun_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library has no Python or
torch dependency; the package binds it with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "libixb200.so")
SOURCES = ["ixb200.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh")) + [os.path.join("..", "..", "include", "ixb200.h")]


def nvcc_path() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the ixb200 CUDA library cannot be built")


STAMP = SO + ".srchash"


def source_hash() -> str:
    """Hash of everything the library is built from (sources, headers, extra defines, this file)."""
    import hashlib

    h = hashlib.sha256()
    for f in [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]:
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(os.environ.get("IXB200_DEFINES", "").encode())
    return h.hexdigest()


def is_stale() -> bool:
    """True unless the library exists and was built from the sources as they are now.  Judged by content, not by
    modification times, which a copy of the tree to another machine does not keep."""
    if not os.path.exists(SO) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile to a temporary file and move it into place, under a file lock: several ranks that find the library
    stale at the same moment build one after the other, and none of them can load a half-written file."""
    import fcntl

    with open(SO + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():       # another process built it while this one waited for the lock
                return SO
            tmp = f"{SO}.tmp{os.getpid()}"
            cmd = [
                nvcc_path(), "-O3", "-std=c++17", "-lineinfo",
                "-gencode", "arch=compute_100a,code=sm_100a",
                "-Xcompiler", "-fPIC", "-shared",
            ] + ([f"-D{d}" for d in os.environ.get("IXB200_DEFINES", "").split()]) + [
                "-o", tmp,
            ] + [os.path.join(CSRC, f) for f in SOURCES]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            env = dict(os.environ)
            env.pop("CC", None)
            env.pop("CXX", None)
            r = subprocess.run(cmd, capture_output=True, text=True, env=env)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed building libixb200.so")
            os.replace(tmp, SO)
            with open(STAMP, "w") as f:
                f.write(source_hash())
            return SO
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
