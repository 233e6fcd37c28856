"""In-tree build of the C-ABI CUDA library (``cats_b200/libcats_b200.so``) for sm_100a.

The library has no Python or torch dependency: it is compiled with plain ``nvcc`` into a shared
object next to this file and loaded with ``ctypes`` (see ``_lib.py``).  ``nvcc`` cross-compiles
without a GPU, so the build also serves as the "does it compile" check on a CPU-only machine.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libcats_b200.so")
STAMP_PATH = os.path.join(HERE, "libcats_b200.stamp")
SOURCES = ["cats_abi.cu"]
HEADERS = [
    os.path.join(CSRC, "cats_common.cuh"),
    os.path.join(CSRC, "cats_kernels.cuh"),
    os.path.join(CSRC, "cats_tma.cuh"),
    os.path.join(CSRC, "cats_mega.cuh"),
    os.path.join(ROOT, "include", "cats_b200.h"),
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libcats_b200.so")
    return cand


def source_digest() -> str:
    h = hashlib.sha256()
    for p in [os.path.join(CSRC, s) for s in SOURCES] + HEADERS:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP_PATH)):
        return False
    with open(STAMP_PATH) as f:
        return f.read().strip() == source_digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if the sources changed; returns the path of the shared object.

    Safe to call from several processes at once (the ranks of a multi-GPU job import the package
    at the same time): a file lock serialises them, the loser of the race finds the library
    current, and the shared object is moved into place in one step."""
    import fcntl

    if not force and is_current():
        return LIB_PATH
    with open(os.path.join(HERE, "libcats_b200.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current():
            return LIB_PATH
        tmp = LIB_PATH + f".tmp{os.getpid()}"
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-o", tmp]
        cmd += [os.path.join(CSRC, s) for s in SOURCES]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        log = proc.stdout + proc.stderr
        with open(os.path.join(HERE, "libcats_b200.buildlog"), "w") as f:
            f.write(" ".join(cmd) + "\n" + log)
        if proc.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("nvcc failed:\n" + log[-4000:])
        if verbose:
            print(log)
        os.replace(tmp, LIB_PATH)
        with open(STAMP_PATH, "w") as f:
            f.write(source_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
