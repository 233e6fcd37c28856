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
OBJ_DIR = os.path.join(HERE, "_obj")
# translation units: (source, extra defines, object name).  The kernels are instantiated once per
# element type in units of their own so that the library compiles in parallel.
UNITS = [("cats_abi.cu", [], "cats_abi.o")]
for _id, _name in ((0, "f32"), (1, "f16"), (2, "bf16")):
    UNITS.append(("cats_inst_stage.cu", [f"-DCATS_ELEM_ID={_id}"], f"cats_inst_stage_{_name}.o"))
    UNITS.append(("cats_inst_mega.cu", [f"-DCATS_ELEM_ID={_id}"], f"cats_inst_mega_{_name}.o"))
UNITS.append(("cats_inst_dense.cu", [], "cats_inst_dense.o"))
SOURCES = sorted({u[0] for u in UNITS})
HEADERS = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))) + [
    os.path.join(ROOT, "include", "cats_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
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
        from concurrent.futures import ThreadPoolExecutor

        os.makedirs(OBJ_DIR, exist_ok=True)
        tmp = LIB_PATH + f".tmp{os.getpid()}"
        nvcc = _nvcc()

        def compile_unit(unit):
            src, defines, obj = unit
            cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", os.path.join(ROOT, "include"), "-c",
                   os.path.join(CSRC, src), "-o", os.path.join(OBJ_DIR, obj)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            return proc.returncode, " ".join(cmd) + "\n" + proc.stdout + proc.stderr

        with ThreadPoolExecutor(max_workers=min(len(UNITS), os.cpu_count() or 1)) as pool:
            results = list(pool.map(compile_unit, UNITS))
        log = "\n".join(r[1] for r in results)
        rc = max(r[0] for r in results)
        if rc == 0:
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--shared", "-o", tmp]
            cmd += [os.path.join(OBJ_DIR, u[2]) for u in UNITS]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            rc = proc.returncode
            log += "\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        with open(os.path.join(HERE, "libcats_b200.buildlog"), "w") as f:
            f.write(log)
        if rc != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("nvcc failed:\n" + log[-6000:])
        if verbose:
            print(log)
        os.replace(tmp, LIB_PATH)
        with open(STAMP_PATH, "w") as f:
            f.write(source_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
