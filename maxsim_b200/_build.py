"""Builds ``libmaxsim_b200.so`` in-tree with nvcc for sm_100a.

The library is plain CUDA C++ with a C ABI (``include/maxsim_b200.h``); it does
not link against torch.  ``python -m maxsim_b200._build`` rebuilds it; the
package never builds implicitly at import time on a machine without nvcc, it
fails with an explicit error instead.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libmaxsim_b200.so"
STAMP_PATH = PKG_DIR / "libmaxsim_b200.stamp"

SOURCES = ["abi.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and Path(cand).exists() else None


def source_digest() -> str:
    h = hashlib.sha256()
    files = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh"))
    files.append(PKG_DIR.parent / "include" / "maxsim_b200.h")
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == source_digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources.  Several
    processes may call this at once (one per GPU): the build runs under a file
    lock, into a temporary name, and whoever comes second finds it done."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libmaxsim_b200.so")
    import fcntl

    with open(PKG_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current():
            return LIB_PATH
        tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
        cmd = [nvcc, *NVCC_FLAGS]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", str(tmp)] + [str(CSRC / s) for s in SOURCES]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        if verbose:
            sys.stderr.write(proc.stderr)
        os.replace(tmp, LIB_PATH)
        STAMP_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
