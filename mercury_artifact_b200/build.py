"""Build recipe for libmercury_b200.so (sm_100a only).

The library is built in-tree with plain ``nvcc -shared``: it links against the
CUDA runtime only (no torch, no Python), which is what keeps its exported
surface a C ABI.  ``python -m mercury_artifact_b200.build`` rebuilds it.
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
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libmercury_b200.so"
STAMP = PKG_DIR / "libmercury_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    return None


def is_current() -> bool:
    """Whether the library on disk was built from the sources on disk (digest stamp written by build())."""
    try:
        return LIB_PATH.exists() and STAMP.exists() and STAMP.read_text().strip() == _digest()
    except OSError:
        return False


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared library; no-op if up to date.

    Safe to call from several processes at once (the ranks of a job importing the package): the
    compile runs under an exclusive file lock into a temporary file that is renamed into place, so
    nobody ever loads a half-written library, and whoever gets the lock second finds it up to date."""
    import fcntl

    if not force and is_current():
        return LIB_PATH
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: libmercury_b200.so cannot be built")
    with open(PKG_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            digest = _digest()
            if not force and is_current():
                return LIB_PATH
            tmp = LIB_PATH.with_suffix(f".tmp{os.getpid()}.so")
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(tmp), *map(str, sources())]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
                print(" ".join(cmd), file=sys.stderr)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
            if verbose:
                print(res.stderr, file=sys.stderr)
            os.replace(tmp, LIB_PATH)
            STAMP.write_text(digest + "\n")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
