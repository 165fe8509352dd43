"""In-tree build of the sm_100a kernel library.

``python -m deberta_b200.build`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into one shared object next to the
package (``deberta_b200/_native/libdb200_kernels.so``). The library has a plain C ABI
and no dependency on libtorch, so a file compiles in seconds and nvcc can
cross-compile it on a machine without a GPU. A content hash of the sources is stored
beside the library; the build is skipped when nothing changed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_native"
LIB_PATH = OUT_DIR / "libdb200_kernels.so"
STAMP = OUT_DIR / "sources.sha256"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP.exists() and STAMP.read_text().strip() == source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the kernel library if it is missing or stale; return its path.

    Safe to call from every rank of a launch at once: one process builds under an exclusive file lock (objects go to a
    private directory, the library and its stamp are moved into place atomically), the others wait for the lock and
    then find the library current.
    """
    if not force and is_current():
        return LIB_PATH
    import fcntl

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    with open(OUT_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():  # another process built it while this one waited
                return LIB_PATH
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    import tempfile

    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    work = Path(tempfile.mkdtemp(prefix=".build-", dir=OUT_DIR))

    def compile_one(src: Path) -> Path:
        obj = work / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    try:
        digest = source_hash()
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
            objs = list(pool.map(compile_one, sources()))
        tmp_lib = work / LIB_PATH.name
        link = [nvcc, "-shared", "-o", str(tmp_lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if STAMP.exists():
            STAMP.unlink()  # never a stamp that vouches for a library it does not describe
        os.replace(tmp_lib, LIB_PATH)
        tmp_stamp = work / STAMP.name
        tmp_stamp.write_text(digest + "\n")
        os.replace(tmp_stamp, STAMP)
    finally:
        shutil.rmtree(work, ignore_errors=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
