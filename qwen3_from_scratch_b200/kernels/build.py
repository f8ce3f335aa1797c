"""Compiles the CUDA sources of ``csrc/`` for sm_100a into one shared library.

The library is built in-tree (``<package>/_build/``) the first time it is needed
and again whenever a source file or a flag changes (content hash, not time
stamps).  When the package directory cannot be written, a per-user directory
under the system's temporary folder is used instead.  Compilation needs only
``nvcc``; no Python headers, no torch headers.  It prints a line per file to
stderr so that a first call that compiles does not look hung.

There is no fallback: without the library the engine does not run.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(PACKAGE_DIR, "csrc")
LIB_NAME = "libq3b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[q3b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def source_files() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _header_files() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)
                  if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in source_files() + _header_files():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _candidate_dirs() -> List[str]:
    dirs = [os.path.join(PACKAGE_DIR, "_build")]
    env = os.environ.get("Q3B200_BUILD_DIR")
    if env:
        dirs.insert(0, env)
    dirs.append(os.path.join(tempfile.gettempdir(), f"q3b200-build-{os.getuid()}"))
    return dirs


def _is_current(build_dir: str, want: str) -> bool:
    meta = os.path.join(build_dir, "build.json")
    lib = os.path.join(build_dir, LIB_NAME)
    if not (os.path.isfile(meta) and os.path.isfile(lib)):
        return False
    try:
        with open(meta) as f:
            return json.load(f).get("hash") == want
    except (OSError, ValueError):
        return False


def _writable_dir() -> str:
    last = None
    for d in _candidate_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            return d
        except OSError as e:
            last = e
    raise BuildError(f"no writable build directory among {_candidate_dirs()}: {last}")


def _compile_one(nvcc: str, src: str, obj: str, verbose_ptxas: bool) -> str:
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-I", CSRC_DIR, "-c", src, "-o", obj]
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
    _log(f"compiled {os.path.basename(src)} in {time.time() - t0:.1f}s")
    return proc.stderr


def build_library(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Returns the path of an up-to-date library, compiling it if needed."""
    want = source_hash()
    if not force:
        for d in _candidate_dirs():
            if _is_current(d, want):
                return os.path.join(d, LIB_NAME)
    nvcc = find_nvcc()
    if nvcc is None:
        raise BuildError(
            "the CUDA kernels are not built and nvcc was not found (set NVCC or CUDA_HOME); "
            "this engine has no CPU or library fallback")
    build_dir = _writable_dir()
    srcs = source_files()
    _log(f"compiling {len(srcs)} CUDA files for sm_100a into {build_dir} (first call only)")
    objs = [os.path.join(build_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with ThreadPoolExecutor(workers) as pool:
        logs = list(pool.map(lambda so: _compile_one(nvcc, so[0], so[1], verbose_ptxas), zip(srcs, objs)))
    tmp_lib = os.path.join(build_dir, f".{LIB_NAME}.{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", tmp_lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, os.path.join(build_dir, LIB_NAME))
    with open(os.path.join(build_dir, "build.json"), "w") as f:
        json.dump({"hash": want, "flags": NVCC_FLAGS, "sources": [os.path.basename(s) for s in srcs]}, f)
    if verbose_ptxas:
        with open(os.path.join(build_dir, "ptxas.log"), "w") as f:
            f.write("\n".join(logs))
    _log("done")
    return os.path.join(build_dir, LIB_NAME)


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv))
