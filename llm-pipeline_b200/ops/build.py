"""Builds the CUDA library of this package for sm_100a and loads it.

The sources under ``csrc/`` are compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
into one shared library, ``csrc/_build/libllmp_b200.so``, at the first call that needs a kernel
(or ahead of time by ``build_library()``). A stamp file holds a hash of the sources and flags, so
an unchanged tree is never compiled twice. When the package folder cannot be written, the build
goes to ``$LLMP_B200_BUILD_DIR`` or to a per-user folder under the system's temporary directory.
There is no fallback when the toolchain or the library is missing: the call raises.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "csrc"))
LIB_NAME = "libllmp_b200.so"
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_lib: Optional[ctypes.CDLL] = None


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[llm-pipeline_b200] {message}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:20]


def find_nvcc() -> str:
    for candidate in (os.environ.get("LLMP_B200_NVCC"), shutil.which("nvcc"),
                      os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                      "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc was not found (set LLMP_B200_NVCC or CUDA_HOME); the CUDA library of "
                     "llm-pipeline_b200 cannot be built and there is no other execution path")


def build_dir() -> str:
    override = os.environ.get("LLMP_B200_BUILD_DIR")
    candidates = [override] if override else [os.path.join(CSRC, "_build")]
    candidates.append(os.path.join(tempfile.gettempdir(), f"llmp_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}")


def build_library(force: bool = False, verbose: bool = True) -> str:
    """Compile (if needed) and return the path of the shared library."""
    out_dir = build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "stamp.txt")
    want = source_hash()
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(lib_path) and os.path.isfile(stamp_path):
                with open(stamp_path) as f:
                    if f.read().strip() == want:
                        return lib_path
            nvcc = find_nvcc()
            srcs = sources()
            start = time.time()
            if verbose:
                _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
            objs = [os.path.join(out_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]

            def job(pair):
                src, obj = pair
                _compile_one(nvcc, src, obj)
                if verbose:
                    _say(f"  compiled {os.path.basename(src)} ({time.time() - start:.0f} s)")

            with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
                list(pool.map(job, zip(srcs, objs)))
            tmp = lib_path + f".tmp{os.getpid()}"
            link = [nvcc, "-shared", "-o", tmp] + objs + ["-lcudart"]
            proc = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}")
            os.replace(tmp, lib_path)
            with open(stamp_path, "w") as f:
                f.write(want + "\n")
            if verbose:
                _say(f"built {LIB_NAME} in {time.time() - start:.0f} s")
            return lib_path
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def library() -> ctypes.CDLL:
    """The loaded library; builds it on first use."""
    global _lib
    if _lib is None:
        path = build_library()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from e
    return _lib
