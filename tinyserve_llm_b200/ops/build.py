"""
Builds the CUDA kernel library (csrc/*.cu) for sm_100a with nvcc and returns the path of the shared
object.  It is compiled at first use: one nvcc process per source file, a few at a time, with a
progress line printed meanwhile.  The library lands beside the package when that folder is
writable, otherwise under the temporary directory; a hash of sources and flags decides whether an
existing build is current.
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

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(PACKAGE_DIR, "csrc")
LIB_NAME = "libtinyserve_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]
LINK_FLAGS = ["-shared", "-cudart", "static"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        candidates.append(which)
    for c in candidates:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels cannot be compiled")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + LINK_FLAGS).encode())
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:20]


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dirs() -> list[str]:
    """Where the library may live, in order of preference."""
    dirs = []
    if os.environ.get("TINYSERVE_B200_BUILD_DIR"):
        dirs.append(os.environ["TINYSERVE_B200_BUILD_DIR"])
    dirs.append(os.path.join(PACKAGE_DIR, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"tinyserve_llm_b200-{os.getuid()}"))
    return dirs


def _log(msg: str) -> None:
    print(f"[tinyserve_llm_b200] {msg}", file=sys.stderr, flush=True)


def build_library(force: bool = False, verbose: bool = True) -> str:
    """Path of an up-to-date kernel library, compiling it if needed."""
    return _build_shared(LIB_NAME, sources(), source_hash(), force, verbose)


def build_extension(name: str, extra_sources: list[str], force: bool = False, verbose: bool = True) -> str:
    """
    Path of a shared library made of a part's own .cu files, compiled like the kernel library (same
    flags, csrc/ on the include path) together with csrc/library.cu, so that the extension reports
    errors through a `ts_last_error` of its own.
    """
    srcs = [os.path.abspath(p) for p in extra_sources] + [os.path.join(CSRC_DIR, "library.cu")]
    h = hashlib.sha256()
    h.update(source_hash().encode())          # flags and the headers an extension may include
    for path in srcs:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return _build_shared(f"libtinyserve_b200_{name}.so", srcs, h.hexdigest()[:20], force, verbose)


def _build_shared(lib_name: str, srcs: list[str], digest: str, force: bool, verbose: bool) -> str:
    for folder in build_dirs():
        lib, stamp = os.path.join(folder, lib_name), os.path.join(folder, lib_name + ".hash")
        if not force and os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return lib
    folder = next((d for d in build_dirs() if _writable(d)), None)
    if folder is None:
        raise BuildError(f"no writable folder for the kernel library among {build_dirs()}")
    nvcc = find_nvcc()
    obj_dir = os.path.join(folder, "obj-" + digest)
    os.makedirs(obj_dir, exist_ok=True)
    if verbose:
        _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {folder} (first use; about a minute)")
    done = [0]
    lock = threading.Lock()
    start = time.time()

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
        with lock:
            done[0] += 1
            if verbose:
                _log(f"  compiled {os.path.basename(src)} ({done[0]}/{len(srcs)}, {time.time() - start:.0f} s)")
        return obj

    stop = threading.Event()

    def heartbeat() -> None:
        while not stop.wait(10.0):
            if verbose:
                _log(f"  still compiling ({done[0]}/{len(srcs)} done, {time.time() - start:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        workers = max(1, min(len(srcs), os.cpu_count() or 4, 8))
        with ThreadPoolExecutor(workers) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp_lib = os.path.join(folder, f".{lib_name}.{os.getpid()}")
        proc = subprocess.run([nvcc, *LINK_FLAGS, "-o", tmp_lib, *objs], capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking the kernel library failed:\n{proc.stdout}\n{proc.stderr}")
        lib = os.path.join(folder, lib_name)
        os.replace(tmp_lib, lib)
        with open(os.path.join(folder, lib_name + ".hash"), "w") as f:
            f.write(digest)
    finally:
        stop.set()
    shutil.rmtree(obj_dir, ignore_errors=True)
    if verbose:
        _log(f"kernel library ready after {time.time() - start:.0f} s: {lib}")
    return lib
