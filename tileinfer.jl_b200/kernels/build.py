"""Compiles the CUDA sources of ``csrc/`` (kernels and their launchers) and the C++ sources of
``csrc/host/`` (the host runtime: the cache's books, the step planner, the decode loop) for sm_100a
into one shared library.

``nvcc`` is run once per source file, in parallel, and the objects are linked with the
static CUDA runtime, so the library depends on nothing but the driver. Objects and the
library live in ``csrc/_build/`` inside the source tree when that is writable, else in a
per-user folder under the system's temporary directory. A stamp of the sources' contents
decides whether anything has to be rebuilt. While compiling, a line is printed to stderr
every few seconds so that a first call does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libtileinfer_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels of "
                     "tileinfer_b200 cannot be built, and there is no fallback without them")


HOST = "host"          # the sub-folder of the host runtime's C++ files


def sources() -> list:
    """Paths relative to ``csrc/``: every ``.cu`` there and every ``.cpp`` of ``csrc/host/``."""
    host = os.path.join(CSRC, HOST)
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu")) + \
        sorted(os.path.join(HOST, f) for f in (os.listdir(host) if os.path.isdir(host) else []) if f.endswith(".cpp"))


def _stamp() -> str:
    h = hashlib.sha256()
    host = os.path.join(CSRC, HOST)
    files = [f for f in os.listdir(CSRC)] + [os.path.join(HOST, f) for f in (os.listdir(host) if os.path.isdir(host) else [])]
    for f in sorted(files):
        if f.endswith((".cu", ".cuh", ".h", ".cpp")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def build_dir() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"tileinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def is_current() -> bool:
    d = build_dir()
    try:
        with open(os.path.join(d, "stamp")) as f:
            return f.read().strip() == _stamp() and os.path.isfile(os.path.join(d, LIB_NAME))
    except OSError:
        return False


def build(verbose: bool = False, force: bool = False) -> str:
    """Build if needed; returns the path of the shared library."""
    if not force and is_current():
        return library_path()
    nvcc = find_nvcc()
    d = build_dir()
    srcs = sources()
    start = time.time()
    done = []
    stop = threading.Event()

    def progress():
        while not stop.wait(5.0):
            print(f"[tileinfer_b200] compiling CUDA kernels for sm_100a: {len(done)}/{len(srcs)} files, "
                  f"{time.time() - start:.0f} s", file=sys.stderr, flush=True)

    print(f"[tileinfer_b200] compiling {len(srcs)} CUDA files for sm_100a into {d}", file=sys.stderr, flush=True)
    reporter = threading.Thread(target=progress, daemon=True)
    reporter.start()

    def compile_one(src: str) -> str:
        obj = os.path.join(d, os.path.splitext(src)[0].replace(os.sep, "_") + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr:
            print(r.stderr, file=sys.stderr)
        done.append(src)
        return obj

    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = os.path.join(d, f".{LIB_NAME}.{os.getpid()}")
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, os.path.join(d, LIB_NAME))
        with open(os.path.join(d, "stamp"), "w") as f:
            f.write(_stamp())
    finally:
        stop.set()
    print(f"[tileinfer_b200] kernels built in {time.time() - start:.0f} s", file=sys.stderr, flush=True)
    return os.path.join(d, LIB_NAME)


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
