"""Compiles the library (the CUDA kernels for sm_100a and the C++ engine around
them) into one shared library, in the tree.

The library is built with nvcc alone (no PyTorch headers), so a first call in a
fresh checkout takes about a minute; while it compiles, a line is printed now and
then.  A record of the sources' hashes beside the library decides
whether it is still current.  The library lands in ``janas_b200/csrc/_build``
when that folder can be written and in a per-user folder under the system's
temporary directory otherwise.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
LIB_NAME = "libjanas_b200.so"
# folders of the package that hold sources of the library
SOURCE_DIRS = ("core", "config", "weights", "cache", "parts", "engine", "api", "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
                           "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    exe = shutil.which("nvcc")
    if exe is None:
        for cand in ("/usr/local/cuda/bin/nvcc", os.path.join(
                os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
            if os.path.isfile(cand):
                exe = cand
                break
    if exe is None:
        raise BuildError("janas_b200: nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda); "
                         "the kernels cannot be compiled")
    return exe


def sources() -> List[str]:
    """Every .cu and .cpp file of the library, as paths below the package."""
    out = []
    for d in SOURCE_DIRS:
        folder = os.path.join(PKG, d)
        if os.path.isdir(folder):
            out += [os.path.join(d, f) for f in os.listdir(folder) if f.endswith((".cu", ".cpp"))]
    return sorted(out)


def _fingerprint(nvcc: str) -> str:
    h = hashlib.sha256()
    for d in SOURCE_DIRS + (os.path.join("include", "janas_b200"),):
        folder = os.path.join(PKG, d)
        if not os.path.isdir(folder):
            continue
        for f in sorted(os.listdir(folder)):
            if f.endswith((".cu", ".cuh", ".h", ".cpp")):
                h.update(os.path.join(d, f).encode())
                with open(os.path.join(folder, f), "rb") as fh:
                    h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    try:
        ver = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
    except OSError:
        ver = ""
    h.update(ver.encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _build_dirs(fingerprint: str) -> List[str]:
    dirs = [os.path.join(CSRC, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"janas_b200_build_{uid}_{fingerprint[:16]}"))
    return dirs


def _current(build_dir: str, fingerprint: str) -> bool:
    rec = os.path.join(build_dir, "build.json")
    lib = os.path.join(build_dir, LIB_NAME)
    if not (os.path.isfile(rec) and os.path.isfile(lib)):
        return False
    try:
        with open(rec, "r", encoding="utf-8") as f:
            return json.load(f).get("fingerprint") == fingerprint
    except (OSError, json.JSONDecodeError):
        return False


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """The path of the current kernel library, compiling it first if it is
    missing or older than its sources."""
    nvcc: Optional[str]
    try:
        nvcc = _nvcc()
    except BuildError:
        nvcc = None
    fp = _fingerprint(nvcc) if nvcc else None
    if fp is not None:
        for d in _build_dirs(fp):
            if _current(d, fp):
                return os.path.join(d, LIB_NAME)
    else:
        # without a compiler a library that was shipped with the tree is taken as it is
        lib = os.path.join(CSRC, "_build", LIB_NAME)
        if os.path.isfile(lib):
            return lib
    if not build_if_needed:
        raise BuildError("janas_b200: the library has not been built")
    if nvcc is None:
        _nvcc()  # raises with the message
    for d in _build_dirs(fp):
        if _writable_dir(d):
            return _compile(nvcc, d, fp, verbose)
    raise BuildError("janas_b200: no folder to build the library in")


def _compile(nvcc: str, build_dir: str, fingerprint: str, verbose: bool) -> str:
    srcs = sources()
    t0 = time.time()
    done = [0]
    stop = threading.Event()

    def say(msg: str) -> None:
        if verbose:
            print(f"janas_b200: {msg}", file=sys.stderr, flush=True)

    def ticker() -> None:
        while not stop.wait(5.0):
            say(f"compiling, {done[0]} of {len(srcs)} files done, "
                f"{time.time() - t0:.0f} s")

    def one(src: str) -> str:
        obj = os.path.join(build_dir, src.replace(os.sep, "_").rsplit(".", 1)[0] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", os.path.join(PKG, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"janas_b200: nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        done[0] += 1
        return obj

    say(f"compiling {len(srcs)} files (kernels for sm_100a, engine) into {build_dir} "
        f"(first call only)")
    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(one, srcs))
        lib_tmp = os.path.join(build_dir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", lib_tmp] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"janas_b200: linking failed:\n{r.stdout}\n{r.stderr}")
        os.replace(lib_tmp, os.path.join(build_dir, LIB_NAME))
        with open(os.path.join(build_dir, "build.json"), "w", encoding="utf-8") as f:
            json.dump({"fingerprint": fingerprint, "sources": srcs, "flags": NVCC_FLAGS}, f)
    finally:
        stop.set()
    say(f"library built in {time.time() - t0:.0f} s")
    return os.path.join(build_dir, LIB_NAME)


if __name__ == "__main__":
    print(library_path())
