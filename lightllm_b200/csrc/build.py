"""Compiles the kernel library for sm_100a with nvcc and finds it again.

The library is plain CUDA with ``extern "C"`` entry points (no Python or torch headers), so a
full build takes well under a minute.  It is built in-tree
(``lightllm_b200/csrc/_build/liblightllm_b200.so``) when that folder can be written, else under
the system's temporary folder, and rebuilt when a source file or a flag changes.  While nvcc
runs a line is printed every few seconds so that a first call does not look hung.
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
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "liblightllm_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the kernel library cannot be built")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC_DIR, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + os.environ.get("LLB_NVCC_EXTRA", "").split()).encode())
    return h.hexdigest()[:16]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    in_tree = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(in_tree):
        return in_tree
    alt = os.path.join(tempfile.gettempdir(), f"lightllm_b200-build-{os.getuid()}")
    if _writable_dir(alt):
        return alt
    raise BuildError(f"neither {in_tree} nor {alt} can be written; the kernel library cannot be built")


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, building it first if needed."""
    bdir = build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "fingerprint.txt")
    fp = _fingerprint()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return lib
    if not build:
        raise BuildError(f"{lib} is missing or stale and building was not allowed")
    _build(bdir, lib, verbose)
    with open(stamp, "w") as f:
        f.write(fp)
    return lib


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError("command failed: " + " ".join(cmd) + "\n" + proc.stdout)
    if os.environ.get("LLB_BUILD_VERBOSE") and proc.stdout.strip():
        print(proc.stdout, file=sys.stderr)


def _build(bdir: str, lib: str, verbose: bool) -> None:
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()
    done = threading.Event()
    finished: List[str] = []

    def heartbeat() -> None:
        while not done.wait(5.0):
            print(f"[lightllm_b200] compiling CUDA kernels for sm_100a: {len(finished)}/{len(srcs)} files, "
                  f"{time.time() - t0:.0f} s", file=sys.stderr, flush=True)

    if verbose:
        print(f"[lightllm_b200] building {LIB_NAME} ({len(srcs)} files) in {bdir}", file=sys.stderr, flush=True)
        threading.Thread(target=heartbeat, daemon=True).start()
    extra = os.environ.get("LLB_NVCC_EXTRA", "").split()
    try:
        objs = []

        def compile_one(src: str) -> str:
            obj = os.path.join(bdir, src[:-3] + ".o")
            _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj])
            finished.append(src)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart"])
        os.replace(tmp, lib)
    finally:
        done.set()
    if verbose:
        print(f"[lightllm_b200] built {LIB_NAME} in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)


HOST_DIR = os.path.join(CSRC_DIR, "host")
TOOL_NAME = "generate"


def tool_path(build: bool = True, verbose: bool = True) -> str:
    """Path of the C++ ``generate`` program (``csrc/host/generate.cpp``), built beside the kernel library and linked
    to it (it finds the library in its own folder).  It is rebuilt when its sources or the library's change."""
    lib = library_path(build, verbose)
    bdir = os.path.dirname(lib)
    tool = os.path.join(bdir, TOOL_NAME)
    stamp = os.path.join(bdir, "generate.fingerprint.txt")
    h = hashlib.sha256(_fingerprint().encode())
    for name in sorted(os.listdir(HOST_DIR)):
        if name.endswith((".cpp", ".h")):
            h.update(name.encode())
            with open(os.path.join(HOST_DIR, name), "rb") as f:
                h.update(f.read())
    fp = h.hexdigest()[:16]
    if os.path.isfile(tool) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return tool
    if not build:
        raise BuildError(f"{tool} is missing or stale and building was not allowed")
    if verbose:
        print(f"[lightllm_b200] building {TOOL_NAME} in {bdir}", file=sys.stderr, flush=True)
    tmp = tool + f".tmp{os.getpid()}"
    _run([_nvcc(), "-O2", "-std=c++17", "-I", CSRC_DIR, os.path.join(HOST_DIR, "generate.cpp"), "-o", tmp,
          "-L", bdir, "-l:" + LIB_NAME, "-lcudart", "-Xlinker", "-rpath=$ORIGIN"])
    os.replace(tmp, tool)
    with open(stamp, "w") as f:
        f.write(fp)
    return tool


if __name__ == "__main__":
    print(library_path())
    print(tool_path())
