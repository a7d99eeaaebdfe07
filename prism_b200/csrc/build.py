"""Builds the CUDA sources of this directory into one shared library for
sm_100a with nvcc, in-tree (``csrc/_build/libprism_kernels.so``), and loads
nothing: ``prism_b200.ops`` opens the result with ctypes.

The sources include no framework headers, so a full build is seconds per
file.  A manifest beside the library records a hash of the sources and
flags; the build is skipped when it matches.  When the package directory is
not writable the build goes to a per-user folder under the system's
temporary directory instead.
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

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libprism_kernels.so"

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
NVCC_FLAGS += os.environ.get("PRISM_NVCC_EXTRA", "").split()      # experiments: extra -D flags
LINK_LIBS = []


class BuildError(RuntimeError):
    pass


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    cands = [os.environ.get("PRISM_NVCC"), shutil.which("nvcc"),
             os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")]
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $PRISM_NVCC, PATH and $CUDA_HOME/bin); "
                     "the CUDA kernels of prism_b200 cannot be built")


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + LINK_LIBS).encode())
    return h.hexdigest()


def build_dir() -> str:
    d = os.environ.get("PRISM_BUILD_DIR") or os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"prism_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(check: bool = True):
    """Path of an up-to-date library, or None."""
    want = source_hash()
    for d in (os.environ.get("PRISM_BUILD_DIR") or os.path.join(CSRC, "_build"),
              os.path.join(tempfile.gettempdir(), f"prism_b200_build_{os.getuid()}")):
        lib, man = os.path.join(d, LIB_NAME), os.path.join(d, "manifest.json")
        if os.path.isfile(lib) and os.path.isfile(man):
            try:
                with open(man) as f:
                    if not check or json.load(f).get("hash") == want:
                        return lib
            except (OSError, ValueError):
                pass
    return None


def _say(msg: str, verbose: bool):
    if verbose:
        print(f"[prism_b200 build] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False, ptxas_info: bool = False) -> str:
    """Compile what is stale and return the library's path."""
    if not force:
        lib = library_path()
        if lib:
            return lib
    nvcc = find_nvcc()
    out = build_dir()
    srcs = sources()
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out}", verbose)
    hdr_hash = hashlib.sha256()
    for f in _headers():
        with open(os.path.join(CSRC, f), "rb") as fh:
            hdr_hash.update(fh.read())
    hdr_hash.update(" ".join(NVCC_FLAGS).encode())
    objman_path = os.path.join(out, "objects.json")
    try:
        with open(objman_path) as f:
            objman = json.load(f)
    except (OSError, ValueError):
        objman = {}
    done = [0]
    lock = threading.Lock()

    def one(src: str):
        obj = os.path.join(out, src[:-3] + ".o")
        with open(os.path.join(CSRC, src), "rb") as fh:
            key = hashlib.sha256(fh.read() + hdr_hash.digest()).hexdigest()
        if not force and objman.get(src) == key and os.path.isfile(obj):
            return src, key, ""
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
              ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{p.stderr[-4000:]}")
        with lock:
            done[0] += 1
            _say(f"  [{done[0]}] {src} ({time.time() - t0:.0f}s)", verbose)
        return src, key, p.stderr

    logs = {}
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for src, key, log in ex.map(one, srcs):
            objman[src] = key
            logs[src] = log
    with open(objman_path, "w") as f:
        json.dump(objman, f)
    lib = os.path.join(out, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp] + [os.path.join(out, s[:-3] + ".o") for s in srcs] + LINK_LIBS
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"link failed:\n{p.stderr[-4000:]}")
    os.replace(tmp, lib)
    with open(os.path.join(out, "manifest.json"), "w") as f:
        json.dump({"hash": source_hash(), "sources": srcs}, f)
    _say(f"built {lib} in {time.time() - t0:.0f}s", verbose)
    if ptxas_info:
        for s, l in logs.items():
            if l:
                print(f"==== {s}\n{l}")
    return lib


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
