"""Builds the package's two native libraries in-tree, at first use.

* ``libkestrel_host.so`` - the C++ host runtime under ``csrc/host`` (cache manager, scheduler,
  packer of a step's description), compiled by g++; it needs no GPU and no CUDA toolkit.
* ``libkestrel_cuda.so`` - every ``.cu`` under ``csrc/kernels`` compiled by nvcc for sm_100a
  (``-gencode arch=compute_100a,code=sm_100a``); kernels take raw pointers and a stream, so no
  framework headers are needed and a file compiles in seconds.  It holds the step runner too,
  which calls the cache manager, so it links against ``libkestrel_host.so`` (found beside it).

A library is rebuilt when the hash of its sources changes.  The build folder is
``csrc/_build`` inside the package; if the package folder cannot be written (a read-only
install) a per-user folder under the system's temporary directory is used instead.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

_HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_DIR = os.path.join(_HERE, "kernels")
HOST_DIR = os.path.join(_HERE, "host")
HEADER = os.path.join(os.path.dirname(_HERE), "include", "kestrel.h")     # the one C header of both libraries

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[kestrel build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"kestrel_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _sources(folder: str, exts) -> List[str]:
    return sorted(os.path.join(folder, n) for n in os.listdir(folder) if n.endswith(tuple(exts)))


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "kernels of this engine cannot be built, and there is no fallback")


def _run(cmd: List[str], what: str) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{r.stdout}")


def _fresh(lib: str, stamp: str, digest: str) -> bool:
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def build_cuda(verbose: bool = True) -> str:
    """Path of libkestrel_cuda.so, compiling it if its sources changed."""
    host_lib = build_host(verbose)
    out = os.path.dirname(host_lib)
    srcs = _sources(KERNEL_DIR, (".cu",))
    deps = srcs + _sources(KERNEL_DIR, (".cuh", ".h")) + [HEADER]
    flags = NVCC_FLAGS + os.environ.get("KESTREL_NVCC_EXTRA", "").split()      # e.g. -DAM_KEYS_STAGES=2 for experiments
    digest = _digest(deps, flags)
    lib = os.path.join(out, "libkestrel_cuda.so")
    stamp = lib + ".stamp"
    if _fresh(lib, stamp, digest):
        return lib
    nvcc = _find_nvcc()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out} (first call only)")
    objs = []

    def one(src: str) -> str:
        obj = os.path.join(out, os.path.basename(src)[:-3] + f".{digest}.o")
        _run([nvcc] + flags + ["-c", src, "-o", obj], f"nvcc {os.path.basename(src)}")
        if verbose:
            _say(f"  {os.path.basename(src)} done ({time.time() - t0:.0f} s)")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(one, srcs))
    tmp = lib + f".tmp{os.getpid()}"
    _run([nvcc, "-shared", "-o", tmp] + objs + ["-L" + out, "-lkestrel_host", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"],
         "link libkestrel_cuda.so")
    os.replace(tmp, lib)
    for o in objs:
        os.remove(o)
    with open(stamp, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"libkestrel_cuda.so ready ({time.time() - t0:.0f} s)")
    return lib


def build_host(verbose: bool = True) -> str:
    """Path of libkestrel_host.so, compiling it if its sources changed."""
    out = build_dir()
    srcs = _sources(HOST_DIR, (".cpp",))
    deps = srcs + _sources(HOST_DIR, (".h", ".hpp")) + [HEADER, os.path.join(KERNEL_DIR, "step_checks.cuh")]
    digest = _digest(deps, GXX_FLAGS)
    lib = os.path.join(out, "libkestrel_host.so")
    stamp = lib + ".stamp"
    if _fresh(lib, stamp, digest):
        return lib
    gxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not gxx:
        raise BuildError("no C++ compiler (g++) found for the host runtime")
    if verbose:
        _say(f"compiling the host runtime ({len(srcs)} files) into {out}")
    tmp = lib + f".tmp{os.getpid()}"
    _run([gxx] + GXX_FLAGS + ["-o", tmp] + srcs, "g++ host runtime")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib


def build_all(verbose: bool = True) -> None:
    build_host(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all()
