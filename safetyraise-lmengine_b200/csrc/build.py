"""Builds the two shared libraries of the package, in the source tree.

* ``libsrlm_runtime.so``: host runtime (cache manager, scheduler), g++.
* ``libsrlm_kernels.so``: CUDA kernels for sm_100a, nvcc.

A library is rebuilt when the hash of its sources and flags changes.  Nothing
is written outside the package folder unless that folder is read-only, in which
case a per-user folder under the system's temporary directory is used.  Progress
goes to stderr, one line per compiled file.
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

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall"]


def _say(msg: str) -> None:
    print(f"[srlm build] {msg}", file=sys.stderr, flush=True)


def lib_dir() -> str:
    d = os.path.join(PKG, "_lib")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"srlm_b200_lib_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _sources(sub: str, exts):
    d = os.path.join(HERE, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def _digest(paths, flags) -> str:
    h = hashlib.sha256(" ".join(flags).encode())
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _fresh(lib: str, digest: str) -> bool:
    stamp = lib + ".stamp"
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def _run(cmd, what):
    t0 = time.time()
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"building {what} failed:\n{' '.join(cmd)}\n{p.stdout}\n{p.stderr}")
    _say(f"{what} ({time.time() - t0:.1f}s)")


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the CUDA kernels "
                       "cannot be built, and there is no other implementation to fall back to")


_lock = threading.Lock()


def build_runtime(force: bool = False) -> str:
    with _lock:
        out = os.path.join(lib_dir(), "libsrlm_runtime.so")
        srcs = _sources("host", (".cpp",))
        hdrs = _sources("host", (".hpp", ".h"))
        digest = _digest(srcs + hdrs, CXX_FLAGS)
        if not force and _fresh(out, digest):
            return out
        cxx = os.environ.get("CXX") or shutil.which("g++") or "c++"
        tmp = out + f".{os.getpid()}.tmp"
        _run([cxx, *CXX_FLAGS, "-shared", *srcs, "-o", tmp], "host runtime")
        os.replace(tmp, out)
        with open(out + ".stamp", "w") as f:
            f.write(digest)
        return out


def build_kernels(force: bool = False) -> str:
    with _lock:
        out = os.path.join(lib_dir(), "libsrlm_kernels.so")
        srcs = _sources("kernels", (".cu",))
        hdrs = _sources("kernels", (".cuh", ".h"))
        digest = _digest(srcs + hdrs, NVCC_FLAGS)
        if not force and _fresh(out, digest):
            return out
        nvcc = find_nvcc()
        obj_dir = os.path.join(lib_dir(), "_build")
        os.makedirs(obj_dir, exist_ok=True)
        _say(f"compiling {len(srcs)} CUDA files for sm_100a (first call only)")
        hdr_digest = _digest(hdrs, NVCC_FLAGS)

        def compile_one(src):
            obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
            d = _digest([src], [hdr_digest])
            if not force and _fresh(obj, d):
                return obj
            _run([nvcc, *NVCC_FLAGS, "-c", src, "-o", obj], os.path.basename(src))
            with open(obj + ".stamp", "w") as f:
                f.write(d)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = out + f".{os.getpid()}.tmp"
        _run([nvcc, "-shared", *objs, "-o", tmp, "-lcudart_static", "-ldl", "-lrt", "-lpthread"],
             "link libsrlm_kernels.so")
        os.replace(tmp, out)
        with open(out + ".stamp", "w") as f:
            f.write(digest)
        return out


def build_all(force: bool = False):
    return build_runtime(force), build_kernels(force)


if __name__ == "__main__":
    print("\n".join(build_all(force="--force" in sys.argv)))
