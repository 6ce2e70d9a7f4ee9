"""Building the native libraries in the tree.

Two shared libraries are made from the sources beside this file:
``librmx_kernels.so`` (CUDA, compiled by nvcc for sm_100a only) and
``librmx_host.so`` (C++: cache manager and scheduler, no CUDA).  Objects and
libraries go to ``_build/`` here; a source is compiled again when its text, a header
or the flags change.  The first call in a fresh checkout compiles everything and
prints a line for every file, so that a caller who waits sees progress.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[rust_mlx_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels cannot be compiled (set NVCC or install CUDA 12.9)")


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(paths):
        with open(p, "rb") as fh:
            h.update(os.path.basename(p).encode())
            h.update(fh.read())
    return h.hexdigest()


def _sources(sub: str, ext: str) -> list:
    d = os.path.join(HERE, sub)
    return sorted(os.path.join(d, n) for n in os.listdir(d) if n.endswith(ext))


def _headers(sub: str) -> list:
    d = os.path.join(HERE, sub)
    return sorted(os.path.join(d, n) for n in os.listdir(d) if n.endswith((".cuh", ".h", ".hpp")))


def _run(cmd, what):
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}")
    return time.time() - t0, proc.stdout


def _build_library(name: str, sub: str, ext: str, compiler: list, flags: list, link: list, verbose: bool) -> str:
    os.makedirs(BUILD, exist_ok=True)
    lib = os.path.join(BUILD, name)
    with open(os.path.join(BUILD, name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        sources, headers = _sources(sub, ext), _headers(sub)
        stamp_path = lib + ".stamp"
        want = _digest(sources + headers, flags)
        if os.path.exists(lib) and os.path.exists(stamp_path) and open(stamp_path).read() == want:
            return lib
        _say(f"compiling {len(sources)} files for {name} (first call in this checkout, or sources changed)")
        jobs = []
        for src in sources:
            obj = os.path.join(BUILD, os.path.basename(src) + ".o")
            ostamp = obj + ".stamp"
            key = _digest([src] + headers, flags)
            if os.path.exists(obj) and os.path.exists(ostamp) and open(ostamp).read() == key:
                continue
            jobs.append((src, obj, ostamp, key))

        def compile_one(job):
            src, obj, ostamp, key = job
            dt, out = _run(compiler + flags + ["-c", src, "-o", obj], f"compiling {os.path.basename(src)}")
            with open(ostamp, "w") as fh:
                fh.write(key)
            _say(f"  {os.path.basename(src)} done in {dt:.1f}s")
            if verbose and out.strip():
                _say(out)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            list(pool.map(compile_one, jobs))
        objs = [os.path.join(BUILD, os.path.basename(s) + ".o") for s in sources]
        tmp = lib + f".tmp{os.getpid()}"
        _run(compiler + link + ["-shared", "-o", tmp] + objs, f"linking {name}")
        os.replace(tmp, lib)
        with open(stamp_path, "w") as fh:
            fh.write(want)
        _say(f"{name} ready")
    return lib


def build_kernels(verbose: bool = False) -> str:
    """Compile the CUDA kernels for sm_100a; returns the library's path."""
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    return _build_library("librmx_kernels.so", "kernels", ".cu", [find_nvcc()], flags,
                          ["-Xcompiler", "-fPIC", "-lcudart"], verbose)


def build_host(verbose: bool = False) -> str:
    """Compile the cache manager and scheduler (plain C++); returns the library's path."""
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++): the cache manager cannot be compiled")
    return _build_library("librmx_host.so", "host", ".cpp", [cxx], CXX_FLAGS, [], verbose)


def build_all(verbose: bool = False) -> dict:
    return {"host": build_host(verbose), "kernels": build_kernels(verbose)}


if __name__ == "__main__":
    print(build_all(verbose="-v" in sys.argv))
