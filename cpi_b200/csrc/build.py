"""Builds the CUDA kernel library for sm_100a with nvcc and returns the path of the shared object.

The library is plain `extern "C"` entry points (no Python or torch headers), so a build is one
nvcc call per source file plus a link, a few seconds each.  The object files and the library go to
`cpi_b200/csrc/_build/` when that folder can be written, otherwise to a per-user folder under the
system's temporary directory.  A build is reused while the sources' digest is unchanged.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libcpi_b200_kernels.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"cpi_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _nvcc() -> str:
    for cand in (os.environ.get("CPI_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("cpi_b200: nvcc was not found (PATH, /usr/local/cuda/bin, or CPI_B200_NVCC); "
                       "the kernel library cannot be built and there is no other compute path")


def library_path(build_if_missing: bool = True, verbose: bool = True) -> str:
    d = _build_dir()
    digest = _digest()
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "digest.txt")
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == digest:
        return lib
    if not build_if_missing:
        raise RuntimeError(f"cpi_b200: kernel library {lib} is missing or out of date")
    build(d, digest, verbose)
    return lib


def build(d: str | None = None, digest: str | None = None, verbose: bool = True) -> str:
    d = d or _build_dir()
    digest = digest or _digest()
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()

    def say(msg):
        if verbose:
            print(f"[cpi_b200 build] {msg}", file=sys.stderr, flush=True)

    say(f"compiling {len(srcs)} CUDA files for sm_100a into {d}")

    def compile_one(src):
        obj = os.path.join(d, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"cpi_b200: nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        say(f"  {src} done ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, srcs))
    lib = os.path.join(d, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"cpi_b200: linking the kernel library failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(os.path.join(d, "digest.txt"), "w") as f:
        f.write(digest)
    say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(library_path())
