"""Compiles the CUDA sources of this folder into one shared library for sm_100a.

The library is built in-tree (``csrc/_build/``) at its first use and reused while
the sources and flags stay the same (their hash is part of the file name).  Where
the tree cannot be written, a per-user folder under the system's temporary folder
is used instead.  A line is printed when each file starts and ends compiling, so a
first call does not look hung.
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
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    cands = [shutil.which("nvcc")]
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise RuntimeError("nvcc not found (looked on PATH, in $CUDA_HOME and in /usr/local/cuda/bin); "
                       "the kernel library cannot be built")


def source_hash() -> str:
    h = hashlib.sha256()
    for name in _sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> str:
    in_tree = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"rustyllm_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def library_path(root: Optional[str] = None) -> str:
    return os.path.join(root or _build_root(), f"librustyllm_b200_{source_hash()}.so")


def _say(msg: str) -> None:
    print(f"[rustyllm_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    t0 = time.time()
    _say(f"compiling {src} ...")
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = p.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {src} ({time.time() - t0:.0f} s)")
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    _say(f"compiled {src} in {time.time() - t0:.1f} s")


def build(force: bool = False, verbose: bool = True) -> str:
    """Build the library if it is not there yet; returns its path."""
    root = _build_root()
    lib = library_path(root)
    if os.path.isfile(lib) and not force:
        return lib
    nvcc = _find_nvcc()
    tag = source_hash()
    objdir = os.path.join(root, f"obj_{tag}")
    os.makedirs(objdir, exist_ok=True)
    srcs = _sources()
    _say(f"building {os.path.basename(lib)} from {len(srcs)} CUDA files for sm_100a")
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in srcs]
    workers = max(1, min(len(srcs), (os.cpu_count() or 2)))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as ex:
        futs = [ex.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
        for f in futs:
            f.result()
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"linking the kernel library failed:\n{p.stdout}")
    os.replace(tmp, lib)  # atomic: a concurrent process sees the old state or the whole file
    shutil.rmtree(objdir, ignore_errors=True)
    for old in os.listdir(root):   # libraries of earlier source states
        if old.startswith("librustyllm_b200_") and old.endswith(".so") and os.path.join(root, old) != lib:
            try:
                os.remove(os.path.join(root, old))
            except OSError:
                pass
    _say(f"built {lib}")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
