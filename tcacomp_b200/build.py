"""Build tcacomp_b200/libtcab.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python -m tcacomp_b200.build [--force] [--jobs N]

Each .cu is compiled to an object in tcacomp_b200/_obj/ (in parallel), then
linked into one shared library beside this file. nvcc cross-compiles without a
GPU. The library links the static CUDA runtime and the driver API (libcuda is
resolved at load time on a GPU box; on a box without a driver the library still
loads and every compute entry point reports TCAB_ERR_CUDA).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libtcab.so")
HOST_LIB = os.path.join(HERE, "libtcab_host.so")  # the C++ builder mirror above the C ABI (csrc/host/)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", OBJ,
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the kernel library cannot be built")
    return exe


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    return cu, cpp


def _digest(path: str, deps: list[str]) -> str:
    h = hashlib.sha256()
    for p in [path] + deps:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _embed_kernel_text() -> None:
    """chain_kernels.cuh as a raw string literal for the run-time compiler (chain_jit.cu)."""
    text = open(os.path.join(CSRC, "chain_kernels.cuh")).read().replace("#pragma once\n", "")
    assert ")TCABSRC\"" not in text
    out = os.path.join(OBJ, "chain_kernels_text.inc")
    new = 'R"TCABSRC(' + text + ')TCABSRC"\n'
    if not os.path.exists(out) or open(out).read() != new:
        with open(out, "w") as f:
            f.write(new)


def _compile(src: str, force: bool, verbose: bool) -> str:
    """Compile one source to an object; skipped when the source and all headers are unchanged."""
    path = os.path.join(CSRC, src)
    headers = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    headers.append(os.path.join(HERE, "..", "include", "tcab.h"))
    obj = os.path.join(OBJ, src + ".o")
    stamp = obj + ".sha"
    dig = _digest(path, headers)
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj
    if src.endswith(".cu"):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
    else:
        cmd = ["g++"] + CXX_FLAGS + ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        with open(obj + ".log", "w") as f:
            f.write(r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{r.stderr[-4000:]}")
    with open(stamp, "w") as f:
        f.write(dig)
    return obj


def build(force: bool = False, jobs: int | None = None, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    _embed_kernel_text()
    cu, cpp = _sources()
    jobs = jobs or min(8, os.cpu_count() or 1)
    before = {s: os.path.getmtime(os.path.join(OBJ, s + ".o")) if os.path.exists(os.path.join(OBJ, s + ".o")) else 0
              for s in cu + cpp}
    with cf.ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), cu + cpp))
    changed = any(os.path.getmtime(o) != before[s] for o, s in zip(objs, cu + cpp))
    if force or changed or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking libtcab.so failed:\n{r.stderr[-4000:]}")
    build_host(force or changed)
    return LIB


def build_host(force: bool = False) -> str:
    """g++ build of csrc/host/*.cpp into libtcab_host.so, linked against libtcab.so beside it."""
    hdir = os.path.join(CSRC, "host")
    srcs = sorted(os.path.join(hdir, f) for f in os.listdir(hdir) if f.endswith(".cpp"))
    deps = srcs + [os.path.join(hdir, f) for f in os.listdir(hdir) if f.endswith(".h")] + \
           [os.path.join(HERE, "..", "include", "tcab.h"), os.path.join(HERE, "..", "include", "tcab_host.h")]
    if not force and os.path.exists(HOST_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(HOST_LIB) for d in deps):
        return HOST_LIB
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", HOST_LIB] + srcs + \
          ["-L" + HERE, "-ltcab", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building libtcab_host.so failed:\n{r.stderr[-4000:]}")
    return HOST_LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true", help="keep ptxas -v logs beside the objects")
    a = ap.parse_args(argv)
    print(build(a.force, a.jobs, a.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
