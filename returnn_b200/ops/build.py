"""
Build the native libraries in-tree:

- ``_build/librb200.so``: all CUDA kernels, compiled for sm_100a only
  (``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo``); nvcc cross-compiles without a GPU.
- ``_build/librb200_host.so`` and ``_build/librb200_atfork.so``: host-only helpers (g++).

``python -m returnn_b200.ops.build [--force] [--verbose]``. Sources are compiled in parallel; objects are cached by
source + header modification times.
"""

from __future__ import annotations
from typing import List, Optional
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
_BUILD = os.path.join(_HERE, "_build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _newer(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd: List[str], verbose: bool):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    out = res.stdout.decode()
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), out))
    if verbose and out.strip():
        print(out)
    return out


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """compile every ``csrc/*.cu`` and link ``librb200.so``"""
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found")
    os.makedirs(_BUILD, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(_CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(_CSRC, "*.cuh")) + glob.glob(os.path.join(_CSRC, "*.h")))
    objs = []
    jobs = []
    for src in sources:
        obj = os.path.join(_BUILD, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-I", _CSRC, "-c", src, "-o", obj]
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            outs = list(ex.map(lambda c: _run(c, verbose), jobs))
        if ptxas_info:
            for o in outs:
                print(o)
    lib = os.path.join(_BUILD, "librb200.so")
    if jobs or force or _newer(lib, objs):
        _run([nvcc, "-shared", "-o", lib] + objs, verbose)
    return lib


def build_host(force: bool = False, verbose: bool = False) -> List[str]:
    """compile ``csrc/host/*.cpp`` into the host helper libraries"""
    os.makedirs(_BUILD, exist_ok=True)
    host_dir = os.path.join(_CSRC, "host")
    res = []
    if not os.path.isdir(host_dir):
        return res
    gxx = shutil.which("g++") or "g++"
    main_srcs = sorted(s for s in glob.glob(os.path.join(host_dir, "*.cpp")) if not os.path.basename(s).startswith("atfork"))
    if main_srcs:
        lib = os.path.join(_BUILD, "librb200_host.so")
        if force or _newer(lib, main_srcs):
            _run([gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-o", lib] + main_srcs + ["-ldl", "-lpthread"], verbose)
        res.append(lib)
    # CPython extension with the frontend's dimension bookkeeping (needs the Python headers)
    pyext = os.path.join(_CSRC, "pyext", "rf_native.cpp")
    if os.path.exists(pyext):
        import sysconfig

        inc = sysconfig.get_paths().get("include")
        if inc and os.path.exists(os.path.join(inc, "Python.h")):
            lib = os.path.join(_BUILD, "_rf_native.so")
            if force or _newer(lib, [pyext]):
                _run([gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-I", inc, "-o", lib, pyext], verbose)
            res.append(lib)
    atfork = os.path.join(host_dir, "atfork_patch.cpp")
    if os.path.exists(atfork):
        lib = os.path.join(_BUILD, "librb200_atfork.so")
        if force or _newer(lib, [atfork]):
            _run([gxx, "-O2", "-shared", "-fPIC", "-o", lib, atfork], verbose)
        res.append(lib)
    return res


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> List[str]:
    """everything"""
    libs = [build_cuda(force=force, verbose=verbose, ptxas_info=ptxas_info)]
    libs += build_host(force=force, verbose=verbose)
    return libs


if __name__ == "__main__":
    args = sys.argv[1:]
    for lib_path in build_all(force="--force" in args, verbose="--verbose" in args, ptxas_info="--ptxas-info" in args):
        print("built", lib_path)
