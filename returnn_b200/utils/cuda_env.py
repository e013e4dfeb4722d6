"""
Where is CUDA: locate the toolkit (nvcc, headers, libraries) and report its version; used by the native code compiler and
by diagnostics.

Parity: returnn/util/cuda_env.py (CudaEnv :11, get_best_nvcc_path_for_cuda_version :273).
"""

from __future__ import annotations
from typing import List, Optional, Tuple
import os
import re
import shutil
import subprocess


def _valid_cuda_path(p: str) -> bool:
    return bool(p) and os.path.isfile(os.path.join(p, "bin", "nvcc")) and os.path.isdir(os.path.join(p, "include"))


def _parse_cuda_version_from_cuda_h(cuda_h_path: str) -> Tuple[int, int]:
    m = re.search(r"#define\s+CUDA_VERSION\s+(\d+)", open(cuda_h_path, errors="replace").read())
    if not m:
        raise ValueError("no CUDA_VERSION in %s" % cuda_h_path)
    v = int(m.group(1))
    return v // 1000, (v % 1000) // 10


def get_cuda_path_candidates_from_common_install_locations() -> List[str]:
    """``/usr/local/cuda*`` and ``/opt/cuda*``, newest first"""
    import glob

    cands = []
    for pat in ("/usr/local/cuda", "/usr/local/cuda-*", "/opt/cuda", "/opt/cuda-*"):
        cands += sorted(glob.glob(pat), reverse=True)
    return [c for c in cands if _valid_cuda_path(c)]


class CudaEnv:
    """the CUDA toolkit of this machine"""

    _instance: Optional["CudaEnv"] = None
    verbose_find_cuda = False

    def __init__(self):
        self.cuda_path: Optional[str] = None
        for cand in self._candidates():
            if self.verbose_find_cuda:
                print("CudaEnv: check", cand)
            if _valid_cuda_path(cand):
                self.cuda_path = cand
                break

    @staticmethod
    def _candidates() -> List[str]:
        cands = []
        for env in ("CUDA_HOME", "CUDA_PATH"):
            if os.environ.get(env):
                cands.append(os.environ[env])
        nvcc = shutil.which("nvcc")
        if nvcc:
            cands.append(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))))
        for p in os.environ.get("LD_LIBRARY_PATH", "").split(":"):
            if "cuda" in p:
                cands.append(os.path.dirname(p.rstrip("/")))
        return cands + get_cuda_path_candidates_from_common_install_locations()

    def is_available(self) -> bool:
        """a toolkit with nvcc was found"""
        return self.cuda_path is not None

    def get_cuda_version(self) -> Tuple[int, int]:
        """(major, minor) from cuda.h"""
        assert self.cuda_path
        return _parse_cuda_version_from_cuda_h(os.path.join(self.cuda_path, "include", "cuda.h"))

    def get_max_compute_capability(self) -> float:
        """highest ``sm_XX`` this nvcc can target"""
        out = subprocess.run([self.get_compiler_bin(), "--list-gpu-arch"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL).stdout.decode()
        caps = [int(m) for m in re.findall(r"compute_(\d+)", out)]
        return max(caps) / 10.0 if caps else 0.0

    def get_compiler_opts(self) -> List[str]:
        """include/lib options for a host compiler that links against the CUDA runtime"""
        assert self.cuda_path
        return ["-I", os.path.join(self.cuda_path, "include"), "-L", self.get_lib_dir_path(), "-x", "cu"]

    def get_lib_dir_path(self) -> str:
        """directory with libcudart"""
        assert self.cuda_path
        for d in ("lib64", "lib"):
            p = os.path.join(self.cuda_path, d)
            if os.path.isdir(p):
                return p
        return os.path.join(self.cuda_path, "lib64")

    def get_compiler_bin(self) -> str:
        """path of nvcc"""
        assert self.cuda_path
        return os.path.join(self.cuda_path, "bin", "nvcc")

    @classmethod
    def get_instance(cls) -> "CudaEnv":
        """process-wide instance"""
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance


def get_best_nvcc_path_for_cuda_version(cuda_version: Tuple[int, int]) -> str:
    """an nvcc whose toolkit has the given major version (closest minor), else the default one"""
    best, best_diff = None, None
    for cand in CudaEnv._candidates():
        if not _valid_cuda_path(cand):
            continue
        try:
            v = _parse_cuda_version_from_cuda_h(os.path.join(cand, "include", "cuda.h"))
        except (OSError, ValueError):
            continue
        if v[0] != cuda_version[0]:
            continue
        diff = abs(v[1] - cuda_version[1])
        if best is None or diff < best_diff:
            best, best_diff = cand, diff
    if best is None:
        return CudaEnv.get_instance().get_compiler_bin()
    return os.path.join(best, "bin", "nvcc")
