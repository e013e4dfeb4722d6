"""
Compile C / C++ / CUDA source text on the fly into a shared library with a content-addressed cache directory.

The cache key covers the code, the compiler options and the versions that matter; concurrent compilations of the same key
are serialised by a lock directory; an ``info.py`` next to the library records how it was built. The framework's own
kernels do not go through this (they are built ahead of time, in-tree, by ``returnn_b200/ops/build.py``); this class
serves user ops (``tools/compile_native_op.py``) and the host helpers.

Parity: returnn/util/native_code_compiler.py (NativeCodeCompiler :15, get_cc_bin :376, get_cpp_bin :393),
returnn/util/py_ext_mod_compiler.py.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import time


def get_cc_bin() -> str:
    """C compiler: ``$CC`` or the first of clang/gcc/cc on PATH"""
    return _find_bin("CC", ["gcc", "clang", "cc"])


def get_cpp_bin() -> str:
    """C++ compiler: ``$CXX`` or the first of g++/clang++/c++ on PATH"""
    return _find_bin("CXX", ["g++", "clang++", "c++"])


def _find_bin(env: str, names: Sequence[str]) -> str:
    v = os.environ.get(env)
    if v:
        return v
    for n in names:
        p = shutil.which(n)
        if p:
            return p
    raise RuntimeError("no compiler found (tried $%s, %s)" % (env, ", ".join(names)))


class NativeCodeCompiler:
    """source text -> cached ``.so``"""

    CacheDirName = "returnn_b200_native"
    CollectedCompilers: Optional[List["NativeCodeCompiler"]] = None
    _cleanup_time_limit_days = 60

    def __init__(self, base_name: str, *, code_version: Union[int, Tuple[int, ...]] = 1, code: str, is_cpp: bool = True,
                 is_cuda: bool = False, c_macro_defines: Optional[Dict[str, Union[str, int, None]]] = None, ld_flags: Optional[Sequence[str]] = None,
                 include_paths: Optional[Sequence[str]] = (), include_deps: Optional[Sequence[str]] = None, static_version_name: Optional[str] = None,
                 should_cleanup_old_all: bool = True, should_cleanup_old_mydir: bool = False, use_cxx11_abi: bool = True, log_stream=None,
                 verbose: Optional[bool] = None):
        """
        :param base_name: name of the module, e.g. ``"my_op"``
        :param code_version: part of the cache key
        :param code: the source
        :param is_cpp: C++ (else C); ``is_cuda``: compile with nvcc for sm_100a
        :param c_macro_defines: ``-D`` definitions (None values are skipped)
        :param include_deps: files whose modification invalidates the cached library
        :param static_version_name: directory name instead of the hash
        """
        if NativeCodeCompiler.CollectedCompilers is not None:
            NativeCodeCompiler.CollectedCompilers.append(self)
        from .basic import get_cache_dir

        self.verbose = (os.environ.get("RETURNN_NATIVE_CODE_COMPILER_VERBOSE") == "1") if verbose is None else verbose
        self.cache_dir = os.path.join(get_cache_dir(), self.CacheDirName)
        self.base_name = base_name
        self.code_version = code_version
        self.code = code
        self.is_cpp = is_cpp
        self.is_cuda = is_cuda
        self.c_macro_defines = {k: v for k, v in (c_macro_defines or {}).items() if v is not None}
        self.ld_flags = list(ld_flags or [])
        self._include_paths = list(include_paths or [])
        self.include_deps = include_deps
        self.static_version_name = static_version_name
        self.use_cxx11_abi = use_cxx11_abi
        self._log_stream = log_stream
        self._ctypes_lib = None
        key = repr((base_name, code_version, hashlib.sha256(code.encode("utf8")).hexdigest(), is_cpp, is_cuda, sorted(self.c_macro_defines.items()),
                    self.ld_flags, self._include_paths, use_cxx11_abi, sys.version_info[:2]))
        self._hash = hashlib.sha256(key.encode("utf8")).hexdigest()[:16]
        if should_cleanup_old_all:
            self._cleanup_old()
        if should_cleanup_old_mydir and os.path.isdir(self._mod_path) and not self._need_recompile():
            pass
        self._maybe_compile()

    # -- paths -------------------------------------------------------------------------------------------------------
    @property
    def _mod_path(self) -> str:
        return os.path.join(self.cache_dir, self.base_name, self.static_version_name or self._hash)

    @property
    def _so_filename(self) -> str:
        return os.path.join(self._mod_path, "%s.so" % self.base_name)

    @property
    def _src_filename(self) -> str:
        ext = "cu" if self.is_cuda else ("cc" if self.is_cpp else "c")
        return os.path.join(self._mod_path, "%s.%s" % (self.base_name, ext))

    @property
    def _info_filename(self) -> str:
        return os.path.join(self._mod_path, "info.py")

    def get_lib_filename(self) -> str:
        """:return: path of the compiled library"""
        return self._so_filename

    # -- cache maintenance -------------------------------------------------------------------------------------------
    def _cleanup_old(self):
        base = self.cache_dir
        if not os.path.isdir(base):
            return
        limit = time.time() - self._cleanup_time_limit_days * 86400
        for op in os.listdir(base):
            op_dir = os.path.join(base, op)
            if not os.path.isdir(op_dir):
                continue
            for h in os.listdir(op_dir):
                d = os.path.join(op_dir, h)
                info = os.path.join(d, "info.py")
                try:
                    if os.path.isfile(info) and os.path.getmtime(info) < limit:
                        shutil.rmtree(d, ignore_errors=True)
                except OSError:
                    pass

    def _need_recompile(self) -> bool:
        if not os.path.isfile(self._so_filename) or not os.path.isfile(self._info_filename):
            return True
        if self.include_deps:
            so_time = os.path.getmtime(self._so_filename)
            for dep in self.include_deps:
                if os.path.exists(dep) and os.path.getmtime(dep) > so_time:
                    return True
        try:
            info = eval(open(self._info_filename).read(), {"__builtins__": {}})
        except Exception:
            return True
        return info.get("hash") != self._hash
    # -- compile -----------------------------------------------------------------------------------------------------
    def _get_compiler_opts(self) -> List[str]:
        opts = ["-O2", "-shared"]
        if self.is_cuda:
            opts += ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC", "-std=c++17"]
        else:
            opts += ["-fPIC"] + (["-std=c++17"] if self.is_cpp else [])
        for k, v in sorted(self.c_macro_defines.items()):
            opts.append("-D%s=%s" % (k, v) if v != "" else "-D%s" % k)
        if self.is_cpp and not self.is_cuda:
            opts.append("-D_GLIBCXX_USE_CXX11_ABI=%i" % (1 if self.use_cxx11_abi else 0))
        for p in self._include_paths:
            opts += ["-I", p]
        return opts

    def _get_compiler_bin(self) -> str:
        if self.is_cuda:
            nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            if not os.path.exists(nvcc):
                raise RuntimeError("nvcc not found")
            return nvcc
        return get_cpp_bin() if self.is_cpp else get_cc_bin()

    def _maybe_compile(self):
        if not self._need_recompile():
            if self.verbose:
                print("%s: cached %s" % (type(self).__name__, self._so_filename), file=self._log_stream or sys.stderr)
            os.utime(self._info_filename, None)  # mark as used for the cleanup
            return
        os.makedirs(self._mod_path, exist_ok=True)
        lock = os.path.join(self._mod_path, "lock")
        t0 = time.time()
        while True:
            try:
                os.mkdir(lock)
                break
            except FileExistsError:
                if time.time() - t0 > 600 or (os.path.exists(lock) and time.time() - os.path.getmtime(lock) > 900):
                    shutil.rmtree(lock, ignore_errors=True)  # stale lock of a dead process
                time.sleep(0.2)
        try:
            if not self._need_recompile():
                return
            with open(self._src_filename, "w") as f:
                f.write(self.code)
            cmd = [self._get_compiler_bin(), self._src_filename] + self._get_compiler_opts() + ["-o", self._so_filename + ".tmp"] + self.ld_flags
            if self.verbose:
                print("%s: %s" % (type(self).__name__, " ".join(cmd)), file=self._log_stream or sys.stderr)
            proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=self._mod_path)
            if proc.returncode != 0:
                raise RuntimeError("%s: compilation of %s failed:\n%s\n%s" % (type(self).__name__, self.base_name, " ".join(cmd), proc.stdout.decode("utf8", "replace")))
            os.replace(self._so_filename + ".tmp", self._so_filename)
            with open(self._info_filename, "w") as f:
                f.write(repr(self._make_info_dict(cmd)) + "\n")
        finally:
            shutil.rmtree(lock, ignore_errors=True)

    def _make_info_dict(self, cmd: Sequence[str] = ()) -> Dict[str, Any]:
        return {"base_name": self.base_name, "code_version": self.code_version, "hash": self._hash, "is_cpp": self.is_cpp, "is_cuda": self.is_cuda,
                "c_macro_defines": self.c_macro_defines, "ld_flags": self.ld_flags, "cmd": list(cmd), "time": time.strftime("%Y-%m-%d %H:%M:%S")}

    def load_lib_ctypes(self) -> ctypes.CDLL:
        """:return: the library via ctypes (loaded once)"""
        if self._ctypes_lib is None:
            self._ctypes_lib = ctypes.CDLL(self._so_filename)
        return self._ctypes_lib

    def __repr__(self):
        return "<%s %r in %r>" % (type(self).__name__, self.base_name, self._mod_path)


class PyExtModCompiler(NativeCodeCompiler):
    """compiles a CPython extension module (adds the Python include path) and imports it"""

    CacheDirName = "returnn_b200_py_ext_mod"

    def __init__(self, include_paths=(), **kwargs):
        import sysconfig

        py_inc = [p for p in {sysconfig.get_paths()["include"], sysconfig.get_paths().get("platinclude")} if p]
        super().__init__(include_paths=list(include_paths) + py_inc, **kwargs)
        self._py_mod = None

    def load_py_module(self):
        """:return: the imported extension module"""
        if self._py_mod is None:
            import importlib.util

            spec = importlib.util.spec_from_file_location(self.base_name, self._so_filename)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            self._py_mod = mod
        return self._py_mod
