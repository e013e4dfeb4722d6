"""
Packaging. The CUDA kernel library is built in-tree for sm_100a before the files are collected (``build_py`` runs
``returnn_b200.ops.build.build_all``), so the wheel ships ``returnn_b200/ops/_build/*.so``; without nvcc only the host
libraries are built and the package works on CPU.

    python setup.py build_ext --inplace     # only compile the native libraries in the tree
    python -m pip install --no-build-isolation .
"""

import os
import sys
from setuptools import setup, find_packages, Command
from setuptools.command.build_py import build_py as _build_py

_root = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _root)


def _build_native():
    from returnn_b200.ops import build

    libs = build.build_all(force=False, verbose=True)
    print("native libraries:", libs)


class build_ext(Command):
    """compile the native libraries into returnn_b200/ops/_build"""

    description = __doc__
    user_options = [("inplace", "i", "ignored: the libraries are always built in the tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class build_py(_build_py):
    """native build + version file, then the normal collection of the Python files"""

    def run(self):
        try:
            _build_native()
        except Exception as exc:  # a CPU-only install is still useful
            print("WARNING: native build failed: %s" % exc)
        from returnn_b200.__setup__ import get_version_str

        with open(os.path.join(_root, "returnn_b200", "_setup_info_generated.py"), "w") as f:
            f.write("version = %r\nlong_version = %r\n" % (get_version_str(), get_version_str(long=True)))
        super().run()


def _version():
    from returnn_b200.__setup__ import get_version_str

    return get_version_str(fallback="0.1.0")


setup(
    name="returnn-b200",
    version=_version(),
    description="Blackwell-native sequence-model training framework with the capability surface of RETURNN",
    long_description=open(os.path.join(_root, "README.md")).read(),
    long_description_content_type="text/markdown",
    packages=find_packages(include=["returnn_b200", "returnn_b200.*"]),
    package_data={"returnn_b200": ["ops/_build/*.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/host/*.cpp"]},
    include_package_data=True,
    python_requires=">=3.9",
    install_requires=["numpy", "torch"],
    extras_require={"hdf": ["h5py"], "audio": ["soundfile"], "spm": ["sentencepiece"]},
    entry_points={"console_scripts": ["returnn-b200=returnn_b200.__main__:main"]},
    cmdclass={"build_py": build_py, "build_ext": build_ext},
    classifiers=["Programming Language :: Python :: 3", "Environment :: GPU :: NVIDIA CUDA :: 12", "Topic :: Scientific/Engineering :: Artificial Intelligence"],
)
