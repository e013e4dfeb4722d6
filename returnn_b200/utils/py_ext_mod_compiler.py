"""
Parity: returnn/util/py_ext_mod_compiler.py (PyExtModCompiler :12). The class lives next to its base class.
"""

from .native_code_compiler import PyExtModCompiler  # noqa: F401
