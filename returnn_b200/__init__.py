"""
returnn_b200: a Blackwell (sm_100a) native training framework with the capability surface of RETURNN.

Layout:

- :mod:`returnn_b200.config`, :mod:`returnn_b200.log`, :mod:`returnn_b200.__main__`: config-file driven entry point.
- :mod:`returnn_b200.tensor`: named-dimension ``Tensor`` / ``Dim``.
- :mod:`returnn_b200.frontend` (``rf``): module API, functional ops, encoder/decoder zoo.
- :mod:`returnn_b200.datasets`: dataset stack.
- :mod:`returnn_b200.torch`: engine, updater, distributed, data pipeline.
- :mod:`returnn_b200.ops`: hand-written sm_100a kernels and their autograd wrappers.
- :mod:`returnn_b200.parallel`: flat parameter arena, fused gradient all-reduce, parameter averaging.
- :mod:`returnn_b200.models`: flagship model builders (Conformer-CTC, BLSTM-CTC, AED, Transformer MT).
- :mod:`returnn_b200.utils`: generic helpers.

Existing RETURNN configs say ``import returnn.frontend as rf``. Call :func:`install_returnn_alias` (``rnn.py`` does it)
to make ``returnn`` / ``returnn.*`` resolve to this package.
"""

from __future__ import annotations

__version__ = "0.1.0"
__long_version__ = "0.1.0+b200"


def install_returnn_alias(force: bool = False) -> bool:
    """
    Make ``import returnn...`` resolve to this package (``returnn.util`` maps to ``returnn_b200.utils``).

    :param force: replace an already imported ``returnn`` package
    :return: whether the alias is active
    """
    from .utils.compat_alias import install

    return install(force=force)
