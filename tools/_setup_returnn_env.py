"""make the package importable when a tool is run from the source tree (as ``returnn_b200`` and under the ``returnn`` alias)"""

import os
import sys

_root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _root not in sys.path:
    sys.path.insert(0, _root)
import returnn_b200  # noqa: E402

returnn_b200.install_returnn_alias()
