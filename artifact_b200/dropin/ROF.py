"""Drop-in for upstream's compiled module `ROF` (ROF/reuse_conv/setup.py:8): put this
directory on sys.path where upstream's scripts put `reuse_conv/` (ROF_evaluation/ROF_main.py:16)
and `import ROF` resolves here."""
import os as _os
import sys as _sys

_root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _root not in _sys.path:
    _sys.path.insert(0, _root)

from artifact_b200.ops import (SAG, GNNA_forward, GNNA_backward, reuse_forward_v1, reuse_backward_v1,  # noqa: E402,F401
                               reuse_forward_v2, reuse_backward_v2)
