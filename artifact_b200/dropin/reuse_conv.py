"""Drop-in for upstream's ROF/reuse_conv/reuse_conv.py: `from reuse_conv import ROF_GCNConv`."""
import os as _os
import sys as _sys

_root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _root not in _sys.path:
    _sys.path.insert(0, _root)

from artifact_b200.reuse_conv import ROF_GCNConvFunc, ROF_GCNConv  # noqa: E402,F401
