"""B200-native tail-biting trellis codec: drop-in for the tile codec of Azimml/trellis-everywhere.

Add the folder that contains this package to ``sys.path`` (the reference does the same
with its ``src/`` folder) and import ``trellis_b200.qtip`` / ``trellis_b200.ldlq`` where
the reference imports ``trellis.qtip`` / ``trellis.ldlq``.
"""
from . import _lib  # noqa: F401  (importing the package does not load the .so; the first call does)

__all__ = ["qtip", "ldlq", "quant", "dist"]
