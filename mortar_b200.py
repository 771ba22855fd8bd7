"""Import alias: the package directory name contains hyphens, so it cannot be named in an
``import`` statement.  ``import mortar_b200`` loads it and behaves as the package itself."""
import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
_pkg = importlib.import_module("morph-orchestrates-recursive-pruned-hierarchies_b200")
sys.modules[__name__] = _pkg
