"""Import alias for the framework package.

The source tree lives in ``jdm-ghassan_v1_pro-_b200/`` (a directory name Python cannot
import directly because of the hyphens).  This module makes it importable as
``ghassan_b200``: the package search path is pointed at that directory and its
``__init__`` is executed in this namespace, so ``ghassan_b200.models`` etc. resolve to
the files there.
"""
import os as _os

_here = _os.path.dirname(_os.path.abspath(__file__))
_src = _os.path.join(_os.path.dirname(_here), "jdm-ghassan_v1_pro-_b200")
__path__ = [_src]
__file__ = _os.path.join(_src, "__init__.py")
with open(__file__, "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), __file__, "exec"))
