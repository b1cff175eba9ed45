"""Import name of the engine.  The sources live in the folder ``qwen25vl-lite_b200`` beside
this one (a name Python cannot import); this package points its search path there and runs
that folder's ``__init__.py``, so ``import qwen25vl_lite`` and ``python -m qwen25vl_lite.cli``
work from a checkout without installation."""

import os as _os

_src = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "qwen25vl-lite_b200")
__path__ = [_src]
with open(_os.path.join(_src, "__init__.py"), "r", encoding="utf-8") as _fh:
    exec(compile(_fh.read(), _os.path.join(_src, "__init__.py"), "exec"))
del _fh
