"""Import name of the engine in a checkout.  The sources live in the folder ``qwen25vl-lite_b200``
beside this one (a name Python cannot import); this module loads that folder as the package
``qwen25vl_lite`` and puts it in its own place in ``sys.modules``, so ``import qwen25vl_lite`` and
``python -m qwen25vl_lite.cli`` work without installation.  An installed copy needs none of this:
``pyproject.toml`` maps the folder to the package name."""

import importlib.util as _util
import os as _os
import sys as _sys

_src = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "qwen25vl-lite_b200")
_spec = _util.spec_from_file_location(__name__, _os.path.join(_src, "__init__.py"), submodule_search_locations=[_src])
_module = _util.module_from_spec(_spec)
_sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
