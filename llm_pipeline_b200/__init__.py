"""Importable name, in a checkout, of the package whose sources live in the folder ``llm-pipeline_b200/``.

A hyphen cannot appear in a Python module name. An installed copy maps the folder to this name (``pyproject.toml``,
``package-dir``); in a checkout this module loads the folder's ``__init__.py`` as the package ``llm_pipeline_b200``
through importlib's own loader and puts it in its place, so that ``import llm_pipeline_b200.engine`` resolves to
``llm-pipeline_b200/engine``.
"""

import importlib.util as _util
import os as _os
import sys as _sys

_real = _os.path.normpath(_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), _os.pardir, "llm-pipeline_b200"))
_spec = _util.spec_from_file_location(__name__, _os.path.join(_real, "__init__.py"), submodule_search_locations=[_real])
_module = _util.module_from_spec(_spec)
_sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
