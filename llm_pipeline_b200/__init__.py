"""Importable name of the package whose sources live in the folder ``llm-pipeline_b200/``.

A hyphen cannot appear in a Python module name, so this module points its ``__path__`` at that
folder and runs the folder's ``__init__.py`` in its own namespace; ``import llm_pipeline_b200.engine``
then resolves to ``llm-pipeline_b200/engine``.
"""

import os as _os

_real = _os.path.normpath(_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), _os.pardir, "llm-pipeline_b200"))
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _f
