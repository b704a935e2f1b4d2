"""Import name of the package whose files live in the folder ``kestrel-llm_b200/``.

A hyphen cannot appear in a Python module name, so this stub points the package's search path
at that folder and runs its ``__init__.py``; every submodule (``kestrel_llm_b200.config`` ...)
is then found there.
"""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "kestrel-llm_b200")
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _f
