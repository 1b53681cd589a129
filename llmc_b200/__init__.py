"""Importable alias of the package stored in the directory ``llm.c_b200`` (whose name, containing a
dot, cannot be imported directly).  ``import llmc_b200`` executes that package in place."""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "llm.c_b200")
__path__ = [_real]
__file__ = _os.path.join(_real, "__init__.py")
with open(__file__) as _fh:
    exec(compile(_fh.read(), __file__, "exec"))
del _os, _fh, _real
