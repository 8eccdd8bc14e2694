"""Import shim: makes the package in ./mamba.py_b200/ importable as `mamba_b200`.

The package directory carries the project's name, which contains a dot and therefore cannot be
written in an import statement.  This module turns itself into that package: it points its
search path at the directory and executes the directory's __init__.py in its own namespace.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "mamba.py_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__) as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f, _os
