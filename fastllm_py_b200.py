"""Import name of the package that lives in the folder `fastllm-py_b200/`.

A hyphen cannot be part of a Python module name, so this one-file module stands
in for the folder: it points its `__path__` at the folder and runs the folder's
`__init__.py`, which makes `import fastllm_py_b200` and
`from fastllm_py_b200.engine import Engine` work as for any package.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "fastllm-py_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
with open(_os.path.join(__path__[0], "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
del _os, _f
