"""Import name of the package that lives in the folder `sglang.c_b200/`.

A folder with a dot in its name cannot be imported directly, so this module
presents it as the package `sglang_c_b200`: it sets `__path__` to that folder
(which makes `import sglang_c_b200.engine` and the like work) and runs the
folder's `__init__.py` in its own namespace.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "sglang.c_b200")]
_init = _os.path.join(__path__[0], "__init__.py")
with open(_init) as _f:
    exec(compile(_f.read(), _init, "exec"))
del _f, _init
