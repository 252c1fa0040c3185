"""Import alias for the package directory ``tpu-mlir_b200`` (its name is not a Python identifier).

``import tpu_mlir_b200`` gives the package; submodules import as ``tpu_mlir_b200.ops`` and so on.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "tpu-mlir_b200")]
with open(_os.path.join(__path__[0], "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
del _f
