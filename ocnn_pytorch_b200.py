"""Import shim: the package directory is named `ocnn-pytorch_b200`, which is not
a Python identifier.  `import ocnn_pytorch_b200` (with the repository root on
sys.path) loads that directory as the package `ocnn_pytorch_b200`."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'ocnn-pytorch_b200')
_spec = importlib.util.spec_from_file_location(
    'ocnn_pytorch_b200', os.path.join(_dir, '__init__.py'), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules['ocnn_pytorch_b200'] = _mod
_spec.loader.exec_module(_mod)
