"""``import pccl`` — the reference-compatible import name of ``pccl_b200``.

Every ``pccl.<x>`` module *is* the corresponding ``pccl_b200.<x>`` module (one
module object under two names), so classes imported through either spelling
are identical.
"""

import importlib
import importlib.abc
import importlib.machinery
import sys

import pccl_b200 as _real

_ALIAS, _REAL = __name__, _real.__name__


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, module):
        self._module = module

    def create_module(self, spec):
        return self._module

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        real_name = _REAL + fullname[len(_ALIAS):]
        try:
            module = importlib.import_module(real_name)
        except ModuleNotFoundError as err:
            if err.name == real_name:
                return None
            raise
        return importlib.machinery.ModuleSpec(fullname, _AliasLoader(module),
                                              is_package=hasattr(module, "__path__"))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
for _name, _module in list(sys.modules.items()):
    if _name.startswith(_REAL + "."):
        sys.modules.setdefault(_ALIAS + _name[len(_REAL):], _module)
sys.modules[_ALIAS] = _real
