"""Import-compatibility alias for scripts written against the reference package name.

``import pithtrain.tasks.pretrain_lm`` resolves to ``pithtrain_b200.tasks.pretrain_lm``, and the reference's
``pithtrain.operators`` sub-package to ``pithtrain_b200.ops``, which also carries the reference's operator module
names (``silu_mul``, ``clamped_swiglu``, ``indexed_bias_add``, ``flash_attn_v4``, ``all_to_all``, ``token_scatter``,
``deepgemm_quantize`` next to ``ring_attention``, ``cross_entropy``, ``grouped_linear``, ``linear``,
``gated_delta_rule``). The alias is a meta-path finder
that hands out the already-imported implementation modules, so both names refer to the same objects and
module-level state (contexts, caches) is never duplicated.
"""

import importlib
import importlib.abc
import importlib.util
import sys

_IMPL = "pithtrain_b200"
_RENAMED = {"operators": "ops"}


def _target(name: str) -> str:
    parts = name.split(".")[1:]
    if parts and parts[0] in _RENAMED:
        parts[0] = _RENAMED[parts[0]]
    return ".".join([_IMPL] + parts)


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)
        self._own_spec = module.__spec__
        return module

    def exec_module(self, module):
        # The implementation module is already initialised. The import system has just stamped the alias spec on
        # it; put its own spec back so that relative imports executed later (inside functions) still see a
        # ``__package__`` that matches ``__spec__.parent``.
        module.__spec__ = self._own_spec


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        impl = _target(fullname)
        try:
            found = importlib.util.find_spec(impl)
        except ModuleNotFoundError:
            return None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(impl), is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

from pithtrain_b200 import *  # noqa: F401,F403,E402
