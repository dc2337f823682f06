"""``elf``: the import paths of topal-team/elf, served by ``elf_b200``.

Code written against the reference package (``from elf import Pipeline``,
``from elf.scheduling.ilp import solve_remat``, ``from elf.utils import Placement`` ...)
runs unchanged: every module path the reference exposes (``elf/__init__.py:1-13`` and its
sub-packages) is an alias of the module of the same role in ``elf_b200`` — the very same
module object, so registries, classes and ``isinstance`` checks are shared between the two
spellings.
"""

from __future__ import annotations

import importlib
import sys

import elf_b200 as _impl
from elf_b200 import *  # noqa: F401,F403
from elf_b200 import __all__ as _impl_all

# reference module path (below ``elf.``) -> implementing module (below ``elf_b200.``)
_MODULES = {
    "pipeline": "pipeline",
    "registry": "registry",
    "zb_utils": "zb_utils",
    "utils": "utils",
    "scheduling": "scheduling",
    "scheduling.scheduling": "scheduling.scheduling",
    "scheduling.schedulers": "scheduling.schedulers",
    "scheduling.comm_scheduling": "scheduling.comm_scheduling",
    "scheduling.ilp": "scheduling.ilp",
    "partitioners": "partitioners",
    "partitioners.utils": "partitioners.utils",
    "partitioners.partition": "partitioners.partition",
    "partitioners.tracing": "partitioners.tracing",
    "partitioners.profile": "partitioners.profile",
    "partitioners.custom": "partitioners.custom",
    "partitioners.metis": "partitioners.metis",
    "partitioners.dagP": "partitioners.dagP",
    "execution": "execution",
    "execution.block": "execution.block",
    "execution.engine": "execution.engine",
    "execution.offload": "execution.offload",
    "execution.remat": "execution.remat",
}

_me = sys.modules[__name__]
for _alias, _target in _MODULES.items():
    _mod = importlib.import_module(f"elf_b200.{_target}")
    sys.modules[f"{__name__}.{_alias}"] = _mod
    _parent, _, _leaf = _alias.rpartition(".")
    setattr(sys.modules[f"{__name__}.{_parent}"] if _parent else _me, _leaf, _mod)

__all__ = list(_impl_all)
__version__ = getattr(_impl, "__version__", "0.1.0")
