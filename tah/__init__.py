"""``tah``: the reference package's import name, served by :mod:`tah_b200`.

Code written against the reference (``from tah import TaHForCausalLM``, ``from tah.model.utils import
TaHForCasualLM_generate``, ``from tah.evaluate.backends import setup_backend`` ...; reference
``tah/__init__.py:6-21``, ``tah/model/__init__.py:7-35``, ``tah/train/__init__.py:3-11``,
``tah/utils/__init__.py:3``, ``tah/evaluate/__init__.py:12-26``) imports unchanged: every ``tah.<sub>`` module
*is* the ``tah_b200.<sub>`` module (the same object, so classes and registries are shared), resolved by a small
import hook instead of duplicated files.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

import tah_b200
from tah_b200 import (IterDeciderLoss, IterLabelDecider, MLPIterDecider, NextTokenPredLoss, TaHCache,  # noqa: F401
                      TaHCausalLMOutputWithPast, TaHConfig, TaHForCausalLM)

__version__ = tah_b200.__version__
__all__ = list(tah_b200.__all__)

_SELF = sys.modules[__name__]


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Resolves ``tah.a.b`` to the already importable ``tah_b200.a.b``."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("tah.") or sys.modules.get("tah") is not _SELF:
            return None
        real = "tah_b200." + fullname[len("tah."):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=False)

    def create_module(self, spec):
        return importlib.import_module("tah_b200." + spec.name[len("tah."):])

    def exec_module(self, module):
        return None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
