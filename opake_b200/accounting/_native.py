"""Loader of the C++ accountant module (built in-tree by :mod:`opake_b200._build`; no torch involved)."""
from __future__ import annotations

import importlib.util
import sys

from .._build import ACCOUNTING_LIB, build_accounting

_MOD = None


def native():
    global _MOD
    if _MOD is None:
        if not ACCOUNTING_LIB.exists():
            build_accounting()
        spec = importlib.util.spec_from_file_location("_opake_accounting", str(ACCOUNTING_LIB))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules.setdefault("_opake_accounting", mod)
        _MOD = mod
    return _MOD
