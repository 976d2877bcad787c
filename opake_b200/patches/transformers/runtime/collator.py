"""Collators and empty batches (packages/opake-patches/src/opake/api/patches/transformers/runtime/collator.py).

Poisson sampling yields an empty batch with probability ``(1 - q)^N``; Hugging Face collators index ``examples[0]``
unconditionally. The patch wraps ``DataCollatorForLanguageModeling.torch_call`` with ``empty_collate``, which learns
the output structure from the first non-empty call and answers an empty list with zero-length tensors of that
structure."""
from __future__ import annotations

import functools

from ....engine.functional import empty_collate

__all__ = ["apply_collator_patches", "COLLATORS"]

_WRAPPER = "_opake_collate"
COLLATORS = ("DataCollatorForLanguageModeling", "DataCollatorWithPadding", "DataCollatorForSeq2Seq", "DataCollatorForTokenClassification")


def _patch_method(cls, name: str) -> bool:
    original = cls.__dict__.get(name)
    if original is None or getattr(original, "__opake_patched__", False):
        return False

    def patched(self, examples, *a, **kw):
        wrapper = self.__dict__.get(_WRAPPER + name)
        if wrapper is None:
            wrapper = empty_collate(functools.partial(original, self))
            self.__dict__[_WRAPPER + name] = wrapper
        return wrapper(examples, *a, **kw) if (a or kw) else wrapper(examples)

    patched.__opake_patched__ = True
    patched.__wrapped__ = original
    setattr(cls, name, patched)
    return True


def apply_collator_patches(*, empty_batches: bool = True) -> int:
    """Idempotent; returns the number of methods patched by this call."""
    if not empty_batches:
        return 0
    try:
        import transformers
    except ImportError:
        return 0
    n = 0
    for cname in COLLATORS:
        cls = getattr(transformers, cname, None)
        if cls is None:
            continue
        n += int(_patch_method(cls, "torch_call") or _patch_method(cls, "__call__"))
    return n
