"""Explicit, immutable random keys.

Key derivation is byte-compatible with the reference so that checkpoints and stream tags carry over
(packages/opake-engine/src/opake/api/engine/random/_engine.py:29-137): a fold hashes, with blake2b-64, the parent
seed and the folded value, each written as a type tag (``i`` / ``s``), a payload (16-byte little-endian signed
integer, or UTF-8 text) and a ``|`` terminator.

On top of that the B200 build adds :func:`philox_counter_key`: the 64-bit seed of a key is the Philox key of the
device noise generator, which indexes noise by global element offset instead of consuming a CPU generator.
"""
from __future__ import annotations

import contextlib
import dataclasses
import hashlib
import os
import secrets

import torch

from ..base.exceptions import ConfigurationError, InputTypeError

__all__ = ["RngKey", "key", "fold_in", "split", "generator_from_key", "random_key", "set_reproducible_pytorch_seed",
           "numpy_generator_from_key"]

_U64 = (1 << 64) - 1
_TORCH_SEED_MOD = 2**63 - 1
DEFAULT_IMPL = "opake_threefry_like"


@dataclasses.dataclass(frozen=True)
class RngKey:
    seed: int
    impl: str = DEFAULT_IMPL


def _digest64(parent_seed: int, value: int | str) -> int:
    h = hashlib.blake2b(digest_size=8)
    for part in (parent_seed, value):
        if isinstance(part, int):
            h.update(b"i" + part.to_bytes(16, "little", signed=True))
        else:
            h.update(b"s" + str(part).encode("utf-8"))
        h.update(b"|")
    return int.from_bytes(h.digest(), "little")


def key(seed: int) -> RngKey:
    if isinstance(seed, bool) or not isinstance(seed, int):
        raise InputTypeError(f"seed must be int, got {type(seed)}")
    return RngKey(seed & _U64)


def fold_in(rng_key: RngKey, *data: int | str) -> RngKey:
    """Derive a child key; several values fold left to right (``fold_in(k, a, b) == fold_in(fold_in(k, a), b)``)."""
    if not isinstance(rng_key, RngKey):
        raise InputTypeError(f"rng_key must be RngKey, got {type(rng_key)}")
    if not data:
        raise ConfigurationError("fold_in requires at least one data argument")
    seed = rng_key.seed
    for d in data:
        if isinstance(d, bool) or not isinstance(d, (int, str)):
            raise InputTypeError(f"data must be int or str, got {type(d)}")
        seed = _digest64(seed, d)
    return RngKey(seed, rng_key.impl)


def split(rng_key: RngKey, num: int = 2) -> tuple[RngKey, ...]:
    if isinstance(num, bool) or not isinstance(num, int):
        raise InputTypeError(f"num must be int, got {type(num)}")
    if num < 1:
        raise ConfigurationError(f"num must be >= 1, got {num}")
    return tuple(fold_in(rng_key, i) for i in range(num))


def generator_from_key(rng_key: RngKey) -> torch.Generator:
    """CPU ``torch.Generator`` seeded from the key (the reference's noise source; kept for its compatibility mode)."""
    return torch.Generator().manual_seed(rng_key.seed % _TORCH_SEED_MOD)


def numpy_generator_from_key(rng_key: RngKey):
    import numpy as np

    return np.random.default_rng(rng_key.seed)


def random_key() -> RngKey:
    return key(secrets.randbits(64))


def set_reproducible_pytorch_seed(key_val: RngKey) -> None:
    """Seed torch (CPU, CUDA), NumPy and switch on deterministic library modes from one key."""
    import numpy as np

    cpu, gpu, npk = split(key_val, 3)
    torch.manual_seed(int(cpu.seed % (2**31 - 1)))
    torch.cuda.manual_seed_all(int(gpu.seed % (2**31 - 1)))
    with contextlib.suppress(Exception):
        np.random.seed(int(npk.seed % 2**32))
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    with contextlib.suppress(AttributeError, RuntimeError):
        torch.use_deterministic_algorithms(True)
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":16:8"
