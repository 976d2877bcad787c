"""Privacy samplers for DP-SGD: Poisson subsampling and k-out-of-t allocation.

Stream derivation, per-step draws and state dictionaries follow packages/opake-dpsgd/src/opake/api/dpsgd/sampling/
(_poisson.py:36-277, _helpers.py:13-33, _k_out_of_t.py:29-176), so a checkpointed sampler resumes on the same
index stream: Poisson uses one ``numpy.random.default_rng(fold_in(key, "opake.dpsgd.poisson").seed)``; each step is
``rng.random(N) < q`` followed by an optional uniform truncation; restore replays ``consumed`` discarded draws.
Samplers are ``torch.utils.data`` batch samplers that yield ``list[int]`` (possibly empty).
"""
from __future__ import annotations

from collections.abc import Iterator, Mapping, Sized
from typing import Any

import numpy as np
from torch.utils.data import Sampler

from ..base.exceptions import ConfigurationError, InputTypeError
from ..base.serialization import register_serializer
from ..engine.random import RngKey, fold_in

POISSON_STREAM_FOLD = "opake.dpsgd.poisson"
K_OUT_OF_T_STREAM_FOLD = "opake.dpsgd.k_out_of_t"


def truncate_indices(rng, indices: np.ndarray, cap: int | None) -> list[int]:
    if cap is not None and indices.size > cap:
        indices = rng.choice(indices, size=cap, replace=False)
    return indices.tolist()


def poisson_step_indices(rng, n: int, q: float, cap: int | None) -> list[int]:
    return truncate_indices(rng, np.where(rng.random(n) < q)[0], cap)


class PoissonSampler(Sampler):
    def __init__(self, data_source: Sized, sample_rate: float, n_steps: int | None = None,
                 truncated_batch_size: int | None = None, *, key: RngKey):
        self._setup(data_source, sample_rate, n_steps, truncated_batch_size, fold_in(key, POISSON_STREAM_FOLD))

    @classmethod
    def _from_stream_key(cls, data_source, sample_rate, n_steps=None, truncated_batch_size=None, *, stream_key):
        s = object.__new__(cls)
        s._setup(data_source, sample_rate, n_steps, truncated_batch_size, stream_key)
        return s

    def _setup(self, data_source, sample_rate, n_steps, cap, stream_key) -> None:
        Sampler.__init__(self)
        if not 0 < sample_rate <= 1:
            raise ConfigurationError(f"sample_rate must be in (0, 1], got {sample_rate}")
        if n_steps is not None and n_steps < 1:
            raise ConfigurationError(f"n_steps must be >= 1 or None, got {n_steps}")
        if cap is not None:
            if type(cap) is not int:
                raise InputTypeError(f"truncated_batch_size must be an int, got {type(cap).__name__}")
            if cap < 1:
                raise ConfigurationError(f"truncated_batch_size must be >= 1, got {cap}")
        self.data_source, self.sample_rate, self.n_steps, self.truncated_batch_size = data_source, sample_rate, n_steps, cap
        self._num_samples = len(data_source)
        self._stream_key = stream_key
        self.generator = np.random.default_rng(stream_key.seed)
        self._consumed = 0

    def _sample_step(self) -> list[int]:
        return poisson_step_indices(self.generator, self._num_samples, self.sample_rate, self.truncated_batch_size)

    def __iter__(self) -> Iterator[list[int]]:
        while self.n_steps is None or self._consumed < self.n_steps:
            batch = self._sample_step()
            self._consumed += 1
            yield batch

    def __len__(self) -> int:
        if self.n_steps is None:
            raise InputTypeError("len() of unsized object (n_steps=None)")
        return self.n_steps - self._consumed

    @property
    def consumed(self) -> int:
        return self._consumed

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples * self.sample_rate

    @property
    def batch_size_variance(self) -> float:
        return self._num_samples * self.sample_rate * (1 - self.sample_rate)

    def state_dict(self) -> dict[str, Any]:
        return _save_poisson(self)

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        other = _load_poisson(self, sd)
        self.__dict__.update(other.__dict__)


def _save_poisson(s: PoissonSampler) -> dict[str, Any]:
    return {"key_seed": int(s._stream_key.seed), "key_impl": str(s._stream_key.impl), "consumed": int(s._consumed),
            "num_samples": int(s._num_samples), "sample_rate": float(s.sample_rate), "n_steps": s.n_steps,
            "truncated_batch_size": s.truncated_batch_size}


def _load_poisson(template: PoissonSampler, sd: Mapping[str, Any]) -> PoissonSampler:
    if int(sd["num_samples"]) != len(template.data_source):
        raise ConfigurationError(f"PoissonSampler.from_state_dict: template dataset length {len(template.data_source)} "
                                 f"does not match snapshot num_samples={int(sd['num_samples'])}.  Restoring with a "
                                 "differently-sized dataset would silently emit a different Poisson stream.")
    s = PoissonSampler._from_stream_key(template.data_source, float(sd["sample_rate"]), template.n_steps,
                                        sd.get("truncated_batch_size"),
                                        stream_key=RngKey(int(sd["key_seed"]), str(sd["key_impl"])))
    for _ in range(int(sd["consumed"])):
        s._sample_step()
    s._consumed = int(sd["consumed"])
    return s


class KOutOfTSampler(Sampler):
    """Every example takes part in exactly ``k`` of ``t`` steps ("block": one step per block; "total": any k steps)."""

    def __init__(self, data_source: Sized, *, k: int, t: int, allocation: str, key: RngKey):
        self._setup(data_source, k, t, allocation, fold_in(key, K_OUT_OF_T_STREAM_FOLD, allocation)
                    if allocation in ("block", "total") else key)

    @classmethod
    def _from_stream_key(cls, data_source, *, k, t, allocation, stream_key):
        s = object.__new__(cls)
        s._setup(data_source, k, t, allocation, stream_key)
        return s

    def _setup(self, data_source, k, t, allocation, stream_key) -> None:
        Sampler.__init__(self)
        if len(data_source) == 0:
            raise ConfigurationError("data_source must not be empty")
        if t < 1:
            raise ConfigurationError(f"t must be >= 1, got {t}")
        if not 1 <= k <= t:
            raise ConfigurationError(f"k must be in [1, t={t}], got {k}")
        if allocation not in ("block", "total"):
            raise ConfigurationError(f"allocation must be 'block' or 'total', got {allocation!r}")
        self.data_source, self.k, self.t, self.allocation = data_source, int(k), int(t), allocation
        self._num_samples, self._stream_key, self._consumed = len(data_source), stream_key, 0

    @property
    def consumed(self) -> int:
        return self._consumed

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples * self.k / self.t

    @property
    def block_sizes(self):
        if self.allocation == "total":
            return None
        lo = self.t // self.k
        n_hi = self.t - lo * self.k
        return (lo,) * (self.k - n_hi) + (lo + 1,) * n_hi

    def _block_bins(self, block: int, size: int) -> list[list[int]]:
        rng = np.random.default_rng(fold_in(self._stream_key, block).seed)
        where = rng.integers(0, size, size=self._num_samples)
        bins: list[list[int]] = [[] for _ in range(size)]
        for i, b in enumerate(where):
            bins[b].append(i)
        return bins

    def _total_batches(self):
        rng = np.random.default_rng(self._stream_key.seed)
        left = np.full(self._num_samples, self.k, dtype=np.int64)
        for step in range(self.t):
            mask = rng.random(self._num_samples) < left / (self.t - step)
            yield np.flatnonzero(mask).tolist()
            left -= mask

    def __iter__(self) -> Iterator[list[int]]:
        if self.allocation == "total":
            for step, batch in enumerate(self._total_batches()):
                if step >= self._consumed:
                    self._consumed = step + 1
                    yield batch
            return
        lo = self.t // self.k
        n_lo = self.k - (self.t - lo * self.k)
        span = n_lo * lo
        bins, cur = None, None
        for step in range(self._consumed, self.t):
            if step < span:
                block, slot, size = step // lo, step % lo, lo
            else:
                off, slot = divmod(step - span, lo + 1)
                block, size = n_lo + off, lo + 1
            if bins is None or block != cur:
                bins, cur = self._block_bins(block, size), block
            self._consumed = step + 1
            yield bins[slot]

    def __len__(self) -> int:
        return self.t - self._consumed

    def state_dict(self) -> dict[str, Any]:
        return _save_kt(self)

    def load_state_dict(self, sd) -> None:
        self.__dict__.update(_load_kt(self, sd).__dict__)


def _save_kt(s: KOutOfTSampler) -> dict[str, Any]:
    return {"key_seed": int(s._stream_key.seed), "key_impl": str(s._stream_key.impl), "consumed": int(s._consumed),
            "num_samples": int(s._num_samples), "k": s.k, "t": s.t, "allocation": s.allocation}


def _load_kt(template: KOutOfTSampler, sd) -> KOutOfTSampler:
    if int(sd["num_samples"]) != len(template.data_source):
        raise ConfigurationError("KOutOfTSampler.from_state_dict: dataset length differs from the snapshot")
    s = KOutOfTSampler._from_stream_key(template.data_source, k=int(sd["k"]), t=int(sd["t"]),
                                        allocation=str(sd["allocation"]),
                                        stream_key=RngKey(int(sd["key_seed"]), str(sd["key_impl"])))
    s._consumed = int(sd["consumed"])
    return s


register_serializer(PoissonSampler, _save_poisson, _load_poisson)
register_serializer(KOutOfTSampler, _save_kt, _load_kt)

__all__ = ["KOutOfTSampler", "PoissonSampler", "POISSON_STREAM_FOLD", "K_OUT_OF_T_STREAM_FOLD"]
