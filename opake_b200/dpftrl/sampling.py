"""Samplers paired with matrix-factorisation mechanisms.

Stream tags, draw order and state dictionaries follow packages/opake-dpftrl/src/opake/api/dpftrl/sampling/
(_poisson.py:47-248, _partitions.py:19-42, _b_min_sep.py:30-, _balls_in_bins.py:45-200, _sequential.py:20-) so a
resumed run continues the same index stream:

* ``CyclicPoissonSampler``: the dataset is split once into ``bands`` groups; step ``i`` Poisson-samples group
  ``i % bands`` (binomial count, then ``choice`` without replacement).
* ``BMinSepSampler``: a Markov chain in which a sampled example is barred for the next ``bands - 1`` steps.
* ``BallsInBinsSampler``: every example is thrown into one of ``num_bins`` bins once; the bins are replayed in order
  every epoch and empty bins still occupy their slot.
* ``SequentialBatchSampler``: fixed consecutive batches (non-amplified baseline).
"""
from __future__ import annotations

from collections import deque
from collections.abc import Iterator, Mapping, Sized
from enum import Enum
from typing import Any

import numpy as np
from torch.utils.data import Sampler

from ..base.exceptions import ConfigurationError, InputTypeError
from ..base.serialization import register_serializer
from ..engine.random import RngKey, fold_in

CYCLIC_POISSON_STREAM_FOLD = "opake.dpftrl.cyclic_poisson"
B_MIN_SEP_STREAM_FOLD = "opake.dpftrl.b_min_sep"
BALLS_IN_BINS_STREAM_FOLD = "opake.dpftrl.balls_in_bins"


class PartitionType(Enum):
    INDEPENDENT = "independent"
    EQUAL_SPLIT = "equal_split"


def _partition(kind: PartitionType, n: int, groups: int, rng, dtype):
    if kind == PartitionType.INDEPENDENT:
        sizes = rng.multinomial(n, np.ones(groups) / groups)
        idx = rng.permutation(n).astype(dtype)
        return np.split(idx, np.cumsum(sizes)[:-1])
    if kind == PartitionType.EQUAL_SPLIT:
        idx = rng.permutation(n).astype(dtype)
        per = n // groups
        return [g[:per] for g in np.array_split(idx, groups)]
    raise ConfigurationError(f"Unsupported partition_type: {kind}")


def _key_of(sd) -> RngKey:
    return RngKey(int(sd["key_seed"]), str(sd["key_impl"]))


def _check_len(name: str, template_n: int, sd, key: str = "num_samples") -> None:
    saved = sd[key] if key in sd else sd["num_samples" if key == "num_examples" else "num_examples"]
    if int(saved) != template_n:
        raise ConfigurationError(f"{name}.from_state_dict: template dataset length {template_n} does not match snapshot "
                                 f"{key}={int(saved)}.")


class _Resumable(Sampler):
    _consumed = 0

    @property
    def consumed(self) -> int:
        return self._consumed

    def state_dict(self):
        from ..base.serialization import state_dict

        return state_dict(self)

    def load_state_dict(self, sd) -> None:
        from ..base.serialization import from_state_dict

        self.__dict__.update(from_state_dict(self, sd).__dict__)


class CyclicPoissonSampler(_Resumable):
    def __init__(self, data_source: Sized, sample_rate: float, bands: int = 1, n_steps: int = 1,
                 partition_type: PartitionType = PartitionType.EQUAL_SPLIT, truncated_batch_size: int | None = None, *,
                 key: RngKey):
        self._setup(data_source, sample_rate, bands, n_steps, partition_type, truncated_batch_size,
                    fold_in(key, CYCLIC_POISSON_STREAM_FOLD))

    @classmethod
    def _from_stream_key(cls, data_source, sample_rate, bands=1, n_steps=1, partition_type=PartitionType.EQUAL_SPLIT,
                         truncated_batch_size=None, *, stream_key):
        s = object.__new__(cls)
        s._setup(data_source, sample_rate, bands, n_steps, partition_type, truncated_batch_size, stream_key)
        return s

    def _setup(self, data_source, q, bands, n_steps, ptype, cap, stream_key):
        Sampler.__init__(self)
        if len(data_source) == 0:
            raise ConfigurationError("data_source must not be empty")
        if not 0 < q <= 1:
            raise ConfigurationError(f"sample_rate must be in (0, 1], got {q}")
        if bands < 1 or n_steps < 1:
            raise ConfigurationError(f"bands and n_steps must be >= 1, got {bands}, {n_steps}")
        if cap is not None and cap < 1:
            raise ConfigurationError(f"truncated_batch_size must be >= 1, got {cap}")
        self.num_examples = len(data_source)
        self._stream_key = stream_key
        self.generator = np.random.default_rng(stream_key.seed)
        self.partition = _partition(ptype, self.num_examples, bands, self.generator, np.min_scalar_type(-self.num_examples))
        self.data_source, self.sample_rate, self.bands, self.n_steps = data_source, q, bands, n_steps
        self.partition_type, self.truncated_batch_size, self._consumed = ptype, cap, 0

    def _sample_step(self, step: int) -> list[int]:
        group = self.partition[step % self.bands]
        k = self.generator.binomial(n=len(group), p=self.sample_rate)
        if self.truncated_batch_size is not None:
            k = min(k, self.truncated_batch_size)
        if k > 0:
            return self.generator.choice(group, size=k, replace=False, shuffle=False).tolist()
        return []

    def __iter__(self) -> Iterator[list[int]]:
        for step in range(self._consumed, self.n_steps):
            b = self._sample_step(step)
            self._consumed += 1
            yield b

    def __len__(self) -> int:
        return self.n_steps - self._consumed

    @property
    def expected_batch_size(self) -> float:
        return self.num_examples / self.bands * self.sample_rate

    @property
    def batch_size_variance(self) -> float:
        return self.num_examples / self.bands * self.sample_rate * (1 - self.sample_rate)


def _save_cyclic(s):
    return {"key_seed": int(s._stream_key.seed), "key_impl": str(s._stream_key.impl), "consumed": int(s._consumed),
            "num_examples": int(s.num_examples), "sample_rate": float(s.sample_rate), "bands": int(s.bands),
            "n_steps": int(s.n_steps), "partition_type": s.partition_type.name,
            "truncated_batch_size": s.truncated_batch_size}


def _load_cyclic(t, sd):
    _check_len("CyclicPoissonSampler", len(t.data_source), sd, "num_examples")
    pt = sd["partition_type"]
    pt = PartitionType[pt] if pt in PartitionType.__members__ else PartitionType(pt)
    s = CyclicPoissonSampler._from_stream_key(t.data_source, float(sd["sample_rate"]), int(sd["bands"]), t.n_steps,
                                              pt, sd.get("truncated_batch_size"),
                                              stream_key=_key_of(sd))
    for i in range(int(sd["consumed"])):
        s._sample_step(i)
    s._consumed = int(sd["consumed"])
    return s


class BMinSepSampler(_Resumable):
    def __init__(self, data_source: Sized, bands: int, sampling_prob: float, n_steps: int, *, key: RngKey):
        self._setup(data_source, bands, sampling_prob, n_steps, fold_in(key, B_MIN_SEP_STREAM_FOLD))

    @classmethod
    def _from_stream_key(cls, data_source, bands, sampling_prob, n_steps, *, stream_key):
        s = object.__new__(cls)
        s._setup(data_source, bands, sampling_prob, n_steps, stream_key)
        return s

    def _setup(self, data_source, bands, p, n_steps, stream_key):
        Sampler.__init__(self)
        if len(data_source) == 0:
            raise ConfigurationError("data_source must not be empty")
        if bands < 1 or n_steps < 1:
            raise ConfigurationError(f"bands and n_steps must be >= 1, got {bands}, {n_steps}")
        if not 0 < p <= 1:
            raise ConfigurationError(f"sampling_prob must be in (0, 1], got {p}")
        self.num_examples, self.data_source, self.bands = len(data_source), data_source, bands
        self.sampling_prob, self.n_steps, self._stream_key = p, n_steps, stream_key
        self.generator = np.random.default_rng(stream_key.seed)
        self._bars_left = np.zeros(self.num_examples, dtype=np.int32)
        if bands > 1:
            # start from the stationary distribution of the chain ("warm start")
            denom = 1.0 + (bands - 1) * p
            for j in range(self.num_examples):
                if self.generator.random() * denom < 1.0:
                    self._bars_left[j] = 0
                else:
                    self._bars_left[j] = int(self.generator.integers(1, bands))
        self._recent: deque = deque(maxlen=max(0, bands - 1))
        self._consumed = 0

    def _sample_step(self) -> list[int]:
        barred = set()
        for b in self._recent:
            barred.update(b)
        eligible = [i for i in range(self.num_examples) if self._bars_left[i] == 0 and i not in barred]
        batch: list[int] = []
        if eligible:
            k = self.generator.binomial(n=len(eligible), p=self.sampling_prob)
            if k > 0:
                pos = self.generator.choice(len(eligible), size=k, replace=False, shuffle=False)
                batch = [eligible[int(j)] for j in pos]
        self._bars_left[self._bars_left > 0] -= 1
        for i in batch:
            self._bars_left[i] = max(self._bars_left[i], self.bands - 1)
        self._recent.append(set(batch))
        return batch

    def __iter__(self):
        for _ in range(self._consumed, self.n_steps):
            b = self._sample_step()
            self._consumed += 1
            yield b

    def __len__(self) -> int:
        return self.n_steps - self._consumed

    @property
    def expected_batch_size(self) -> float:
        p, b = self.sampling_prob, self.bands
        return self.num_examples * p / (1.0 + (b - 1) * p)


def _save_bms(s):
    return {"key_seed": int(s._stream_key.seed), "key_impl": str(s._stream_key.impl), "consumed": int(s._consumed),
            "num_examples": int(s.num_examples), "bands": int(s.bands), "sampling_prob": float(s.sampling_prob),
            "n_steps": int(s.n_steps)}


def _load_bms(t, sd):
    _check_len("BMinSepSampler", len(t.data_source), sd, "num_examples")
    s = BMinSepSampler._from_stream_key(t.data_source, int(sd["bands"]), float(sd["sampling_prob"]), t.n_steps,
                                        stream_key=_key_of(sd))
    for _ in range(int(sd["consumed"])):
        s._sample_step()
    s._consumed = int(sd["consumed"])
    return s


class BallsInBinsSampler(_Resumable):
    def __init__(self, data_source: Sized, num_bins: int, n_steps: int | None = None, *, key: RngKey):
        self._setup(data_source, num_bins, n_steps, fold_in(key, BALLS_IN_BINS_STREAM_FOLD))

    @classmethod
    def _from_stream_key(cls, data_source, num_bins, n_steps=None, *, stream_key):
        s = object.__new__(cls)
        s._setup(data_source, num_bins, n_steps, stream_key)
        return s

    def _setup(self, data_source, num_bins, n_steps, stream_key):
        Sampler.__init__(self)
        if len(data_source) == 0:
            raise ConfigurationError("data_source must not be empty")
        if num_bins < 2:
            raise ConfigurationError(f"num_bins must be >= 2, got {num_bins}")
        if n_steps is not None:
            if n_steps < 1:
                raise ConfigurationError(f"n_steps must be >= 1 or None, got {n_steps}")
            if n_steps % num_bins:
                raise ConfigurationError(f"n_steps ({n_steps}) must be a positive multiple of num_bins ({num_bins}); BnB "
                                         "analysis assumes integer epochs.")
        self.data_source, self.num_bins, self.n_steps = data_source, num_bins, n_steps
        self._num_samples, self._stream_key = len(data_source), stream_key
        where = np.random.default_rng(stream_key.seed).integers(0, num_bins, size=self._num_samples)
        self._bins: list[list[int]] = [[] for _ in range(num_bins)]
        for i, b in enumerate(where):
            self._bins[b].append(i)
        self._consumed = 0

    @property
    def num_epochs(self):
        return None if self.n_steps is None else self.n_steps // self.num_bins

    def __iter__(self):
        i = self._consumed
        while self.n_steps is None or i < self.n_steps:
            self._consumed = i + 1
            yield self._bins[i % self.num_bins]
            i += 1

    def __len__(self) -> int:
        if self.n_steps is None:
            raise InputTypeError("len() of unsized object (n_steps=None)")
        return self.n_steps - self._consumed

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples / self.num_bins

    @property
    def sample_rate(self) -> float:
        return 1.0 / self.num_bins


def _save_bnb(s):
    return {"key_seed": int(s._stream_key.seed), "key_impl": str(s._stream_key.impl), "consumed": int(s._consumed),
            "num_samples": int(s._num_samples), "num_bins": int(s.num_bins), "n_steps": s.n_steps}


def _load_bnb(t, sd):
    _check_len("BallsInBinsSampler", len(t.data_source), sd)
    s = BallsInBinsSampler._from_stream_key(t.data_source, int(sd["num_bins"]), t.n_steps, stream_key=_key_of(sd))
    s._consumed = int(sd["consumed"])
    return s


class SequentialBatchSampler(_Resumable):
    def __init__(self, data_source: Sized, batch_size: int, n_steps: int | None = None):
        Sampler.__init__(self)
        if batch_size < 1:
            raise ConfigurationError(f"batch_size must be >= 1, got {batch_size}")
        self.data_source, self.batch_size, self.n_steps = data_source, batch_size, n_steps
        self._num_samples, self._consumed = len(data_source), 0

    def __iter__(self):
        n, b = self._num_samples, self.batch_size
        per_epoch = max(1, (n + b - 1) // b)
        i = self._consumed
        while self.n_steps is None or i < self.n_steps:
            k = i % per_epoch
            self._consumed = i + 1
            yield list(range(k * b, min(n, (k + 1) * b)))
            i += 1

    def __len__(self) -> int:
        if self.n_steps is None:
            raise InputTypeError("len() of unsized object (n_steps=None)")
        return self.n_steps - self._consumed


def _save_seq(s):
    return {"consumed": int(s._consumed), "num_samples": int(s._num_samples), "batch_size": int(s.batch_size),
            "n_steps": s.n_steps}


def _load_seq(t, sd):
    _check_len("SequentialBatchSampler", len(t.data_source), sd)
    s = SequentialBatchSampler(t.data_source, int(sd["batch_size"]), t.n_steps)
    s._consumed = int(sd["consumed"])
    return s


register_serializer(CyclicPoissonSampler, _save_cyclic, _load_cyclic)
register_serializer(BMinSepSampler, _save_bms, _load_bms)
register_serializer(BallsInBinsSampler, _save_bnb, _load_bnb)
register_serializer(SequentialBatchSampler, _save_seq, _load_seq)

__all__ = ["BMinSepSampler", "BallsInBinsSampler", "CyclicPoissonSampler", "SequentialBatchSampler", "PartitionType"]
