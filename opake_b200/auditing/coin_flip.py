"""Canary selection and random inclusion for one-run privacy audits (packages/opake-auditing/src/opake/api/auditing/
_coin_flip.py:42-398). Canaries are drawn without replacement with one RNG stream and each is included in training
with probability 1/2 by a second stream; both streams derive from the caller's key by ``fold_in`` with fixed tags,
so an audit is reproducible from the key alone. Scores always travel with the dataset indices they belong to
(``CanaryScores``): the membership split joins on identifiers, never on position."""
from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np
from torch.utils.data import Subset

from ..base.exceptions import ConfigurationError, InputTypeError
from ..engine.random import fold_in

__all__ = ["CanaryScores", "CoinFlip", "canary_scores", "coin_flip"]

_SELECTION_TAG = "opake.auditing.canary_selection"
_COIN_TAG = "opake.auditing.coin_flip"


@dataclasses.dataclass(frozen=True)
class CanaryScores:
    """Membership scores (higher = more likely a training member) with the dataset index of each scored canary."""
    scores: np.ndarray
    canary_indices: np.ndarray

    def __post_init__(self):
        sc = np.array(self.scores, dtype=float)
        ids = np.array(self.canary_indices)
        if sc.ndim != 1:
            raise ConfigurationError(f"scores must be 1-D, got shape {sc.shape}")
        if ids.ndim != 1 or not np.issubdtype(ids.dtype, np.integer):
            raise ConfigurationError(f"canary_indices must be a 1-D integer array, got shape {ids.shape}, dtype {ids.dtype}")
        if sc.shape != ids.shape:
            raise ConfigurationError(f"scores and canary_indices must have equal length, got {sc.shape[0]} scores for "
                                     f"{ids.shape[0]} indices")
        if np.unique(ids).size != ids.size:
            raise ConfigurationError("canary_indices must be unique; duplicate identifiers make the score join ambiguous")
        sc.setflags(write=False)
        ids.setflags(write=False)
        object.__setattr__(self, "scores", sc)
        object.__setattr__(self, "canary_indices", ids)

    def __len__(self):
        return self.scores.shape[0]

    def __array__(self, dtype=None, copy=None):
        return np.array(self.scores, dtype=dtype) if copy else np.asarray(self.scores, dtype=dtype)

    def __repr__(self):
        return f"CanaryScores(num_canaries={len(self)})"


def canary_scores(scores: Any, *, canary_indices: Any) -> CanaryScores:
    return CanaryScores(scores, canary_indices=canary_indices)


@dataclasses.dataclass(frozen=True)
class CoinFlip:
    num_canaries: int
    canary_indices: np.ndarray
    _in_mask: np.ndarray
    in_indices: np.ndarray
    out_indices: np.ndarray
    dataset_size: int | None = None

    def __repr__(self):
        return f"CoinFlip(num_canaries={self.num_canaries}, n_in={len(self.in_indices)}, n_out={len(self.out_indices)})"

    def train_indices(self, dataset_size: int | None = None) -> list[int]:
        """All dataset indices except the canaries whose coin came up 'out'."""
        size = self.dataset_size if dataset_size is None else dataset_size
        if size is None:
            raise ConfigurationError("dataset_size must be provided when not recorded on CoinFlip")
        keep = np.ones(size, dtype=bool)
        keep[self.out_indices[self.out_indices < size]] = False
        return np.nonzero(keep)[0].tolist()

    def train_subset(self, dataset) -> Subset:
        return Subset(dataset, self.train_indices(len(dataset)))

    def _join(self, scores: CanaryScores) -> np.ndarray:
        """Scores re-ordered to this partition's canary order; identifiers must match one-to-one."""
        want, have = self.canary_indices, scores.canary_indices
        if want.size == 0:
            if have.size:
                raise ConfigurationError(f"got {have.size} scores for a partition with no canaries")
            return np.empty(0, dtype=float)
        slot_of = {int(v): i for i, v in enumerate(want)}
        if len(slot_of) != want.size:
            raise ConfigurationError("canary_indices of this partition contain duplicates; the score join is ambiguous")
        unknown = [int(v) for v in have if int(v) not in slot_of]
        if unknown:
            raise ConfigurationError(f"{len(unknown)} score identifier(s) are not canaries of this partition (e.g. "
                                     f"{unknown[:5]}); the scores were computed for different examples or a different CoinFlip.")
        missing = set(slot_of) - {int(v) for v in have}
        if missing:
            raise ConfigurationError(f"score identifiers do not cover the partition's canaries one-to-one: "
                                     f"{len(missing)} missing (e.g. {sorted(missing)[:5]}). Check for drop_last=True, "
                                     "distributed samplers, or scoring a wrong subset.")
        out = np.empty(want.size, dtype=float)
        out[[slot_of[int(v)] for v in have]] = scores.scores
        return out

    def split_scores(self, scores: CanaryScores) -> tuple[np.ndarray, np.ndarray]:
        if not isinstance(scores, CanaryScores):
            raise InputTypeError(f"split_scores() requires CanaryScores, got {type(scores).__name__}. Bare score arrays "
                                 "cannot prove score-to-membership pairing; score with loss_scores(..., coin_flip=cf, "
                                 "dataset=dataset) / gradient_scores(...), or attest identifiers explicitly with "
                                 "canary_scores(values, canary_indices=...).")
        joined = self._join(scores)
        return joined[self._in_mask], joined[~self._in_mask]


def _pool(candidate_indices, n: int) -> np.ndarray:
    pool = np.asarray(candidate_indices)
    if pool.ndim != 1:
        raise ConfigurationError(f"candidate_indices must be 1-D, got shape {pool.shape}")
    if pool.size == 0:
        return np.empty(0, dtype=np.intp)
    if not np.issubdtype(pool.dtype, np.integer):
        raise ConfigurationError(f"candidate_indices must contain integers, got dtype {pool.dtype}")
    uniq = np.unique(pool)
    if uniq.size != pool.size:
        raise ConfigurationError("candidate_indices must be unique")
    bad = uniq[(uniq < 0) | (uniq >= n)]
    if bad.size:
        raise ConfigurationError(f"candidate_indices must be within range(len(dataset)); got {bad[:5].tolist()}")
    return uniq


def coin_flip(dataset, *, num_canaries: int, key, candidate_indices=None) -> CoinFlip:
    n = len(dataset)
    if num_canaries < 0:
        raise ConfigurationError(f"num_canaries must be non-negative, got {num_canaries}")
    if candidate_indices is None:
        population, size, what = n, n, "dataset size"
    else:
        population = _pool(candidate_indices, n)
        size, what = population.size, "candidate pool size"
    if num_canaries > size:
        raise ConfigurationError(f"num_canaries ({num_canaries}) exceeds {what} ({size})")
    chosen = np.random.default_rng(fold_in(key, _SELECTION_TAG).seed).choice(population, size=num_canaries, replace=False)
    included = np.asarray(np.random.default_rng(fold_in(key, _COIN_TAG).seed).random(num_canaries) < 0.5, dtype=bool)
    return CoinFlip(num_canaries=num_canaries, canary_indices=chosen, _in_mask=included, in_indices=chosen[included],
                    out_indices=chosen[~included], dataset_size=n)
