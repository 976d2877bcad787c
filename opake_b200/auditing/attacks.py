"""Membership scoring attacks for audits (packages/opake-auditing/src/opake/api/auditing/attacks/_loss.py:30-149,
_gradient.py:36-170, _helpers.py:80-232): minus the per-example loss, or minus the squared per-example gradient
norm. Both walk the canaries of a ``CoinFlip`` in a fixed order through an index-carrying loader and return
``CanaryScores`` bound to dataset indices."""
from __future__ import annotations

from typing import Any, Callable

import numpy as np

from ..base.exceptions import ConfigurationError, InputTypeError
from .coin_flip import CanaryScores, CoinFlip

__all__ = ["loss_scores", "gradient_scores"]


def _check_argnums(batch_argnums, n_other: int) -> None:
    if not batch_argnums:
        raise ConfigurationError(f"batch_argnums must be non-empty, got {batch_argnums}")
    if any(a < 0 for a in batch_argnums):
        raise ConfigurationError(f"batch_argnums must be non-negative, got {batch_argnums}")
    if len(set(batch_argnums)) != len(batch_argnums):
        raise ConfigurationError(f"batch_argnums must be unique, got {batch_argnums}")
    if tuple(sorted(batch_argnums)) != tuple(batch_argnums):
        raise ConfigurationError(f"batch_argnums must be sorted, got {batch_argnums}")
    total = n_other + len(batch_argnums)
    if max(batch_argnums) >= total:
        raise ConfigurationError(f"batch_argnums index {max(batch_argnums)} out of range for {total} total arguments "
                                 f"({n_other} non-batched + {len(batch_argnums)} batched), got {batch_argnums}")


def _interleave(args, batch_items, batch_argnums) -> list:
    total = len(args) + len(batch_argnums)
    out: list = [None] * total
    for pos, item in zip(batch_argnums, batch_items):
        out[pos] = item
    rest = iter(args)
    for i in range(total):
        if i not in batch_argnums:
            out[i] = next(rest)
    return out


def _batch_items(batch, batch_argnums) -> tuple:
    if isinstance(batch, (list, tuple)):
        return tuple(batch[i] for i in range(len(batch_argnums)))
    return (batch,)


class _Canaries:
    def __init__(self, dataset, ids):
        self.dataset, self.ids = dataset, ids

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, pos):
        return pos, self.dataset[int(self.ids[pos])]


def _loader(dataset, cf: CoinFlip, batch_size, collate_fn, reference_scores):
    import torch.utils.data as tud
    n = len(dataset)
    if cf.dataset_size is not None and n != cf.dataset_size:
        raise ConfigurationError(f"dataset length ({n}) does not match the dataset size ({cf.dataset_size}) the CoinFlip "
                                 "was constructed from; scoring requires the full concatenated dataset, not a training "
                                 "subset or split")
    if np.any(cf.canary_indices < 0) or np.any(cf.canary_indices >= n):
        raise ConfigurationError(f"canary indices must be within dataset bounds [0, {n})")
    if isinstance(batch_size, bool) or not isinstance(batch_size, int):
        raise InputTypeError(f"batch_size must be an int, got {type(batch_size).__name__}")
    if batch_size < 1:
        raise ConfigurationError(f"batch_size must be positive, got {batch_size}")
    if reference_scores is not None and not isinstance(reference_scores, CanaryScores):
        raise InputTypeError("reference_scores must carry canary identifiers; compute it with the same coin_flip= and "
                             "dataset=, or attest identifiers with canary_scores(values, canary_indices=...)")
    inner = tud.default_collate if collate_fn is None else collate_fn

    def collate(items):
        pos = [p for p, _ in items]
        out = inner([e for _, e in items])
        probe = out[0] if isinstance(out, (list, tuple)) and out else out
        shape = getattr(probe, "shape", None)
        if shape is not None and len(shape) and int(shape[0]) != len(pos):
            raise ConfigurationError(f"collate_fn returned {int(shape[0])} rows for a batch of {len(pos)} canaries; it "
                                     "must emit exactly one row per example, in the order received")
        return pos, out

    return tud.DataLoader(_Canaries(dataset, cf.canary_indices), batch_size=batch_size, shuffle=False, collate_fn=collate)


def _bind(scores, positions, cf: CoinFlip, reference_scores) -> CanaryScores:
    ids = cf.canary_indices[np.asarray(positions, dtype=int)]
    if reference_scores is not None:
        ref = dict(zip(reference_scores.canary_indices.tolist(), reference_scores.scores.tolist()))
        try:
            scores = scores - np.array([ref[int(i)] for i in ids], dtype=float)
        except KeyError:
            raise ConfigurationError("reference_scores do not cover the scored canaries; compute the reference over the "
                                     "same coin_flip and dataset") from None
    return CanaryScores(scores, canary_indices=ids)


def loss_scores(loss_fn: Callable, *args: Any, batch_argnums: tuple[int, ...], coin_flip: CoinFlip, dataset: Any,
                reference_scores: CanaryScores | None = None, batch_size: int = 32,
                collate_fn: Callable | None = None) -> CanaryScores:
    """Score = minus the example's loss (``loss_fn`` takes one example; it is vmapped over the batched arguments).
    ``reference_scores`` (same canaries, e.g. from a model trained without them) are subtracted for calibration."""
    import torch
    _check_argnums(batch_argnums, len(args))
    loader = _loader(dataset, coin_flip, batch_size, collate_fn, reference_scores)
    total = len(args) + len(batch_argnums)
    fn = torch.func.vmap(loss_fn, in_dims=tuple(0 if i in batch_argnums else None for i in range(total)))
    positions, chunks = [], []
    with torch.no_grad():
        for pos, batch in loader:
            positions.extend(int(p) for p in pos)
            losses = fn(*_interleave(args, _batch_items(batch, batch_argnums), batch_argnums))
            chunks.append(-losses.detach().float().cpu().numpy())
    scores = np.concatenate(chunks) if chunks else np.empty(0)
    return _bind(scores, positions, coin_flip, reference_scores)


def gradient_scores(loss_fn: Callable, *args: Any, batch_argnums: tuple[int, ...], coin_flip: CoinFlip, dataset: Any,
                    reference_scores: CanaryScores | None = None, batch_size: int = 32,
                    collate_fn: Callable | None = None) -> CanaryScores:
    """Score = minus the squared norm of the example's gradient with respect to argument 0 of ``loss_fn``."""
    import torch
    from ..engine.pytree import global_norm
    _check_argnums(batch_argnums, len(args))
    if 0 in batch_argnums:
        raise ConfigurationError("gradient_scores differentiates w.r.t. the first argument (position 0), which must not "
                                 f"be in batch_argnums. Got batch_argnums={batch_argnums}.")
    loader = _loader(dataset, coin_flip, batch_size, collate_fn, reference_scores)
    grad = torch.func.grad(loss_fn)
    positions, scores = [], []
    for pos, batch in loader:
        positions.extend(int(p) for p in pos)
        items = _batch_items(batch, batch_argnums)
        for j in range(items[0].shape[0]):
            g = grad(*_interleave(args, tuple(t[j] for t in items), batch_argnums))
            scores.append(-float(global_norm(g).pow(2)))
            del g
    return _bind(np.array(scores, dtype=float), positions, coin_flip, reference_scores)
