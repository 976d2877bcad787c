"""Reference-policy helpers for preference optimisation (packages/opake-alignment/src/opake/api/alignment/dpo/
reference/_precompute.py:345-480, _adapter.py:110-219, _sync.py:29-72)."""
from __future__ import annotations

import hashlib
import json
import math
import tempfile
from collections.abc import Mapping, Sequence
from contextlib import contextmanager
from pathlib import Path
from typing import Any, Callable

import torch

from ...base.exceptions import ConfigurationError, InputTypeError, OperationError
from ...engine import distributed as D
from ...engine.pytree import tree_map

__all__ = ["compute_ref_logprobs_for_dataset", "ema_update_reference", "null_ref_context", "with_disabled_adapter"]

_FINGERPRINT_VERSION = 2


# ------------------------------------------------------------------------------------------- TR-DPO sync
def ema_update_reference(ref_params, policy_params, alpha: float):
    """``ref <- (1 - alpha) * ref + alpha * policy`` leaf-wise; ``alpha = 1`` is a hard sync."""
    return tree_map(lambda r, p: (1 - alpha) * r + alpha * p, ref_params, policy_params)


# ------------------------------------------------------------------------------------------- adapters
def _is_peft_model(model) -> bool:
    try:
        from peft import PeftModel          # type: ignore
        return isinstance(model, PeftModel)
    except ImportError:
        return hasattr(model, "peft_config")


@contextmanager
def with_disabled_adapter(model):
    if not _is_peft_model(model):
        yield
        return
    with model.disable_adapter():
        yield


@contextmanager
def null_ref_context(model, ref_model=None):
    """Context in which ``model`` behaves as the reference policy: nothing to do when a separate ``ref_model`` is
    given or the model has no adapters; otherwise the ``"ref"`` adapter is activated if present, else adapters are
    disabled (base model = reference)."""
    if ref_model is model:
        raise ConfigurationError("ref_model must be a separate model; omit ref_model to use the policy's PEFT "
                                 "reference adapter or adapter-disabled base model.")
    if ref_model is not None or not _is_peft_model(model):
        yield
        return
    if "ref" in model.peft_config:
        saved = getattr(model, "active_adapters", None)
        if saved is None:
            saved = getattr(model, "active_adapter", None)
        model.set_adapter("ref")
        try:
            yield
        finally:
            if saved:
                names = [saved] if isinstance(saved, str) else list(saved)
                model.set_adapter(names[0] if len(names) == 1 else names)
        return
    with with_disabled_adapter(model):
        yield


# ------------------------------------------------------------------------------------------- precompute + cache
def _canonical(value, path="cache_identity"):
    if value is None or isinstance(value, (str, bool, int)):
        return value
    if isinstance(value, float):
        if not math.isfinite(value):
            raise ConfigurationError(f"{path} contains a non-finite float")
        return value
    if isinstance(value, Mapping):
        out = {}
        for k, v in value.items():
            if not isinstance(k, str):
                raise InputTypeError(f"{path} mapping keys must be strings, got {type(k)!r}")
            out[k] = _canonical(v, f"{path}.{k}")
        return out
    if isinstance(value, Sequence) and not isinstance(value, (str, bytes, bytearray)):
        return [_canonical(v, f"{path}[{i}]") for i, v in enumerate(value)]
    raise InputTypeError(f"{path} contains unsupported value {type(value)!r}; use only JSON-like scalars, "
                         "string-keyed mappings, and sequences")


def _fingerprint(dataset, identity, columns) -> str:
    ds_id = getattr(dataset, "_fingerprint", None)
    if ds_id is None:
        raise ConfigurationError("dataset must expose a deterministic `_fingerprint` for reference caching")
    payload = {"version": _FINGERPRINT_VERSION, "dataset": str(ds_id), "identity": _canonical(identity),
               "output_columns": list(columns)}
    enc = json.dumps(payload, ensure_ascii=False, sort_keys=True, separators=(",", ":"), allow_nan=False)
    return hashlib.sha256(enc.encode("utf-8")).hexdigest()


def _secure(path: Path) -> None:
    try:
        path.parent.mkdir(parents=True, exist_ok=True, mode=0o700)
        path.parent.chmod(0o700)
        if path.exists():
            path.chmod(0o600)
    except PermissionError as e:
        raise PermissionError(f"cannot secure reference-logprob cache directory {path.parent}; pass a private "
                              "writable cache_dir or set use_cache=False") from e


def _load(path: Path, columns, rows: int):
    if not path.exists():
        return None
    try:
        from safetensors.torch import load_file
        flat = load_file(str(path))
    except Exception:
        return None
    if any(c not in flat or flat[c].shape[:1] != (rows,) for c in columns):
        return None
    return {c: flat[c] for c in columns}


def _add_columns(dataset, columns, values):
    out = dataset
    for c in columns:
        out = out.add_column(c, values[c].detach().cpu().float().tolist())
    return out


def compute_ref_logprobs_for_dataset(dataset, ref: Callable[[dict], dict], collator: Callable[[list], dict],
                                     output_columns: Sequence[str], *, cache_identity: Any, batch_size: int = 8,
                                     cache_dir: str | None = None, use_cache: bool = True, shard: bool | None = None):
    """Runs ``ref(batch) -> {column: tensor[B]}`` over the dataset once and returns the dataset with those columns
    added. Results are cached on disk (safetensors, private permissions) under a SHA-256 of dataset fingerprint,
    ``cache_identity`` and the column names. With a live process group the rows are sharded contiguously over ranks
    and gathered; all ranks must agree on dataset size and fingerprint."""
    from torch.utils.data import DataLoader
    columns = tuple(output_columns)
    n = len(dataset)
    sharded = D.is_distributed() if shard is None else shard
    if shard and not D.is_distributed():
        raise OperationError("shard=True requires an initialised process group; call "
                             "torch.distributed.init_process_group first, or pass shard=None.")
    if sharded:
        D.assert_scalar_equal(n, name="reference precompute dataset size")
        ds_id = getattr(dataset, "_fingerprint", None)
        D.assert_string_equal(None if ds_id is None else str(ds_id), name="reference precompute dataset fingerprint")
        if ds_id is None:
            raise ConfigurationError("dataset must expose a deterministic `_fingerprint` for distributed reference "
                                     "precomputation")
    path, cached = None, None
    if use_cache:
        base = Path(cache_dir) if cache_dir is not None else Path(tempfile.gettempdir()) / "opake_ref_cache"
        path = base / f"{_fingerprint(dataset, cache_identity, columns)}.safetensors"
        _secure(path)
        cached = _load(path, columns, n)
    hit = cached is not None
    if D.is_distributed():
        hit = bool(D.reduce_scalar(int(hit), op="min"))
    if hit:
        return _add_columns(dataset, columns, cached)

    rank, world = (D.get_rank(), D.get_world_size()) if sharded else (0, 1)
    part = D.local_shard(dataset, rank=rank, world_size=world) if world > 1 else dataset
    parts: dict[str, list] = {c: [] for c in columns}
    with torch.no_grad():
        for batch in DataLoader(part, batch_size=batch_size, collate_fn=collator):
            out = ref(batch)
            for c in columns:
                parts[c].append(torch.as_tensor(out[c]).detach())
    local = None if all(not v for v in parts.values()) else {c: torch.cat(parts[c], dim=0) for c in columns}
    gathered = D.gather_pytree(local, dim=0) if sharded else local
    if gathered is None:
        gathered = {c: torch.empty((0,), dtype=torch.float32) for c in columns}
    for c in columns:
        if int(gathered[c].shape[0]) != n:
            raise OperationError(f"reference column {c!r} yielded {int(gathered[c].shape[0])} values for a dataset of "
                                 f"{n} examples; either `ref` did not return one value per row, or the ranks disagree "
                                 "on the dataset")
    if use_cache and D.is_main_process():
        from safetensors.torch import save_file
        save_file({c: gathered[c].detach().cpu().contiguous() for c in columns}, str(path))
        path.chmod(0o600)
    D.barrier()
    return _add_columns(dataset, columns, gathered)
