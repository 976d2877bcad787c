"""Matrix-factorisation Gaussian mechanism: ``noise_fn(ClippedPytree, MFNoiseState) -> (NoisedPytree, MFNoiseState)``.

Behaviour of packages/opake-dpftrl/src/opake/api/dpftrl/noise/_mf_gaussian_noise.py:55-275 and _engine.py:38-520:
column ``t`` of iid noise is drawn from ``fold_in(key, "opake.dpftrl.mf_gaussian", t)``, pushed through the strategy's
streaming ``C^{-1}`` and added with ``sigma = noise_multiplier * max_norm``; the realised stddev reported on the output
is ``sigma * ||row_t(C^{-1})||``; the horizon ``n_steps`` is enforced; ``max_norm`` must stay constant over the run.
On CUDA leaves the draw uses the device Philox generator; the sharded engine instead fuses the BLT state update into
its step kernel (csrc/kernels/dp_step.cu) for buffered-linear-Toeplitz strategies.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, replace
from typing import Any

import torch

from ..base.exceptions import ConfigurationError, InputTypeError, OperationError
from ..base.serialization import register_serializer, state_dict as _sd, from_state_dict as _fsd
from ..dpsgd.noise import add_gaussian_noise_tree
from ..engine.noise_allocation import per_group_noise_stddev
from ..engine.pytree import tree_map
from ..engine.random import RngKey, fold_in
from ..engine.types import ClippedPytree, NoisedPytree, NoiseState, PerGroup, SecondMomentClippingOutput
from .strategies import IdentityStrategy, MfStrategy, serialize_strategy

MF_STREAM_FOLD = "opake.dpftrl.mf_gaussian"
MF_COLUMN_FOLD = "mf_gaussian_column"
SECOND_MOMENT_FIRST_FOLD = "opake.dpftrl.second_moment.first"
SECOND_MOMENT_SECOND_FOLD = "opake.dpftrl.second_moment.second"
STATE_LAYOUT_VERSION = 1


@dataclass(frozen=True)
class MFNoiseState(NoiseState):
    _inner_state: Any
    _step_counter: int
    _rng_key: RngKey
    _first_max_norm: Any = None
    _strategy_fingerprint: str = ""
    _n_steps: int = 0


def _check_horizon(step: int, n_steps: int) -> None:
    if step >= n_steps:
        raise OperationError(f"matrix-factorisation noise was built for n_steps={n_steps}; step {step} is past the "
                             "horizon. Rebuild the mechanism (and recalibrate) for a longer run.")


def _same_norm(a, b) -> bool:
    if isinstance(a, PerGroup) or isinstance(b, PerGroup):
        return isinstance(a, PerGroup) and isinstance(b, PerGroup) and dict(a.values) == dict(b.values)
    return float(a) == float(b)


def iid_normal_like(tree, key: RngKey, *, compute_dtype=torch.float32, backend: str = "auto"):
    """Unit Gaussian noise shaped like ``tree`` (same streams as the DP-SGD mechanism's backends)."""
    zeros = tree_map(lambda t: torch.zeros_like(t, dtype=compute_dtype) if isinstance(t, torch.Tensor) else t, tree)
    return add_gaussian_noise_tree(zeros, 1.0, key, compute_dtype=compute_dtype, backend=backend)


def mf_gaussian_noise(grad_template, strategy: MfStrategy, *, n_steps: int, min_sep: int = 1,
                      max_participations: int | None = None, noise_multiplier: float, key: RngKey,
                      compute_dtype: torch.dtype = torch.float32, second_moment_strategy: MfStrategy | None = None,
                      backend: str = "auto"):
    if noise_multiplier is None or float(noise_multiplier) < 0:
        raise ConfigurationError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
    if n_steps < 1:
        raise ConfigurationError(f"n_steps must be >= 1, got {n_steps}")
    if not isinstance(key, RngKey):
        raise InputTypeError(f"key must be RngKey, got {type(key)}")
    nm = float(noise_multiplier)
    if second_moment_strategy is not None:
        from .second_moment import make_second_moment_mf_noise

        return make_second_moment_mf_noise(grad_template, strategy, second_moment_strategy, n_steps=n_steps,
                                           min_sep=min_sep, max_participations=max_participations, noise_multiplier=nm,
                                           key=key, compute_dtype=compute_dtype, backend=backend)
    streaming = strategy.streaming_matrix(n_steps=n_steps, min_sep=min_sep, max_participations=max_participations)
    row_l2 = None if isinstance(strategy, IdentityStrategy) else streaming.row_norms_squared(n_steps).clamp_min(0).sqrt()
    fingerprint = repr(sorted(serialize_strategy(strategy).items(), key=lambda kv: kv[0]))
    state0 = MFNoiseState(streaming.init_multiply(grad_template), 0, key, None, fingerprint, n_steps)

    def noise_fn(clipped_grads, st: MFNoiseState):
        with torch.profiler.record_function("opake::mf_gaussian_noise"):
            if isinstance(clipped_grads, SecondMomentClippingOutput):
                raise InputTypeError("mf_gaussian_noise was constructed without `second_moment_strategy` and cannot "
                                     "consume SecondMomentClippingOutput inputs.")
            if isinstance(clipped_grads, NoisedPytree) or not isinstance(clipped_grads, ClippedPytree):
                raise InputTypeError("mf_gaussian_noise expects ClippedPytree inputs.")
            t = st._step_counter
            _check_horizon(t, n_steps)
            mn = clipped_grads.max_norm
            if st._first_max_norm is not None and not _same_norm(st._first_max_norm, mn):
                raise ConfigurationError("matrix-factorisation noise requires a constant max_norm over the run; got "
                                         f"{mn!r} after {st._first_max_norm!r}")
            base = per_group_noise_stddev(mn, nm) if isinstance(mn, PerGroup) else (0.0 if nm == 0 else nm * mn)
            # column key and order of operations as in the reference's streaming engine (_engine.py:41-52,415-432): the iid
            # column is scaled by the noise stddev BEFORE it goes through C^{-1}, so the streaming state holds scaled
            # values and a state written by either implementation continues correctly in the other
            z = iid_normal_like(clipped_grads.pytree, fold_in(st._rng_key, MF_STREAM_FOLD, MF_COLUMN_FOLD, t),
                                compute_dtype=compute_dtype, backend=backend)
            from ..engine.pytree import tree_flatten_with_paths, tree_unflatten

            paths, zl, td = tree_flatten_with_paths(z)
            if isinstance(base, PerGroup):
                z = tree_unflatten(td, [x * base.for_path(p) for p, x in zip(paths, zl)])
            else:
                z = tree_unflatten(td, [x * base for x in zl])
            w, inner = streaming.multiply_next(z, st._inner_state)
            noisy = tree_map(lambda g, x: (g.to(compute_dtype) + x.to(compute_dtype)).to(g.dtype), clipped_grads.pytree, w)
            r = 1.0 if row_l2 is None else float(row_l2[t])
            return (NoisedPytree(noisy, mn, base * r),
                    replace(st, _inner_state=inner, _step_counter=t + 1, _first_max_norm=mn))

    return noise_fn, state0


# ------------------------------------------------------------------------------------------------ state codec
# Wire layout of packages/opake-dpftrl/src/opake/api/dpftrl/noise/_state_codec.py:348-446 (layout version 1):
#   layout_version, _step_counter, _rng_key.seed, _rng_key.impl,
#   _inner_state[1][i]                  the i-th tensor of the streaming state, leaves in sorted-key order
#   _inner_state_fields                 JSON list of those keys
#   _first_max_norm                     JSON: {"kind": "none"} | {"kind": "scalar", "value": c} | {"kind": "per_group", ...}
#   _first_max_norm_sync_fingerprint    leading signed 64 bits of SHA-256 over a canonical JSON of the latched norm
def _json(value) -> str:
    import json

    return json.dumps(value, sort_keys=True, separators=(",", ":"))


def _encode_max_norm(mn) -> str:
    if mn is None:
        return _json({"kind": "none"})
    if isinstance(mn, PerGroup):
        return _json({"kind": "per_group", "groups": [[list(p), g] for p, g in mn.groups.items()],
                      "values": [[g, v] for g, v in mn.values.items()]})
    return _json({"kind": "scalar", "value": float(mn)})


def _decode_max_norm(text, template):
    import json

    if not isinstance(text, str):
        return None if text is None else float(text)
    obj = json.loads(text)
    if obj["kind"] == "none":
        return None
    if obj["kind"] == "scalar":
        return float(obj["value"])
    return PerGroup({tuple(p): g for p, g in obj["groups"]}, {g: v for g, v in obj["values"]})


def max_norm_fingerprint(mn) -> int | None:
    import hashlib

    if mn is None:
        return None
    if isinstance(mn, PerGroup):
        payload = {"kind": "mf_noise_per_group_max_norm", "groups": sorted(mn.groups.items()), "values": sorted(mn.values.items())}
    else:
        payload = {"kind": "mf_noise_scalar_max_norm", "c": float(mn)}
    return int.from_bytes(hashlib.sha256(_json(payload).encode()).digest()[:8], "big", signed=True)


def _inner_tensors(inner) -> list[torch.Tensor]:
    from ..engine.pytree import tree_flatten

    return [t for t in tree_flatten(inner)[0] if isinstance(t, torch.Tensor)]


def _save_state(s: MFNoiseState) -> dict[str, Any]:
    out: dict[str, Any] = {"layout_version": STATE_LAYOUT_VERSION}
    fields = []
    for i, t in enumerate(_inner_tensors(s._inner_state)):
        name = f"_inner_state[1][{i}]"
        out[name] = t
        fields.append(name)
    out.update({"_step_counter": int(s._step_counter), "_rng_key.seed": s._rng_key.seed, "_rng_key.impl": s._rng_key.impl,
                "_first_max_norm_sync_fingerprint": max_norm_fingerprint(s._first_max_norm),
                "_first_max_norm": _encode_max_norm(s._first_max_norm), "_inner_state_fields": _json(sorted(fields))})
    return out


def _load_state(template: MFNoiseState, sd) -> MFNoiseState:
    from ..base.exceptions import CheckpointError
    from ..engine.pytree import tree_flatten, tree_unflatten

    ver = sd.get("layout_version")
    if ver != STATE_LAYOUT_VERSION:
        raise CheckpointError(f"unsupported MF noise-state layout version {ver!r}; expected {STATE_LAYOUT_VERSION}")
    step = int(sd.get("_step_counter", 0))
    if "_inner_state_fields" in sd:
        import json

        fields = json.loads(sd["_inner_state_fields"])
        leaves, td = tree_flatten(template._inner_state)
        slots = [i for i, t in enumerate(leaves) if isinstance(t, torch.Tensor)]
        if len(fields) != len(slots):
            raise CheckpointError(f"MF noise-state holds {len(fields)} tensors, the configured strategy and parameter tree "
                                  f"need {len(slots)}: rebuild the mechanism with the checkpoint's strategy")
        for i, name in zip(slots, sorted(fields, key=lambda f: [int(x) for x in f.replace("]", "").split("[")[1:]])):
            saved, want = sd[name], leaves[i]
            if tuple(saved.shape) != tuple(want.shape):
                raise CheckpointError(f"MF noise-state tensor {name} has shape {tuple(saved.shape)}, the configured strategy "
                                      f"needs {tuple(want.shape)}")
            leaves[i] = saved.to(device=want.device, dtype=want.dtype)
        # streaming states that count their own steps (banded Toeplitz ring) follow the mechanism's step counter
        leaves = [step if (isinstance(t, int) and not isinstance(t, bool)) else t for t in leaves]
        inner = tree_unflatten(td, leaves)
        mn = _decode_max_norm(sd.get("_first_max_norm"), template._first_max_norm)
        fp = sd.get("_first_max_norm_sync_fingerprint")
        if mn is not None and fp is not None and fp != max_norm_fingerprint(mn):
            raise CheckpointError("MF max-norm latch fingerprint does not match its saved value")
    else:       # files of earlier versions of this package: dotted inner-state keys, plain max norm
        inner = _fsd({"_inner_state": template._inner_state}, sd)["_inner_state"]
        mn = template._first_max_norm
        if "_first_max_norm" in sd:
            mn = float(sd["_first_max_norm"])
        elif isinstance(mn, PerGroup):
            mn = PerGroup(mn.groups, {g: sd.get(f"_first_max_norm.values.{g}", v) for g, v in mn.values.items()})
    return MFNoiseState(inner, step,
                        RngKey(int(sd.get("_rng_key.seed", template._rng_key.seed)),
                               str(sd.get("_rng_key.impl", template._rng_key.impl))), mn, template._strategy_fingerprint,
                        template._n_steps)


register_serializer(MFNoiseState, _save_state, _load_state)


def sync_mf_noise_state(state: MFNoiseState) -> MFNoiseState:
    from ..engine import distributed as D

    D.assert_string_equal(str(state._rng_key.seed), name="MFNoiseState._rng_key.seed")
    D.assert_scalar_equal(state._step_counter, name="MFNoiseState._step_counter")
    D.assert_string_equal(state._strategy_fingerprint, name="MFNoiseState strategy")
    return state


def _register():
    from ..engine import distributed as D

    D.register_sync_type(MFNoiseState, sync_mf_noise_state)


_register()

from .strategies import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, identity_strategy,  # noqa: E402,F401
                         lambda_cgd_strategy)

__all__ = ["MFNoiseState", "mf_gaussian_noise", "MF_STREAM_FOLD", "sync_mf_noise_state", "iid_normal_like"]
