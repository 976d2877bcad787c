"""User-extensible model-family machinery (packages/opake-patches/src/opake/api/patches/transformers/_family.py:100-246,
_factory.py:118-260, _registry.py).

Built-in families are rows of ``registry.FAMILIES`` (a declarative ``FamilySpec`` each) handled by
``patches.apply_transformers_model_patches``. A downstream architecture that is not one of them registers an APPLY
FUNCTION instead, built from two factories:

``make_apply_family_patches``  module-level replacements in the family's modeling module (``repeat_kv``,
    ``eager_attention_forward``, the module's own ``"sdpa"`` attention entry, ``apply_rotary_pos_emb``, the mask
    builders bound in that module). Idempotent per family and per concern.
``make_apply_model_patches``   per-instance forward replacements by role (``"mlp"``, ``"rms_norm"``, ``"decoder_layer"``,
    ``"experts"``, ``"causal_lm"``) chosen by KIND: a registered name or a factory ``original_forward -> new_forward``.

``register_family(name, apply_fn)`` makes ``apply_model_patches(model)`` route models with that ``model_type`` to the
function. Kinds are registered with ``register_activation_kind`` / ``register_rms_norm_kind`` /
``register_fused_add_rms_kind`` / ``register_moe_kind``.
"""
from __future__ import annotations

import importlib
import types
from typing import Any, Callable

from ...base.exceptions import ConfigurationError
from ..kernels.functions import opake_fused_add_rms_norm, opake_geglu, opake_rms_norm, opake_swiglu
from . import components as C
from .registry import FAMILIES, FamilySpec
from .registry import register_family as _register_spec

__all__ = ["family_name", "supported_families", "register_family", "get_family_apply_fn", "make_apply_family_patches",
           "make_apply_model_patches", "register_activation_kind", "register_rms_norm_kind", "register_fused_add_rms_kind",
           "register_moe_kind"]

ForwardFactory = Callable[[Callable], Callable]
_USER_FAMILIES: dict[str, Callable] = {}
_PATCHED_CONCERNS: dict[str, set] = {}


def family_name(model) -> str | None:
    """``model.config.model_type`` when present, else the ``transformers.models.<name>`` part of the class's module."""
    kind = getattr(getattr(model, "config", None), "model_type", None)
    if kind:
        return str(kind)
    parts = type(model).__module__.split(".")
    if len(parts) >= 3 and parts[0] == "transformers" and parts[1] == "models":
        return parts[2]
    return None


def register_family(name_or_spec, apply_fn: Callable | None = None):
    """``register_family(FamilySpec(...))`` adds a declarative built-in style family; ``register_family(name, apply_fn)``
    routes models of that type to ``apply_fn(model, *, performance=True, compat=True, **kwargs)``. Re-registering a name
    replaces the previous entry."""
    if isinstance(name_or_spec, FamilySpec):
        return _register_spec(name_or_spec)
    if not callable(apply_fn):
        raise ConfigurationError("register_family(name, apply_fn) needs a callable apply function")
    _USER_FAMILIES[str(name_or_spec)] = apply_fn
    return apply_fn


def get_family_apply_fn(name: str | None):
    return _USER_FAMILIES.get(name) if name else None


def supported_families() -> list[str]:
    return sorted(set(FAMILIES) | set(_USER_FAMILIES))


# ---------------------------------------------------------------------------------------------- kinds
def _swiglu(original):
    def forward(self, x):
        return self.down_proj(opake_swiglu(self.gate_proj(x), self.up_proj(x)))
    return forward


def _geglu(approximate: str):
    def factory(original):
        def forward(self, x):
            return self.down_proj(opake_geglu(self.gate_proj(x), self.up_proj(x), approximate=approximate))
        return forward
    return factory


def _fused_gate_up_swiglu(original):
    def forward(self, x):
        g, u = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(opake_swiglu(g, u))
    return forward


def _rms(offset: float):
    def factory(original):
        def forward(self, hidden_states):
            eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
            return opake_rms_norm(hidden_states, self.weight, eps, offset)
        return forward
    return factory


def _fused_add_rms_llama(original):
    """Pre-norm decoder layer (Llama layout: ``input_layernorm``, ``self_attn``, ``post_attention_layernorm``, ``mlp``):
    the residual add after attention and the following RMSNorm run as one kernel (and one in the backward)."""
    def forward(self, hidden_states, *args, **kwargs):
        residual = hidden_states
        h = self.input_layernorm(hidden_states)
        attn = self.self_attn(h, *args, **kwargs) if args else self.self_attn(hidden_states=h, **kwargs)
        attn = attn[0] if isinstance(attn, tuple) else attn
        norm = self.post_attention_layernorm
        eps = getattr(norm, "variance_epsilon", getattr(norm, "eps", 1e-6))
        h2, summed = opake_fused_add_rms_norm(attn, residual, norm.weight, eps, getattr(norm, "_opake_offset", 0.0))
        return summed + self.mlp(h2)
    return forward


def _dense_experts(original):
    return C.dense_experts_forward


_ACTIVATION_KINDS: dict[str, ForwardFactory] = {"swiglu": _swiglu, "geglu_exact": _geglu("none"), "geglu_approx": _geglu("tanh"),
                                                "fused_gate_up_swiglu": _fused_gate_up_swiglu}
_RMS_NORM_KINDS: dict[str, ForwardFactory] = {"llama": _rms(0.0), "gemma": _rms(1.0)}
_FUSED_ADD_RMS_KINDS: dict[str, ForwardFactory] = {"llama": _fused_add_rms_llama}
_MOE_KINDS: dict[str, ForwardFactory] = {"dense": _dense_experts}


def register_activation_kind(name: str, factory: ForwardFactory) -> None:
    _ACTIVATION_KINDS[name] = factory


def register_rms_norm_kind(name: str, factory: ForwardFactory) -> None:
    _RMS_NORM_KINDS[name] = factory


def register_fused_add_rms_kind(name: str, factory: ForwardFactory) -> None:
    _FUSED_ADD_RMS_KINDS[name] = factory


def register_moe_kind(name: str, factory: ForwardFactory) -> None:
    _MOE_KINDS[name] = factory


def _resolve(spec, table: dict[str, ForwardFactory]):
    if spec is None:
        return None
    if callable(spec):
        return spec
    if spec in table:
        return table[spec]
    raise ConfigurationError(f"unknown kind {spec!r}; registered: {sorted(table)}. Pass a callable, or register the name first")


# ---------------------------------------------------------------------------------------------- factories
def make_apply_family_patches(*, family: str, module_path: str, repeat_kv_replacement=C.repeat_kv,
                              eager_attention_replacement=C.eager_attention_forward,
                              sdpa_attention_replacement=C.vmap_sdpa_attention_forward,
                              rope_replacement: Any = "wrap", masking_module_patcher: Any = "default"):
    """Returns ``apply(*, performance=True, compat=True, kernels=None, **kwargs)`` that patches module-level names of
    ``module_path``. ``eager_attention`` (default: ``compat``) covers ``repeat_kv``, ``eager_attention_forward``, the
    module's own ``"sdpa"`` entry and the mask builders bound in the module; ``rope`` (default: ``kernels``, itself
    defaulting to ``performance``) covers ``apply_rotary_pos_emb``. ``None`` for a replacement skips it.
    ``rope_replacement="wrap"`` keeps the module's own function off the fast path (partial rotary dimensions etc.)."""

    def apply(*, performance: bool = True, compat: bool = True, kernels: bool | None = None, **kwargs) -> None:
        kernels = performance if kernels is None else kernels
        want = set()
        if kwargs.get("eager_attention", compat):
            want.add("eager_attention")
        if kwargs.get("rope", kernels):
            want.add("rope")
        done = _PATCHED_CONCERNS.setdefault(family, set())
        if not want or want <= done:
            return
        try:
            mod = importlib.import_module(module_path)
        except ImportError:
            return
        if "eager_attention" in want and "eager_attention" not in done:
            if repeat_kv_replacement is not None and hasattr(mod, "repeat_kv"):
                mod.repeat_kv = repeat_kv_replacement
            if eager_attention_replacement is not None and hasattr(mod, "eager_attention_forward"):
                mod.eager_attention_forward = eager_attention_replacement
            table = mod.__dict__.get("ALL_ATTENTION_FUNCTIONS")
            if sdpa_attention_replacement is not None and table is not None and not hasattr(table, "_global_mapping"):
                table["sdpa"] = sdpa_attention_replacement          # a mapping owned by this module alone
            if masking_module_patcher == "default":
                from .runtime.masking import apply_masking_patches

                apply_masking_patches()
            elif masking_module_patcher is not None:
                masking_module_patcher(mod)
            done.add("eager_attention")
        if "rope" in want and "rope" not in done and rope_replacement is not None and hasattr(mod, "apply_rotary_pos_emb"):
            fn = mod.apply_rotary_pos_emb
            if not getattr(fn, "_opake_rope", False):
                mod.apply_rotary_pos_emb = C.rope.make_rope_replacement(fn) if rope_replacement == "wrap" else rope_replacement
            done.add("rope")

    apply.__name__ = apply.__qualname__ = f"apply_{family}_family_patches"
    apply._opake_family = family
    return apply


def _patch_instances(model, cls_name: str | None, factory, mark: str) -> int:
    if cls_name is None or factory is None:
        return 0
    n = 0
    for m in model.modules():
        if type(m).__name__ == cls_name and not getattr(m, mark, False):
            new = factory(type(m).forward)
            m.forward = types.MethodType(new, m)
            setattr(m, mark, True)
            n += 1
    return n


def make_apply_model_patches(*, family: str, family_apply: Callable | None, module_path: str, classes: dict[str, str],
                             activation_kind=None, rms_norm_kind=None, fused_add_rms_kind=None, moe_kind=None,
                             fused_linear_cross_entropy: bool = True, chunked_linear_cross_entropy: bool | int = False):
    """Returns ``apply(model=None, *, performance=True, compat=True, kernels=None, **kwargs) -> dict`` (a report of what
    was patched). Per-concern keywords default into the umbrella flags: ``rope``, ``rms_norm``, ``activation``,
    ``cross_entropy`` -> ``kernels`` (default: ``performance``); ``kv_cache``, ``fused_linear_cross_entropy`` ->
    ``performance``; ``eager_attention``, ``batchify``, ``dropout``, ``moe`` -> ``compat``. Recognised roles in
    ``classes``: ``"mlp"``, ``"rms_norm"``, ``"decoder_layer"``, ``"experts"``, ``"causal_lm"``; absent roles are
    skipped. ``chunked_linear_cross_entropy`` is accepted for compatibility: the fused loss of this package chooses its
    own formulation (tensor-core epilogue on CUDA bf16, chunked elsewhere)."""
    act = _resolve(activation_kind, _ACTIVATION_KINDS)
    rms = _resolve(rms_norm_kind, _RMS_NORM_KINDS)
    far = _resolve(fused_add_rms_kind, _FUSED_ADD_RMS_KINDS)
    moe = _resolve(moe_kind, _MOE_KINDS)
    if isinstance(chunked_linear_cross_entropy, int) and not isinstance(chunked_linear_cross_entropy, bool) \
            and chunked_linear_cross_entropy < 0:
        raise ConfigurationError("chunked_linear_cross_entropy must be a boolean or a non-negative integer")

    def apply(model=None, *, performance: bool = True, compat: bool = True, kernels: bool | None = None, **kwargs) -> dict:
        kernels = performance if kernels is None else kernels
        if family_apply is not None:
            family_apply(performance=performance, compat=compat, kernels=kernels, **kwargs)
        report = {"family": family, "mlps": 0, "norms": 0, "decoder_layers": 0, "experts": 0, "kv_cache": 0, "batchify": 0,
                  "dropouts": 0, "loss_function": 0, "fused_linear_cross_entropy": False}
        if model is None:
            return report
        root = next((m for m in model.modules() if type(m).__name__ == classes.get("causal_lm")), None)
        if root is not None and kwargs.get("fused_linear_cross_entropy", performance) and fused_linear_cross_entropy:
            cls = type(root)
            if hasattr(root, "lm_head") and hasattr(root, "model"):
                cls.forward = C.make_fused_ce_causal_lm_forward(cls.forward)
                report["fused_linear_cross_entropy"] = True
        if kwargs.get("dropout", compat):
            report["dropouts"] = C.disable_dropout(model)
        if root is not None and kwargs.get("kv_cache", performance):
            C.disable_kv_cache(root)
            report["kv_cache"] = C.apply_kv_cache_patch(type(root), model)
        if root is not None and kwargs.get("batchify", compat):
            report["batchify"] = C.apply_batchify_patch(type(root), model)
        if kwargs.get("activation", kernels):
            report["mlps"] = _patch_instances(model, classes.get("mlp"), act, "_opake_patched")
        if kwargs.get("rms_norm", kernels):
            report["norms"] = _patch_instances(model, classes.get("rms_norm"), rms, "_opake_patched")
        if kwargs.get("fused_add_rms_norm", kernels):
            report["decoder_layers"] = _patch_instances(model, classes.get("decoder_layer"), far, "_opake_layer_patched")
        if kwargs.get("moe", compat):
            report["experts"] = _patch_instances(model, classes.get("experts"), moe, "_opake_patched")
        if root is not None and kwargs.get("cross_entropy", kernels) and hasattr(root, "loss_function"):
            report["loss_function"] = C.apply_causal_lm_loss_function_patch(model, type(root))
        return report

    apply.__name__ = apply.__qualname__ = f"apply_{family}_patches"
    apply._opake_family = family
    return apply
