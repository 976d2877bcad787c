"""Causal-LM loss replacements (packages/opake-patches/src/opake/api/patches/transformers/components/
cross_entropy.py:12-368).

``opake_causal_lm_loss`` is a drop-in for a model's ``loss_function``: shift, cross entropy through this package's
kernel function (which has a batching rule), mean over the non-ignored tokens OF THE CALL. Under ``vmap(grad)`` the
call sees one example, so the reduction never couples examples; reductions over a batch (``num_items_in_batch``) are
refused for that reason.

``make_fused_ce_causal_lm_forward`` wraps a ``*ForCausalLM.forward``: a labelled call with ``loss_only=True`` skips the
logits and feeds the final hidden states to the fused linear cross entropy (tcgen05 GEMM with the softmax statistics in
its epilogue on CUDA bf16, a chunked formulation elsewhere); every other call goes to the original forward."""
from __future__ import annotations

import functools

import torch
import torch.nn as nn

from ....ops.lce import opake_linear_cross_entropy_loss
from ...kernels.functions import opake_cross_entropy

__all__ = ["opake_causal_lm_loss", "apply_causal_lm_loss_function_patch", "make_fused_ce_causal_lm_forward",
           "apply_fused_linear_ce_patch", "fused_linear_ce_supports"]

_MARK = "_opake_fused_ce"
# families whose ``*ForCausalLM`` is backbone -> lm_head -> loss with nothing in between
_PLAIN_HEADS = ("llama", "mistral", "ministral", "mellum", "qwen2", "qwen3", "smollm3", "gemma", "gemma2", "gemma3", "gemma3_text",
                "granite", "cohere", "cohere2", "olmo2", "olmo3", "glm4", "exaone4", "phi3", "mixtral", "qwen3_moe", "olmoe")


def opake_causal_lm_loss(logits, labels, vocab_size: int, ignore_index: int = -100, shift_labels=None,
                         label_smoothing: float = 0.0, num_items_in_batch=None, **_kw) -> torch.Tensor:
    if num_items_in_batch is not None:
        raise ValueError("a loss normalised by num_items_in_batch couples the examples of a batch; per-example clipping "
                         "needs a per-example loss")
    if shift_labels is None:
        shift_labels = nn.functional.pad(labels, (0, 1), value=ignore_index)[..., 1:]
    flat = logits.reshape(-1, vocab_size)
    lab = shift_labels.reshape(-1).to(flat.device)
    if label_smoothing:
        return nn.functional.cross_entropy(flat.float(), lab, ignore_index=ignore_index, label_smoothing=float(label_smoothing))
    nll = opake_cross_entropy(flat, lab, ignore_index=ignore_index)
    return nll.sum() / (lab != ignore_index).sum().clamp(min=1)


def apply_causal_lm_loss_function_patch(model, target_cls: type | None = None) -> int:
    n = 0
    for m in model.modules():
        if (target_cls is None and hasattr(m, "loss_function") and hasattr(m, "lm_head")) or (target_cls is not None and type(m) is target_cls):
            m.loss_function = opake_causal_lm_loss
            n += 1
    return n


def fused_linear_ce_supports(model) -> bool:
    cfg = getattr(model, "config", None)
    return (getattr(cfg, "model_type", None) in _PLAIN_HEADS and hasattr(model, "lm_head") and hasattr(model, "model")
            and isinstance(getattr(model, "lm_head"), nn.Linear) and model.lm_head.bias is None)


def _fused_call_ok(logits_to_keep, kwargs) -> bool:
    if not isinstance(logits_to_keep, int) or isinstance(logits_to_keep, bool) or logits_to_keep != 0:
        return False
    if kwargs.get("shift_labels") is not None or kwargs.get("weight") is not None or kwargs.get("num_items_in_batch") is not None:
        return False
    if kwargs.get("label_smoothing"):
        return False
    return not torch.is_tensor(kwargs.get("ignore_index", -100))


def make_fused_ce_causal_lm_forward(original):
    if getattr(original, _MARK, False):
        return original

    @functools.wraps(original)
    def forward(self, *args, labels=None, logits_to_keep=0, loss_only: bool = False, **kwargs):
        router = kwargs.get("output_router_logits")
        if router is None:
            router = getattr(self.config, "output_router_logits", False)
        if labels is None or not loss_only or router or not _fused_call_ok(logits_to_keep, kwargs):
            return original(self, *args, labels=labels, logits_to_keep=logits_to_keep, **kwargs)
        ignore_index = int(kwargs.pop("ignore_index", -100))
        return_dict = kwargs.pop("return_dict", None)
        return_dict = return_dict if return_dict is not None else getattr(self.config, "return_dict", True)
        outputs = self.model(*args, **kwargs)
        hidden = outputs[0]
        scale = getattr(self, "logit_scale", None)
        if scale is None:
            scale = getattr(self.config, "logit_scale", None)
        scale = float(1.0 if scale is None else scale) / float(getattr(self.config, "logits_scaling", None) or 1.0)
        softcap = float(getattr(self.config, "final_logit_softcapping", None) or 0.0)
        nll_sum = opake_linear_cross_entropy_loss(hidden, self.lm_head.weight, labels, ignore_index=ignore_index,
                                                  logit_softcapping=softcap, logit_scale=scale)
        n_valid = (labels[..., 1:] != ignore_index).sum().clamp(min=1)
        loss = nll_sum.sum() / n_valid          # mean over the non-ignored tokens of the call (one example under vmap)
        if not return_dict:
            return (loss, None, *outputs[1:])
        from transformers.modeling_outputs import CausalLMOutputWithPast, MoeCausalLMOutputWithPast

        common = dict(loss=loss, logits=None, past_key_values=getattr(outputs, "past_key_values", None),
                      hidden_states=getattr(outputs, "hidden_states", None), attentions=getattr(outputs, "attentions", None))
        if hasattr(outputs, "router_logits"):
            return MoeCausalLMOutputWithPast(aux_loss=None, router_logits=outputs.router_logits, **common)
        return CausalLMOutputWithPast(**common)

    setattr(forward, _MARK, True)
    return forward


def apply_fused_linear_ce_patch(model) -> bool:
    """Installs the conditional fused forward on ``type(model)`` when the family's head is plain. Returns whether."""
    if not fused_linear_ce_supports(model):
        return False
    cls = type(model)
    if not getattr(cls.forward, _MARK, False):
        cls.forward = make_fused_ce_causal_lm_forward(cls.forward)
    return True
