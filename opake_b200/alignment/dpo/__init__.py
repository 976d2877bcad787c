"""``alignment.dpo``: per-sequence log-probabilities, per-pair loss heads, preference collator, reference-policy
helpers, reward telemetry and prompt extraction."""
from . import collator, data, loss, metric, reference
from ..logprob import fused_sequence_logp, sequence_logp
from .collator import preference_collator
from .data import extract_prompt
from .loss import *  # noqa: F401,F403
from .metric import reward_metrics
from .reference import compute_ref_logprobs_for_dataset, ema_update_reference, null_ref_context, with_disabled_adapter

__all__ = ["collator", "data", "loss", "metric", "reference", "sequence_logp", "fused_sequence_logp",
           "preference_collator", "extract_prompt", "reward_metrics", "compute_ref_logprobs_for_dataset",
           "ema_update_reference", "null_ref_context", "with_disabled_adapter", *loss.__all__]
