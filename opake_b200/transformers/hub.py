"""Model card and Hub helpers (packages/opake-transformers/src/opake/api/transformers/trainer/_hub.py:80-460). The
model card gets a differential-privacy section between two fixed markers so that re-saving replaces it in place.
Uploading needs ``huggingface_hub`` and network access; both are checked at call time."""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from ..base.exceptions import OperationError

__all__ = ["DPTrainingSummary", "create_model_card", "init_hf_repo", "push_to_hub", "DP_BEGIN", "DP_END"]

DP_BEGIN = "<!-- opake:dp-summary:begin -->"
DP_END = "<!-- opake:dp-summary:end -->"


@dataclass
class DPTrainingSummary:
    model_name: str = "model"
    base_model: str | None = None
    dataset: str | None = None
    epsilon: float | None = None
    delta: float | None = None
    noise_multiplier: float | None = None
    clipping_norm: float | str | None = None
    clipping_mode: str = "fixed"
    mechanism: str = "gaussian"
    sampling: str = "poisson"
    sample_rate: float | None = None
    steps: int | None = None
    expected_batch_size: float | None = None
    optimizer: str | None = None
    learning_rate: float | None = None
    metrics: dict = field(default_factory=dict)

    def privacy_section(self) -> str:
        def fmt(v, spec="g"):
            return "n/a" if v is None else (format(v, spec) if isinstance(v, (int, float)) else str(v))
        rows = [("Guarantee", f"({fmt(self.epsilon, '.4g')}, {fmt(self.delta, '.3g')})-DP" if self.epsilon is not None else "not accounted"),
                ("Noise mechanism", self.mechanism), ("Noise multiplier", fmt(self.noise_multiplier, ".6g")),
                ("Clipping", f"{self.clipping_mode}, norm {fmt(self.clipping_norm)}"), ("Sampling", self.sampling),
                ("Sampling rate", fmt(self.sample_rate, ".6g")), ("Expected batch size", fmt(self.expected_batch_size)),
                ("Optimizer steps", fmt(self.steps)), ("Optimizer", fmt(self.optimizer)), ("Learning rate", fmt(self.learning_rate))]
        table = "\n".join(f"| {k} | {v} |" for k, v in rows)
        return (f"{DP_BEGIN}\n## Differential privacy\n\nThis model was trained with per-example gradient clipping and calibrated "
                f"noise. The guarantee covers the training examples under add/remove adjacency.\n\n| | |\n|---|---|\n{table}\n{DP_END}")


def create_model_card(summary: DPTrainingSummary, existing: str | None = None) -> str:
    """New card, or ``existing`` with its DP section replaced (appended if it had none)."""
    section = summary.privacy_section()
    if existing:
        if DP_BEGIN in existing and DP_END in existing:
            head, rest = existing.split(DP_BEGIN, 1)
            return head + section + rest.split(DP_END, 1)[1]
        return existing.rstrip() + "\n\n" + section + "\n"
    meta = ["---", "library_name: opake", "tags:", "- differential-privacy"]
    if summary.base_model:
        meta.append(f"base_model: {summary.base_model}")
    if summary.dataset:
        meta += ["datasets:", f"- {summary.dataset}"]
    meta.append("---")
    body = [f"# {summary.model_name}", ""]
    if summary.base_model:
        body.append(f"Fine-tuned from `{summary.base_model}`" + (f" on `{summary.dataset}`." if summary.dataset else "."))
        body.append("")
    if summary.metrics:
        body += ["## Evaluation", ""] + [f"- {k}: {v}" for k, v in summary.metrics.items()] + [""]
    return "\n".join(meta + body) + section + "\n"


def init_hf_repo(repo_id: str, token: str | None = None, private: bool | None = None) -> str:
    try:
        from huggingface_hub import create_repo
    except Exception as e:
        raise OperationError("push_to_hub needs the huggingface_hub package") from e
    return create_repo(repo_id, token=token, private=private, exist_ok=True).repo_id


def push_to_hub(folder: str, repo_id: str, *, token: str | None = None, commit_message: str = "End of training",
                revision: str | None = None, private: bool | None = None) -> str:
    try:
        from huggingface_hub import upload_folder
    except Exception as e:
        raise OperationError("push_to_hub needs the huggingface_hub package") from e
    if not os.path.isdir(folder):
        raise OperationError(f"nothing to push: {folder} does not exist")
    init_hf_repo(repo_id, token, private)
    return str(upload_folder(repo_id=repo_id, folder_path=folder, token=token, commit_message=commit_message, revision=revision,
                             ignore_patterns=["checkpoint-*", "*.tmp"]))
