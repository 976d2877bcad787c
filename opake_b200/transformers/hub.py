"""Model card and Hub helpers (packages/opake-transformers/src/opake/api/transformers/trainer/_hub.py:80-460).

The card has the usual Hugging Face layout (metadata block, description, evaluation results, training
hyper-parameters, training results table, framework versions) plus a differential-privacy section between two fixed
markers, so that re-saving a card replaces that section in place. The privacy values come from the trainer, in this
order: the last logged ``privacy_epsilon`` / ``privacy_delta`` / ``privacy_noise_multiplier`` (the budget actually
spent), the live accountant, the resolved values in the trainer state, the arguments. Uploading needs
``huggingface_hub`` and network access; both are checked at call time, and only process zero touches the Hub."""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Any

from ..base.exceptions import OperationError

__all__ = ["DPTrainingSummary", "create_model_card", "init_hf_repo", "push_to_hub", "build_privacy_summary", "splice_dp_section",
           "DP_BEGIN", "DP_END", "CARD_TAGS"]

DP_BEGIN = "<!-- opake:dp-summary:begin -->"
DP_END = "<!-- opake:dp-summary:end -->"
CARD_TAGS = ("differential-privacy", "opake")
_HYPERPARAMETERS = ("learning_rate", "per_device_train_batch_size", "per_device_eval_batch_size", "seed", "optim", "lr_scheduler",
                    "warmup_steps", "num_train_epochs", "max_steps", "weight_decay", "adam_beta1", "adam_beta2", "adam_epsilon",
                    "bf16", "clipping_mode", "clipping_norm", "privacy_noise_mechanism", "sampling_mode", "microbatch_size")
_FRAMEWORK_RE = re.compile(r"(### Framework versions\b.*?)(?=\n## |\Z)", re.DOTALL)


def _package_version() -> str:
    try:
        from .. import __version__

        return str(__version__)
    except Exception:
        return "unknown"


def _as_list(v) -> list:
    if v is None:
        return []
    return [v] if isinstance(v, str) else list(v)


def build_privacy_summary(trainer) -> dict[str, Any]:
    """``{"epsilon", "delta", "noise_multiplier", "clipping_norm"}``; a value nobody knows is the string ``"unknown"``."""
    a, st = trainer.args, trainer.state
    eps: Any = "unknown"
    delta: Any = "unknown"
    nm: Any = "unknown"
    for entry in reversed(getattr(st, "log_history", []) or []):
        if "privacy_epsilon" in entry and entry["privacy_epsilon"] is not None:
            eps = round(float(entry["privacy_epsilon"]), 4)
        if entry.get("privacy_delta") is not None:
            delta = entry["privacy_delta"]
        if entry.get("privacy_noise_multiplier") is not None:
            nm = round(float(entry["privacy_noise_multiplier"]), 6)
        if eps != "unknown":
            break
    rt = getattr(trainer, "_rt", None) or {}
    accountant = getattr(trainer, "accountant", None)
    if eps == "unknown" and accountant is not None and rt.get("target_delta") is not None:
        try:
            eps = round(float(accountant.epsilon_at(rt["target_delta"])), 4)
            delta = rt["target_delta"]
        except Exception:
            pass
    if eps == "unknown" and getattr(st, "privacy_epsilon", None) is not None:
        eps = round(float(st.privacy_epsilon), 4)
    if nm == "unknown":
        for v in (rt.get("noise_multiplier"), getattr(st, "privacy_resolved_noise_multiplier", None), a.privacy_noise_multiplier):
            if v is not None:
                nm = round(float(v), 6)
                break
    if delta == "unknown":
        for v in (rt.get("target_delta"), getattr(st, "privacy_delta", None), getattr(a, "privacy_target_delta", None)):
            if v is not None:
                delta = v
                break
    cn = rt.get("clip_norm", a.clipping_norm)
    if cn is None:
        clip: Any = "unknown"
    elif hasattr(cn, "effective"):
        clip = round(float(cn.effective), 4)
    elif isinstance(cn, dict):
        clip = json.dumps(cn, sort_keys=True)
    else:
        clip = float(cn)
    return {"epsilon": eps, "delta": delta, "noise_multiplier": nm, "clipping_norm": clip}


@dataclass
class DPTrainingSummary:
    model_name: str = "model"
    base_model: str | None = None
    dataset: str | list | None = None
    language: str | list | None = None
    license: str | None = None
    tags: list = field(default_factory=list)
    tasks: str | list | None = None
    dataset_tags: str | list | None = None
    dataset_args: str | list | None = None
    epsilon: float | str | None = None
    delta: float | str | None = None
    noise_multiplier: float | str | None = None
    clipping_norm: float | str | None = None
    clipping_mode: str = "fixed"
    mechanism: str = "gaussian"
    sampling: str = "poisson"
    sample_rate: float | None = None
    steps: int | None = None
    expected_batch_size: float | None = None
    optimizer: str | None = None
    learning_rate: float | None = None
    metrics: dict = field(default_factory=dict)               # last evaluation
    hyperparameters: dict = field(default_factory=dict)
    eval_lines: list = field(default_factory=list)             # training results table rows

    # ---------------------------------------------------------------------------------------------- from a trainer
    @classmethod
    def from_trainer(cls, trainer, language=None, license=None, tags=None, model_name=None, finetuned_from=None, tasks=None,
                     dataset_tags=None, dataset=None, dataset_args=None) -> "DPTrainingSummary":
        a, st = trainer.args, trainer.state
        rt = getattr(trainer, "_rt", None) or {}
        if finetuned_from is None:
            cfg = getattr(getattr(trainer, "model", None), "config", None)
            name = getattr(cfg, "_name_or_path", None)
            if name and not os.path.isdir(str(name)):
                finetuned_from = name
        if license is None:
            license = getattr(getattr(getattr(trainer, "model", None), "config", None), "license", None)
        all_tags = _as_list(tags)
        for t in CARD_TAGS + tuple(getattr(getattr(trainer, "model", None), "model_tags", None) or ()):
            if t not in all_tags:
                all_tags.append(t)
        priv = build_privacy_summary(trainer)
        metrics, lines, last_train = {}, [], None
        for entry in getattr(st, "log_history", []) or []:
            if "loss" in entry:
                last_train = entry
            ev = {k[5:]: v for k, v in entry.items() if k.startswith("eval_") and not k.endswith(("_runtime", "_per_second"))}
            if ev:
                metrics = ev
                lines.append({"Training Loss": None if last_train is None else last_train.get("loss"), "Epoch": entry.get("epoch"),
                              "Step": entry.get("step"), **{k.replace("_", " ").title(): v for k, v in ev.items()}})
        hyper = {}
        for k in _HYPERPARAMETERS:
            v = getattr(a, k, None)
            if v is not None and v != {} and not callable(v):
                hyper[k] = v
        hyper["logical_batch_size"] = rt.get("expected_batch", a.per_device_train_batch_size * max(1, getattr(trainer.ddp, "world_size", 1)))
        return cls(model_name=model_name or os.path.basename(os.path.abspath(a.output_dir or "model")), base_model=finetuned_from,
                   dataset=dataset, language=language, license=license, tags=all_tags, tasks=tasks, dataset_tags=dataset_tags,
                   dataset_args=dataset_args, epsilon=priv["epsilon"], delta=priv["delta"], noise_multiplier=priv["noise_multiplier"],
                   clipping_norm=priv["clipping_norm"], clipping_mode=a.clipping_mode, mechanism=a.privacy_noise_mechanism,
                   sampling=getattr(a, "resolved_sampling_mode", a.sampling_mode), sample_rate=rt.get("sample_rate"),
                   steps=st.global_step, expected_batch_size=rt.get("expected_batch"), optimizer=a.optim,
                   learning_rate=a.learning_rate, metrics=metrics, hyperparameters=hyper, eval_lines=lines)

    # ---------------------------------------------------------------------------------------------- rendering
    def privacy_section(self) -> str:
        def fmt(v, spec="g"):
            if v is None:
                return "n/a"
            return format(v, spec) if isinstance(v, (int, float)) and not isinstance(v, bool) else str(v)

        known = self.epsilon is not None and self.epsilon != "unknown"
        rows = [("Guarantee", f"({fmt(self.epsilon, '.4g')}, {fmt(self.delta, '.3g')})-DP" if known else "not accounted"),
                ("Noise mechanism", self.mechanism), ("Noise multiplier", fmt(self.noise_multiplier, ".6g")),
                ("Clipping", f"{self.clipping_mode}, norm {fmt(self.clipping_norm)}"), ("Sampling", self.sampling),
                ("Sampling rate", fmt(self.sample_rate, ".6g")), ("Expected batch size", fmt(self.expected_batch_size)),
                ("Optimizer steps", fmt(self.steps)), ("Optimizer", fmt(self.optimizer)), ("Learning rate", fmt(self.learning_rate))]
        table = "\n".join(f"| {k} | {v} |" for k, v in rows)
        return (f"{DP_BEGIN}\n### Privacy budget\n\nThis model was trained with per-example gradient clipping and calibrated "
                f"noise. The guarantee covers the training examples under add/remove adjacency.\n\n| | |\n|---|---|\n{table}\n{DP_END}")

    def metadata_block(self) -> str:
        meta = ["---", "library_name: opake"]
        for key, val in (("language", self.language), ("license", self.license), ("base_model", self.base_model)):
            vals = _as_list(val)
            if len(vals) == 1:
                meta.append(f"{key}: {vals[0]}")
            elif vals:
                meta += [f"{key}:"] + [f"- {v}" for v in vals]
        meta += ["tags:"] + [f"- {t}" for t in (self.tags or list(CARD_TAGS))]
        ds = _as_list(self.dataset_tags) or _as_list(self.dataset)
        if ds:
            meta += ["datasets:"] + [f"- {d}" for d in ds]
        if self.tasks:
            meta += ["pipeline_tag: " + _as_list(self.tasks)[0]]
        meta.append("---")
        return "\n".join(meta)

    def to_model_card(self) -> str:
        out = [self.metadata_block(), "", f"# {self.model_name}", ""]
        ds = ", ".join(f"`{d}`" for d in _as_list(self.dataset))
        if self.base_model:
            out.append(f"This model is a fine-tuned version of `{self.base_model}`" + (f" on {ds}." if ds else "."))
        elif ds:
            out.append(f"This model was trained on {ds}.")
        if self.metrics:
            out += ["It achieves the following results on the evaluation set:"] + [f"- {k.replace('_', ' ').title()}: {v}" for k, v in self.metrics.items()]
        out += ["", "## Training procedure", ""]
        if self.hyperparameters:
            out += ["### Training hyperparameters", "", "The following hyperparameters were used during training:"]
            out += [f"- {k}: {v}" for k, v in self.hyperparameters.items()] + [""]
        if self.eval_lines:
            cols = list(self.eval_lines[0].keys())
            out += ["### Training results", "", "| " + " | ".join(cols) + " |", "|" + "|".join(":---:" for _ in cols) + "|"]
            for ln in self.eval_lines:
                out.append("| " + " | ".join("No log" if ln.get(c) is None else (f"{ln[c]:.4f}" if isinstance(ln[c], float) else str(ln[c]))
                                             for c in cols) + " |")
            out.append("")
        out += ["### Framework versions", "", f"- opake_b200 {_package_version()}"]
        for mod in ("transformers", "torch", "tokenizers", "datasets"):
            try:
                out.append(f"- {mod} {__import__(mod).__version__}")
            except Exception:
                pass
        return splice_dp_section("\n".join(out) + "\n", self.privacy_section())


def splice_dp_section(card: str, section: str) -> str:
    """Replaces the marked block in place; else inserts it after ``### Framework versions``; else appends it."""
    pattern = re.compile(re.escape(DP_BEGIN) + ".*?" + re.escape(DP_END), re.DOTALL)
    if pattern.search(card):
        return pattern.sub(lambda _m: section, card)
    m = _FRAMEWORK_RE.search(card)
    if m:
        return card[: m.end()].rstrip("\n") + "\n\n" + section + "\n" + card[m.end():]
    return card.rstrip("\n") + "\n\n" + section + "\n"


def create_model_card(source, existing: str | None = None, **kwargs) -> str:
    """``create_model_card(trainer, language=..., license=..., tags=..., model_name=..., finetuned_from=..., tasks=...,
    dataset_tags=..., dataset=..., dataset_args=...)`` writes ``README.md`` into ``args.output_dir`` (process zero only)
    and returns the text. ``create_model_card(summary, existing=None)`` renders a summary; with ``existing`` only the
    privacy section of that card is replaced."""
    if isinstance(source, DPTrainingSummary):
        if existing:
            return splice_dp_section(existing, source.privacy_section())
        return source.to_model_card()
    trainer = source
    summary = DPTrainingSummary.from_trainer(trainer, **kwargs)
    a = trainer.args
    if a.output_dir is None:
        return summary.to_model_card()
    path = os.path.join(a.output_dir, "README.md")
    if os.path.exists(path) and DP_BEGIN in open(path, encoding="utf-8").read():
        card = splice_dp_section(open(path, encoding="utf-8").read(), summary.privacy_section())
    else:
        card = summary.to_model_card()
    if trainer.is_world_process_zero():
        os.makedirs(a.output_dir, exist_ok=True)
        with open(path, "w", encoding="utf-8") as f:
            f.write(card)
    return card


def _hub():
    try:
        import huggingface_hub

        return huggingface_hub
    except Exception as e:
        raise OperationError("push_to_hub needs the huggingface_hub package") from e


def init_hf_repo(trainer_or_repo, token: str | None = None, private: bool | None = None) -> str | None:
    """Creates (or validates) the repository. Given a trainer: named after ``hub_model_id`` or the output directory,
    stored as ``trainer.hub_model_id``; process zero only."""
    if isinstance(trainer_or_repo, str):
        return _hub().create_repo(trainer_or_repo, token=token, private=private, exist_ok=True).repo_id
    trainer = trainer_or_repo
    if not trainer.is_world_process_zero():
        return None
    a = trainer.args
    name = a.hub_model_id or os.path.basename(os.path.abspath(a.output_dir))
    repo_id = _hub().create_repo(name, token=token if token is not None else a.hub_token, private=a.hub_private_repo,
                                 exist_ok=True).repo_id
    trainer.hub_model_id = repo_id
    return repo_id


def push_to_hub(source, repo_id: str | None = None, *, commit_message: str = "End of training", blocking: bool = True,
                token: str | None = None, revision: str | None = None, private: bool | None = None, **card_kwargs):
    """``push_to_hub(trainer, ...)``: saves the model (parameters restored into the module first), writes the card and
    uploads ``args.output_dir`` without checkpoints, underscore-prefixed files and ``runs/``. ``push_to_hub(folder,
    repo_id, ...)`` uploads a folder as it is."""
    hub = _hub()
    if isinstance(source, (str, os.PathLike)):
        if not os.path.isdir(source):
            raise OperationError(f"nothing to push: {source} does not exist")
        init_hf_repo(repo_id, token, private)
        return hub.upload_folder(repo_id=repo_id, folder_path=str(source), token=token, commit_message=commit_message,
                                 revision=revision, run_as_future=not blocking, ignore_patterns=["_*", "checkpoint-*", "runs/**", "*.tmp"])
    trainer = source
    if not trainer.is_world_process_zero():
        return None
    handler = getattr(trainer, "callback_handler", None)
    if handler is not None:
        trainer.control = handler.call_event("on_push_begin", trainer.args, trainer.state, trainer.control)
    a = trainer.args
    tok = token if token is not None else a.hub_token
    if getattr(trainer, "hub_model_id", None) is None:
        init_hf_repo(trainer, token=tok)
    trainer.save_model()
    card_kwargs.setdefault("model_name", trainer.hub_model_id.split("/")[-1])
    create_model_card(trainer, **card_kwargs)
    return hub.upload_folder(repo_id=trainer.hub_model_id, folder_path=a.output_dir, commit_message=commit_message, token=tok,
                             run_as_future=not blocking, revision=revision if revision is not None else a.hub_revision,
                             ignore_patterns=["_*", "checkpoint-*", "runs/**"])
