"""``DPOTrainer`` / ``DPOConfig`` (packages/opake-transformers/src/opake/api/transformers/trl/_dpo_trainer.py:275-903):
differentially private preference optimisation. One example = one (prompt, chosen, rejected) triple; the per-example
loss combines the policy's sequence log-probabilities with reference log-probabilities that are precomputed once
(the reference never sees gradients, so its outputs are public functions of each example alone). TR-DPO style
reference updates (EMA or hard sync every ``ref_model_sync_steps``) are supported for a separate reference copy."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

import torch

from ...alignment.dpo import loss as L
from ...alignment.dpo.collator import preference_collator
from ...alignment.dpo.metric import reward_metrics
from ...alignment.dpo.reference import ema_update_reference, null_ref_context
from ...alignment.logprob import sequence_logp
from ...base.exceptions import ConfigurationError
from ..dp_trainer import DPTrainer
from ..training_arguments import TrainingArguments

__all__ = ["DPOConfig", "DPOTrainer"]

_REFERENCE_FREE = ("simpo", "orpo")
_LENGTH_NORMALISED = ("simpo", "orpo", "ipo")


@dataclass
class DPOConfig(TrainingArguments):
    beta: float = 0.1
    loss_type: str | list = "sigmoid"
    loss_weights: list | None = None
    label_smoothing: float = 0.0
    max_length: int = 1024
    pad_to_multiple_of: int | None = None
    reference_free: bool = False
    precompute_ref_log_probs: bool = True
    precompute_ref_batch_size: int | None = None
    ref_cache_dir: str | None = None
    use_ref_cache: bool = False
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.6
    ref_model_sync_steps: int = 512
    f_divergence_type: str = "reverse_kl"
    f_alpha_divergence_coef: float = 1.0
    simpo_gamma: float = 0.5
    discopop_tau: float = 0.05
    ld_alpha: float | None = None
    use_weighting: bool = False
    rpo_alpha: float | None = None
    loss_kwargs: dict = field(default_factory=dict)

    def __post_init__(self):
        super().__post_init__()
        names = [self.loss_type] if isinstance(self.loss_type, str) else list(self.loss_type)
        for n in names:
            if n not in L.LOSS_HEADS:
                raise ConfigurationError(f"unknown DPO loss_type {n!r}; known: {sorted(L.LOSS_HEADS)}")
        if self.loss_weights is not None and len(self.loss_weights) != len(names):
            raise ConfigurationError("loss_weights needs one weight per loss_type")
        if self.sync_ref_model and self.precompute_ref_log_probs:
            raise ConfigurationError("sync_ref_model changes the reference during training; set precompute_ref_log_probs=False")

    @classmethod
    def from_trl(cls, trl_config, **dp_overrides):
        """From a TRL ``DPOConfig`` (or a mapping with its field names)."""
        from ..hf_convert import convert_trl_config
        return convert_trl_config(trl_config, cls, **dp_overrides)


class DPOTrainer(DPTrainer):
    def __init__(self, model=None, ref_model=None, args: DPOConfig | None = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, processing_class=None, **kw):
        args = args if args is not None else DPOConfig()
        if ref_model is model and model is not None:
            raise ConfigurationError("ref_model must be a separate model (or None to use a frozen copy of the policy)")
        if data_collator is None:
            pad = getattr(processing_class, "pad_token_id", None) if processing_class is not None else None
            data_collator = preference_collator(pad if pad is not None else 0, args.max_length, pad_to_multiple_of=args.pad_to_multiple_of)
        self._names = [args.loss_type] if isinstance(args.loss_type, str) else list(args.loss_type)
        self._needs_ref = not args.reference_free and any(n not in _REFERENCE_FREE for n in self._names)
        self.ref_model = ref_model
        if self._needs_ref and ref_model is None and not _has_adapters(model):
            self.ref_model = copy.deepcopy(model)
        if self.ref_model is not None:
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
            self.ref_model.eval()
        super().__init__(model=model, args=args, data_collator=data_collator, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         processing_class=processing_class, **kw)
        if self._needs_ref and args.precompute_ref_log_probs:
            self.train_dataset = self._with_reference(self.train_dataset)
            if self.eval_dataset is not None:
                self.eval_dataset = self._with_reference(self.eval_dataset)

    # ------------------------------------------------------------------ reference log-probabilities
    def _policy_logps(self, forward, batch, normalized: bool):
        out = {}
        for side in ("chosen", "rejected"):
            ids, cm = batch[f"{side}_input_ids"], batch[f"{side}_completion_mask"]
            res = forward(input_ids=ids, attention_mask=batch[f"{side}_attention_mask"])
            logits = res["logits"] if isinstance(res, dict) else res.logits
            out[side] = sequence_logp(logits, ids, cm, length_normalized=normalized, ld_alpha=None)
        return out["chosen"], out["rejected"]

    def _reference_forward(self, batch):
        batch = {k: v.to(self.device) if isinstance(v, torch.Tensor) else v for k, v in batch.items()}
        ref = self.ref_model if self.ref_model is not None else self.model
        ref.to(self.device)
        with torch.no_grad(), null_ref_context(self.model, self.ref_model):
            c, r = self._policy_logps(lambda **kw: ref(**kw), batch, normalized=False)
        return {"ref_chosen_logps": c.float().cpu(), "ref_rejected_logps": r.float().cpu()}

    def _with_reference(self, dataset):
        a = self.args
        if hasattr(dataset, "add_column") and a.use_ref_cache:
            from ...alignment.dpo.reference import compute_ref_logprobs_for_dataset
            return compute_ref_logprobs_for_dataset(dataset, self._reference_forward, self.data_collator,
                                                    ("ref_chosen_logps", "ref_rejected_logps"),
                                                    cache_identity={"beta": a.beta, "max_length": a.max_length},
                                                    batch_size=a.precompute_ref_batch_size or a.per_device_eval_batch_size,
                                                    cache_dir=a.ref_cache_dir, use_cache=True)
        from torch.utils.data import DataLoader
        cols: dict[str, list] = {"ref_chosen_logps": [], "ref_rejected_logps": []}
        for batch in DataLoader(dataset, batch_size=a.precompute_ref_batch_size or a.per_device_eval_batch_size,
                                collate_fn=self.data_collator):
            out = self._reference_forward(batch)
            for k in cols:
                cols[k].extend(out[k].tolist())
        return _WithColumns(dataset, cols)

    # ------------------------------------------------------------------ loss
    def dpo_loss(self, pc, pr, rc, rr):
        """Per-example loss from policy (``pc``, ``pr``) and reference (``rc``, ``rr``) sequence log-probabilities."""
        a = self.args
        losses = {}
        for name in self._names:
            head = L.LOSS_HEADS[name]
            if name == "orpo":
                losses[name] = head(pc, pr)
                continue
            if name in ("sft", "chosen_nll"):
                losses[name] = head(pc)
                continue
            c_lr, r_lr = (pc, pr) if (name in _REFERENCE_FREE or a.reference_free) else (pc - rc, pr - rr)
            if a.f_divergence_type != "reverse_kl" and name == "sigmoid":
                z = L.f_divergence_logits(c_lr, r_lr, f_divergence_type=a.f_divergence_type, alpha=a.f_alpha_divergence_coef)
                losses[name] = L.sigmoid_loss(z, torch.zeros_like(z), beta=a.beta, label_smoothing=a.label_smoothing)
                continue
            kw = dict(a.loss_kwargs)
            if name in ("sigmoid", "robust", "simpo", "exo", "exo_pair"):
                kw.setdefault("label_smoothing", a.label_smoothing if name != "exo" and name != "exo_pair" else max(a.label_smoothing, 1e-3))
            if name == "simpo":
                kw.setdefault("gamma", a.simpo_gamma)
            if name == "discopop":
                kw.setdefault("discopop_tau", a.discopop_tau)
            losses[name] = head(c_lr, r_lr, beta=a.beta, **kw)
        if len(losses) == 1 and a.rpo_alpha is None:
            return next(iter(losses.values()))
        weights = dict(zip(self._names, a.loss_weights or [1.0] * len(self._names)))
        if a.rpo_alpha is not None:
            losses["rpo_nll"], weights["rpo_nll"] = L.chosen_nll_loss(pc), a.rpo_alpha
        return L.mpo_combine(losses, weights)

    def compute_per_example_loss_and_metrics(self, call, params, inputs):
        """Loss of one preference pair plus its reward telemetry (``rewards/chosen``, ``rewards/rejected``,
        ``rewards/accuracies``, ``rewards/margins``), logged as batch means during training. These are statistics of
        the training data that no mechanism protects: log them for diagnosis, do not publish them."""
        a = self.args
        normalized = any(n in _LENGTH_NORMALISED for n in self._names)
        pc, pr = self._policy_logps(lambda **kw: call(params, **kw), inputs, normalized)
        rc = inputs.get("ref_chosen_logps")
        rr = inputs.get("ref_rejected_logps")
        if self._needs_ref and rc is None:
            with torch.no_grad():
                ref = self.ref_model
                rc, rr = self._policy_logps(lambda **kw: ref(**kw), inputs, normalized)
        if rc is None:
            rc, rr = torch.zeros_like(pc), torch.zeros_like(pr)
        loss = self.dpo_loss(pc, pr, rc.to(pc.dtype), rr.to(pr.dtype))
        lc, lr_ = (pc - rc).detach().reshape(-1)[0], (pr - rr).detach().reshape(-1)[0]
        tele = {"rewards/chosen": a.beta * lc, "rewards/rejected": a.beta * lr_, "rewards/accuracies": (lc > lr_).to(lc.dtype),
                "rewards/margins": a.beta * (lc - lr_)}
        return (loss[0] if loss.dim() else loss), tele

    def compute_per_example_loss(self, call, params, inputs):
        return self.compute_per_example_loss_and_metrics(call, params, inputs)[0]

    def prediction_step(self, inputs, prediction_loss_only=None):
        with torch.no_grad():
            params = self._rt.get("params")
            call = (lambda p, **kw: self._call_model(p, kw)) if params is not None else (lambda p, **kw: self.model(**kw))
            normalized = any(n in _LENGTH_NORMALISED for n in self._names)
            pc, pr = self._policy_logps(lambda **kw: call(params, **kw), inputs, normalized)
            rc, rr = inputs.get("ref_chosen_logps"), inputs.get("ref_rejected_logps")
            if rc is None:
                if self._needs_ref and self.ref_model is not None:
                    rc, rr = self._policy_logps(lambda **kw: self.ref_model(**kw), inputs, normalized)
                else:
                    rc, rr = torch.zeros_like(pc), torch.zeros_like(pr)
            losses = self.dpo_loss(pc, pr, rc.to(pc.dtype), rr.to(pr.dtype))
            self._last_rewards = reward_metrics(pc - rc, pr - rr, beta=self.args.beta)
        return losses, None, None

    def training_step(self, batch):
        out = super().training_step(batch)
        a = self.args
        if a.sync_ref_model and self.ref_model is not None and (self.state.global_step + 1) % a.ref_model_sync_steps == 0:
            self._publish_params()
            new = ema_update_reference(dict(self.ref_model.named_parameters()), dict(self.model.named_parameters()), a.ref_model_mixup_alpha)
            with torch.no_grad():
                for k, p in self.ref_model.named_parameters():
                    p.copy_(new[k])
        return out


def _has_adapters(model) -> bool:
    return hasattr(model, "peft_config") or hasattr(model, "disable_adapter")


class _WithColumns(torch.utils.data.Dataset):
    """A dataset view with extra per-row columns (for datasets without ``add_column``)."""

    def __init__(self, base, columns: dict):
        self.base, self.columns = base, columns

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        ex = dict(self.base[i])
        for k, v in self.columns.items():
            ex[k] = v[i]
        return ex
