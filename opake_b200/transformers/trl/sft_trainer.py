"""``SFTTrainer`` / ``SFTConfig`` (packages/opake-transformers/src/opake/api/transformers/trl/_sft_trainer.py:137-730):
supervised fine-tuning with per-example NLL (or DFT) loss, optional completion-only masking, and the fused linear
cross-entropy path that works from the last hidden states instead of materialised logits."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ...alignment.sft.collator import language_modeling_collator
from ...alignment.sft.loss import dft_loss, fused_dft_loss, fused_nll_loss, nll_loss
from ...base.exceptions import ConfigurationError
from ..dp_trainer import DPTrainer
from ..training_arguments import TrainingArguments

__all__ = ["SFTConfig", "SFTTrainer"]


@dataclass
class SFTConfig(TrainingArguments):
    max_length: int = 1024
    completion_only_loss: bool | None = None      # None: on when the dataset carries completion masks
    assistant_only_loss: bool = False
    loss_type: str = "nll"                         # "nll" | "dft"
    dataset_text_field: str = "text"
    pad_to_multiple_of: int | None = None
    pad_token: str | None = None
    use_fused_linear_cross_entropy: bool | None = None   # None: on for CUDA bf16 models that expose hidden states
    packing: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.loss_type not in ("nll", "dft"):
            raise ConfigurationError(f"loss_type must be 'nll' or 'dft', got {self.loss_type!r}")
        if self.packing:
            raise ConfigurationError("packing merges several examples into one sequence, which breaks the per-example "
                                     "privacy unit; it is not supported")

    @classmethod
    def from_trl(cls, trl_config, **dp_overrides):
        """From a TRL ``SFTConfig`` (or a mapping with its field names)."""
        from ..hf_convert import convert_trl_config
        return convert_trl_config(trl_config, cls, **dp_overrides)


class SFTTrainer(DPTrainer):
    def __init__(self, model=None, args: SFTConfig | None = None, data_collator=None, train_dataset=None, eval_dataset=None,
                 processing_class=None, formatting_func=None, **kw):
        args = args if args is not None else SFTConfig()
        self.formatting_func = formatting_func
        if data_collator is None:
            pad_id = self._pad_id(processing_class, args)
            completion_only = bool(args.completion_only_loss) or args.assistant_only_loss
            data_collator = language_modeling_collator(pad_id, args.max_length, completion_only_loss=completion_only,
                                                       pad_to_multiple_of=args.pad_to_multiple_of)
        train_dataset = self._prepare(train_dataset, processing_class, args)
        eval_dataset = self._prepare(eval_dataset, processing_class, args)
        super().__init__(model=model, args=args, data_collator=data_collator, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         processing_class=processing_class, **kw)

    @staticmethod
    def _pad_id(tok, args) -> int:
        if tok is None:
            return 0
        if args.pad_token is not None:
            return tok.convert_tokens_to_ids(args.pad_token)
        pid = getattr(tok, "pad_token_id", None)
        return pid if pid is not None else (getattr(tok, "eos_token_id", 0) or 0)

    def _prepare(self, dataset, tok, args):
        """Tokenizes text / chat datasets lazily; already tokenized datasets (``input_ids``) pass through."""
        if dataset is None or tok is None:
            return dataset
        try:
            first = dataset[0]
        except Exception:
            return dataset
        if isinstance(first, dict) and "input_ids" in first:
            return dataset
        return _Tokenized(dataset, tok, args, self.formatting_func)

    def compute_per_example_loss(self, call, params, inputs):
        a = self.args
        labels = inputs["labels"]
        model_inputs = {k: v for k, v in inputs.items() if k in ("input_ids", "attention_mask", "position_ids")}
        fused = a.use_fused_linear_cross_entropy
        head = self._lm_head(params)
        if fused is None:
            fused = head is not None and labels.is_cuda and head.dtype == torch.bfloat16
        if fused and head is not None:
            out = call(params, **model_inputs, output_hidden_states=True)
            hidden = out.get("last_hidden_state") if isinstance(out, dict) else getattr(out, "hidden_states", [None])[-1]
            if hidden is not None:
                loss = (fused_dft_loss if a.loss_type == "dft" else fused_nll_loss)(hidden, head, labels)
                return loss[0] if loss.dim() else loss
        out = call(params, **model_inputs)
        logits = out["logits"] if isinstance(out, dict) else out.logits
        loss = (dft_loss if a.loss_type == "dft" else nll_loss)(logits, labels)
        return loss[0] if loss.dim() else loss

    def _lm_head(self, params):
        for name in ("lm_head.weight", "model.lm_head.weight"):
            if name in params:
                return params[name]
            if name in self._rt.get("frozen", {}):
                return self._rt["frozen"][name]
        return None


class _Tokenized(torch.utils.data.Dataset):
    def __init__(self, base, tok, args, formatting_func):
        self.base, self.tok, self.args, self.fmt = base, tok, args, formatting_func

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        ex = self.base[i]
        a = self.args
        if self.fmt is not None:
            ex = {a.dataset_text_field: self.fmt(ex)}
        if "messages" in ex:
            if a.assistant_only_loss:
                from ...alignment.data import apply_chat_template_with_mask
                return apply_chat_template_with_mask(self.tok, ex["messages"])
            ids = self.tok.apply_chat_template(ex["messages"], tokenize=True)
            return {"input_ids": list(ids)[: a.max_length]}
        if "prompt" in ex and "completion" in ex:
            p = self.tok(ex["prompt"], add_special_tokens=True)["input_ids"]
            c = self.tok(ex["completion"], add_special_tokens=False)["input_ids"]
            eos = getattr(self.tok, "eos_token_id", None)
            c = c + ([eos] if eos is not None else [])
            return {"input_ids": (p + c)[: a.max_length], "completion_mask": ([0] * len(p) + [1] * len(c))[: a.max_length]}
        ids = self.tok(ex[a.dataset_text_field], add_special_tokens=True)["input_ids"]
        return {"input_ids": list(ids)[: a.max_length]}
