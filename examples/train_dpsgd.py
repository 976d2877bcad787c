"""DP-SGD language-model training with ``DPTrainer`` (Poisson sampling, Gaussian noise, PLD accounting):
``python examples/train_dpsgd.py --cpu --max-steps 5``. ``--fsdp`` under ``torchrun`` shards optimizer state and
gradient sums over the ranks of the native engine."""
import argparse

import torch

from _common import SyntheticLM, add_common, preset, training_kwargs
from opake_b200.alignment.sft import language_modeling_collator
from opake_b200.models.native import NativeCausalLM
from opake_b200.transformers import DPTrainer, TrainingArguments


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    add_common(p)
    p.add_argument("--fsdp", action="store_true")
    p.add_argument("--sampling", default="auto", choices=("auto", "poisson", "k_out_of_t"))
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    cfg = preset(a.model)
    cuda = torch.cuda.is_available() and not a.cpu
    model = NativeCausalLM(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device="cuda" if cuda else None)
    args = TrainingArguments(fsdp=a.fsdp, sampling_mode=a.sampling, **training_kwargs(a))
    trainer = DPTrainer(model, args, data_collator=language_modeling_collator(0, a.seq_len),
                        train_dataset=SyntheticLM(a.dataset_size, cfg.vocab_size, a.seq_len, a.seed))
    out = trainer.train()
    print({k: (round(v, 5) if isinstance(v, float) else v) for k, v in out.metrics.items()})
    return out


if __name__ == "__main__":
    main()
