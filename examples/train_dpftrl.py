"""DP-FTRL (matrix-factorisation noise) with ``DPTrainer``: banded / BLT / BISR / BSR / lambda-CGD strategies with their
matching samplers and accounting: ``python examples/train_dpftrl.py --cpu --mechanism mf_band --max-steps 8``."""
import argparse

import torch

from _common import SyntheticLM, add_common, preset, training_kwargs
from opake_b200.alignment.sft import language_modeling_collator
from opake_b200.models.native import NativeCausalLM
from opake_b200.transformers import DPTrainer, TrainingArguments


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    add_common(p)
    p.add_argument("--mechanism", default="mf_band", choices=("mf_identity", "mf_band", "mf_blt", "mf_bisr", "mf_bsr", "mf_lambda_cgd"))
    p.add_argument("--bands", type=int, default=4)
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    cfg = preset(a.model)
    cuda = torch.cuda.is_available() and not a.cpu
    model = NativeCausalLM(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device="cuda" if cuda else None)
    mkw = {"bands": a.bands} if a.mechanism == "mf_band" else {}
    args = TrainingArguments(privacy_noise_mechanism=a.mechanism, privacy_noise_mechanism_kwargs=mkw, **training_kwargs(a))
    trainer = DPTrainer(model, args, data_collator=language_modeling_collator(0, a.seq_len),
                        train_dataset=SyntheticLM(a.dataset_size, cfg.vocab_size, a.seq_len, a.seed))
    out = trainer.train()
    print({k: (round(v, 5) if isinstance(v, float) else v) for k, v in out.metrics.items()})
    return out


if __name__ == "__main__":
    main()
