"""DP supervised fine-tuning from the command line (``SFTTrainer``). Synthetic data by default so that it runs
without network access: ``python examples/train_sft.py --cpu --max-steps 5``. On a CUDA machine the native sm_100a
engine runs the step (``--model llama3.2-1b --batch-size 64``)."""
import argparse

import torch

from _common import SyntheticLM, add_common, preset, training_kwargs
from opake_b200.models.native import NativeCausalLM
from opake_b200.transformers import SFTConfig, SFTTrainer


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    add_common(p)
    p.add_argument("--loss-type", default="nll", choices=("nll", "dft"))
    p.add_argument("--completion-only", action="store_true")
    p.add_argument("--mechanism", default="gaussian", help="gaussian or an mf_* matrix-factorisation mechanism (DP-FTRL)")
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    cfg = preset(a.model)
    cuda = torch.cuda.is_available() and not a.cpu
    model = NativeCausalLM(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device="cuda" if cuda else None)
    args = SFTConfig(max_length=a.seq_len, loss_type=a.loss_type, completion_only_loss=a.completion_only,
                     privacy_noise_mechanism=a.mechanism, **training_kwargs(a))
    trainer = SFTTrainer(model, args, train_dataset=SyntheticLM(a.dataset_size, cfg.vocab_size, a.seq_len, a.seed))
    out = trainer.train()
    print({k: (round(v, 5) if isinstance(v, float) else v) for k, v in out.metrics.items()})
    return out


if __name__ == "__main__":
    main()
