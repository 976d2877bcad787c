"""DP preference optimisation from the command line (``DPOTrainer``): ``python examples/train_dpo.py --cpu``."""
import argparse

from _common import SyntheticPreferences, add_common, preset, training_kwargs
from opake_b200.models.native import NativeCausalLM
from opake_b200.transformers import DPOConfig, DPOTrainer


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    add_common(p)
    p.add_argument("--beta", type=float, default=0.1)
    p.add_argument("--loss-type", nargs="+", default=["sigmoid"])
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    cfg = preset(a.model)
    kw = training_kwargs(a)
    kw["use_cpu"] = True if a.cpu else kw["use_cpu"]
    args = DPOConfig(beta=a.beta, loss_type=a.loss_type if len(a.loss_type) > 1 else a.loss_type[0], max_length=a.seq_len,
                     native_engine=False, **kw)
    data = SyntheticPreferences(a.dataset_size, cfg.vocab_size, a.seq_len // 4, a.seq_len // 4, a.seed)
    trainer = DPOTrainer(NativeCausalLM(cfg), None, args, train_dataset=data, eval_dataset=SyntheticPreferences(64, cfg.vocab_size, a.seq_len // 4, a.seq_len // 4, 1))
    out = trainer.train()
    print({k: (round(v, 5) if isinstance(v, float) else v) for k, v in out.metrics.items()}, trainer.evaluate())
    return out


if __name__ == "__main__":
    main()
