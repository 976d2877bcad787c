"""The command line: presets fill defaults and explicit flags win; every training command runs a few steps on the CPU;
the accounting command reproduces the accountant."""
import json

import pytest

from opake_b200 import cli


def _args(argv):
    return cli.resolve(cli.build_parser().parse_args(argv))


def test_presets_and_overrides():
    a = _args(["dpsgd", "--preset", "llama8b-dpsgd-fsdp"])
    assert (a.model_name, a.batch_size, a.max_seq_len, a.noise_multiplier, a.shard) == ("llama3-8b", 256, 2048, 0.9, "full")
    a = _args(["dpsgd", "--preset", "llama8b-dpsgd-fsdp", "--batch-size", "64", "--shard", "state"])
    assert a.batch_size == 64 and a.shard == "state" and a.model_name == "llama3-8b"
    a = _args(["dpftrl", "--preset", "llama1b-dpftrl-blt"])
    assert a.mechanism == "mf_blt" and a.max_buffers == 4
    a = _args(["dpsgd"])
    assert a.target_epsilon == 8.0 and a.noise_multiplier is None      # a privacy target is always set
    a = _args(["dpsgd", "--microbatch-size", "0"])
    assert a.microbatch_size is None


def test_training_arguments_mapping():
    from opake_b200.transformers import TrainingArguments
    a = _args(["dpsgd", "--preset", "smoke", "--cpu", "--clipping-mode", "adaptive", "--target-clipping-rate", "0.7", "--sampler",
               "k_out_of_t", "--k", "2", "--allocation", "block", "--noise-multiplier", "1.2", "--lr-warmup-steps", "3"])
    t = cli.training_arguments(a, TrainingArguments)
    assert t.clipping_mode == "adaptive" and t.clipping_kwargs["target_quantile"] == 0.7
    assert t.sampling_mode == "k_out_of_t" and t.sampling_kwargs == {"k": 2, "allocation": "block"}
    assert t.privacy_noise_multiplier == 1.2 and t.max_steps == 16 and t.warmup_steps == 3


@pytest.mark.parametrize("command,extra", [("dpsgd", []), ("dpftrl", ["--mechanism", "mf_band", "--bands", "2"]), ("sft", []),
                                           ("dpo", ["--loss-type", "ipo"])])
def test_training_commands_run_on_cpu(tmp_path, command, extra, capsys):
    out = cli.main([command, "--preset", "smoke", "--cpu", "--stop-at-step", "2", "--output-dir", str(tmp_path), *extra])
    assert out["train_loss"] > 0 and 0 < out["privacy_epsilon"] <= 8.0 + 1e-6


def test_account_command(capsys):
    out = cli.main(["account", "--dataset-size", "60000", "--batch-size", "256", "--steps", "200", "--noise-multiplier", "1.1",
                    "--target-delta", "1e-5"])
    assert out["epsilon"] == pytest.approx(0.28687, abs=2e-4)
    cal = cli.main(["account", "--dataset-size", "60000", "--batch-size", "256", "--steps", "200", "--target-epsilon", "1.0",
                    "--target-delta", "1e-5"])
    assert cal["epsilon"] <= 1.0 and cal["epsilon"] > 0.98
    fams = cli.main(["families"])
    assert fams["llama"]["native"] and fams["gemma2"]["softcap"] == 50.0
    json.dumps(fams)
