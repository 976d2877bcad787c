"""DPTrainer / SFTTrainer / DPOTrainer, TrainingArguments, checkpoints and patches on CPU."""
import os

import pytest
import torch
from torch import nn


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1, self.l2 = nn.Linear(8, 16), nn.Linear(16, 3)

    def forward(self, x, labels=None):
        return {"logits": self.l2(torch.tanh(self.l1(x)))}


class _DS(torch.utils.data.Dataset):
    def __init__(self, n, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(n, 8, generator=g)
        self.y = (self.x[:, 0] > 0).long() + (self.x[:, 1] > 0).long()

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return {"x": self.x[i], "labels": self.y[i]}


def _args(out, **kw):
    from opake_b200.transformers import TrainingArguments
    base = dict(output_dir=str(out), per_device_train_batch_size=32, max_steps=8, learning_rate=0.05, optim="adamw-bc",
                privacy_target_epsilon=6.0, logging_steps=4, save_steps=4, eval_strategy="steps", eval_steps=4, use_cpu=True,
                lr_scheduler="cosine", warmup_steps=2, save_total_limit=2, use_compat_patches=False)
    base.update(kw)
    return TrainingArguments(**base)


def test_training_arguments_validation_and_hf_conversion():
    from opake_b200.base.exceptions import ConfigurationError
    from opake_b200.transformers import TrainingArguments
    a = TrainingArguments(privacy_noise_mechanism="mf_band")
    assert a.resolved_sampling_mode == "cyclic_poisson" and a.resolved_mechanism_kwargs == {"bands": 16} and a.is_dpftrl
    assert TrainingArguments().target_delta(10_000) == pytest.approx(10_000 ** -1.1)
    with pytest.raises(ConfigurationError):
        TrainingArguments(privacy_noise_mechanism="mf_blt", sampling_mode="poisson")
    both = TrainingArguments(privacy_target_epsilon=1.0, privacy_noise_multiplier=1.0)      # stop-at-epsilon mode
    assert both.privacy_target_epsilon == 1.0 and both.privacy_noise_multiplier == 1.0
    with pytest.raises(ConfigurationError):
        TrainingArguments(torch_compile=True)
    b = TrainingArguments.from_hf({"per_device_train_batch_size": 4, "gradient_accumulation_steps": 8, "max_grad_norm": 0.5,
                                   "optim": "adamw_torch_fused", "lr_scheduler_type": "cosine", "warmup_ratio": 0.1},
                                  privacy_target_epsilon=8.0)
    assert (b.per_device_train_batch_size, b.microbatch_size, b.clipping_norm, b.optim, b.lr_scheduler) == (32, 4, 0.5, "adamw", "cosine")
    with pytest.raises(ConfigurationError):
        TrainingArguments.from_hf({"deepspeed": "ds.json"})
    assert TrainingArguments.from_dict(b.to_dict()).to_dict() == b.to_dict()


def test_dp_trainer_trains_checkpoints_and_resumes_bit_exactly(tmp_path):
    from opake_b200.transformers import DPTrainer
    from opake_b200.transformers.checkpoint import load_runtime
    torch.manual_seed(0)
    tr = DPTrainer(_Net(), _args(tmp_path), train_dataset=_DS(600), eval_dataset=_DS(100, 1))
    out = tr.train()
    assert out.global_step == 8 and out.metrics["privacy_epsilon"] == pytest.approx(6.0, abs=1e-3)
    names = sorted(os.listdir(tmp_path))
    assert names == ["checkpoint-4", "checkpoint-8"]
    files = set(os.listdir(tmp_path / "checkpoint-8"))
    assert {"accountant.json", "dp_optimizer.pt", "dp_state.pt", "rng_state.pth", "trainer_state.json", "training_args.bin"} <= files
    rt = load_runtime(str(tmp_path / "checkpoint-8" / "dp_state.pt"))
    assert rt.version == 8 and rt.mechanism_kind == "gaussian" and rt.total_steps == 8 and rt.sampler_state
    final = {k: v.clone() for k, v in tr.model.state_dict().items()}
    torch.manual_seed(0)
    tr2 = DPTrainer(_Net(), _args(tmp_path), train_dataset=_DS(600), eval_dataset=_DS(100, 1))
    out2 = tr2.train(resume_from_checkpoint=str(tmp_path / "checkpoint-4"))
    assert out2.global_step == 8
    for k, v in tr2.model.state_dict().items():
        assert torch.equal(v, final[k]), k           # sampler replay + noise counter + optimizer state all restored
    assert tr2.privacy_spent() == pytest.approx(tr.privacy_spent(), rel=1e-9)
    pred = tr.predict(_DS(40, 2))
    assert pred.predictions.shape == (40, 3) and "test_loss" in pred.metrics


def test_resume_refuses_privacy_relevant_drift_for_horizon_runs(tmp_path):
    from opake_b200.base.exceptions import CheckpointError
    from opake_b200.transformers import DPTrainer
    kw = dict(privacy_noise_mechanism="mf_band", privacy_noise_mechanism_kwargs={"bands": 2}, privacy_target_epsilon=None,
              privacy_noise_multiplier=1.0, eval_strategy="no", per_device_train_batch_size=16)
    tr = DPTrainer(_Net(), _args(tmp_path, **kw), train_dataset=_DS(400))
    tr.train()
    kw2 = dict(kw, privacy_noise_multiplier=2.0)
    tr2 = DPTrainer(_Net(), _args(tmp_path, **kw2), train_dataset=_DS(400))
    with pytest.raises(CheckpointError):
        tr2.train(resume_from_checkpoint=str(tmp_path / "checkpoint-4"))


def test_callbacks_and_early_stop(tmp_path):
    from opake_b200.transformers import DPTrainer, TrainerCallback
    seen = []

    class Stop(TrainerCallback):
        def on_step_end(self, args, state, control, **kw):
            seen.append(state.global_step)
            if state.global_step == 3:
                control.should_training_stop = True
            return control

    tr = DPTrainer(_Net(), _args(tmp_path, save_strategy="no", eval_strategy="no"), train_dataset=_DS(300), callbacks=[Stop()])
    assert tr.train().global_step == 3 and seen == [1, 2, 3]


def test_sft_and_dpo_trainers_on_native_model(tmp_path):
    from opake_b200.models.config import tiny_llama
    from opake_b200.models.native import NativeCausalLM
    from opake_b200.transformers import DPOConfig, DPOTrainer, SFTConfig, SFTTrainer
    cfg = tiny_llama(n_layers=1, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128, vocab_size=128)

    class LM(torch.utils.data.Dataset):
        def __len__(self):
            return 64

        def __getitem__(self, i):
            g = torch.Generator().manual_seed(i)
            n = int(torch.randint(6, 14, (1,), generator=g))
            return {"input_ids": torch.randint(0, 128, (n,), generator=g).tolist(), "completion_mask": [0] * 3 + [1] * (n - 3)}

    common = dict(output_dir=str(tmp_path), per_device_train_batch_size=8, max_steps=2, privacy_noise_multiplier=1.0, use_cpu=True,
                  save_strategy="no", max_length=16, use_compat_patches=False, logging_steps=1)
    m = NativeCausalLM(cfg)
    before = m.flat.detach().clone()
    out = SFTTrainer(m, SFTConfig(completion_only_loss=True, **common), train_dataset=LM()).train()
    assert out.global_step == 2 and not torch.equal(m.flat.detach(), before) and out.metrics["privacy_epsilon"] > 0

    class Pref(torch.utils.data.Dataset):
        def __len__(self):
            return 48

        def __getitem__(self, i):
            g = torch.Generator().manual_seed(i)
            p, c, r = (torch.randint(0, 128, (k,), generator=g).tolist() for k in (4, 3, 5))
            return {"chosen_input_ids": p + c, "rejected_input_ids": p + r, "chosen_completion_mask": [0] * 4 + [1] * 3,
                    "rejected_completion_mask": [0] * 4 + [1] * 5}

    t = DPOTrainer(NativeCausalLM(cfg), None, DPOConfig(loss_type=["sigmoid", "sft"], loss_weights=[1.0, 0.1], **common),
                   train_dataset=Pref(), eval_dataset=Pref())
    assert "ref_chosen_logps" in t.train_dataset[0]
    assert t.train().global_step == 2 and "eval_loss" in t.evaluate()
    # per-example reward telemetry rides the clipping transform's aux channel into the training logs
    train_logs = [e for e in t.state.log_history if "rewards/margins" in e and "loss" in e]
    assert len(train_logs) == 2 and all(0.0 <= e["rewards/accuracies"] <= 1.0 for e in train_logs)
    assert all(e["rewards/margins"] == pytest.approx(e["rewards/chosen"] - e["rewards/rejected"], abs=1e-5) for e in train_logs)


def test_hf_weight_mapping_and_patches_roundtrip():
    transformers = pytest.importorskip("transformers")
    from opake_b200 import patches
    from opake_b200.models.native import NativeCausalLM
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(vocab_size=96, hidden_size=32, intermediate_size=64,
                                                                 num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                                                 max_position_embeddings=32)).eval()
    ids = torch.randint(0, 96, (2, 11))
    with torch.no_grad():
        want = hf(ids).logits
    native = NativeCausalLM.from_hf(hf)
    with torch.no_grad():
        assert (native(ids)["logits"] - want).abs().max() < 1e-5
    hf2 = transformers.LlamaForCausalLM(hf.config)
    hf2.load_state_dict(native.to_hf_state_dict(), strict=False)
    with torch.no_grad():
        assert (hf2(ids).logits - want).abs().max() < 1e-5
    rep = patches.apply_model_patches(hf)
    assert rep["family"] == "llama" and rep["norms"] == 5 and rep["mlps"] == 2 and patches.is_runtime_patched()
    with torch.no_grad():
        assert (hf(ids).logits - want).abs().max() < 1e-5
    assert len(patches.FAMILIES) >= 27 and patches.FAMILIES["olmoe"].moe


def test_lora_functions_vmap_and_ghost_norms():
    from opake_b200.patches.kernels.lora import lora_grad_sq_norms, lora_linear
    from opake_b200.patches.peft import apply_peft_model_patches, inject_lora
    torch.manual_seed(0)
    W, A, B = torch.randn(20, 16), torch.randn(4, 16), torch.randn(20, 4)
    xb = torch.randn(5, 7, 16)
    loss = lambda A, B, x: lora_linear(x, W, A, B, 0.5).pow(2).sum()
    ref = lambda A, B, x: (x @ W.t() + 0.5 * (x @ A.t()) @ B.t()).pow(2).sum()
    gA, gB = torch.func.vmap(torch.func.grad(loss, argnums=(0, 1)), in_dims=(None, None, 0))(A, B, xb)
    rA, rB = torch.func.vmap(torch.func.grad(ref, argnums=(0, 1)), in_dims=(None, None, 0))(A, B, xb)
    assert torch.allclose(gA, rA, atol=1e-4) and torch.allclose(gB, rB, atol=1e-4)
    dy = 2 * (xb @ W.t() + 0.5 * (xb @ A.t()) @ B.t())
    na, nb = lora_grad_sq_norms(xb, dy, A, B, 0.5)
    assert torch.allclose(na, rA.pow(2).sum((1, 2)), rtol=1e-4) and torch.allclose(nb, rB.pow(2).sum((1, 2)), rtol=1e-4)
    net = nn.Sequential()
    net.q_proj, net.other = nn.Linear(16, 16), nn.Linear(16, 16)
    assert inject_lora(net, ("q_proj",)) == 1 and apply_peft_model_patches(net) == 1
    assert [n for n, p in net.named_parameters() if p.requires_grad] == ["q_proj.lora_A.default.weight", "q_proj.lora_B.default.weight"]


def test_moe_routes_agree_and_checkpoint_segment():
    from opake_b200.patches.kernels.moe import dense_moe, grouped_moe, moe_dispatch_plan
    from opake_b200.patches.torch_checkpoint import checkpoint_under_vmap
    torch.manual_seed(0)
    T, d, I, E, k = 37, 16, 24, 6, 2
    x, gu, dn = torch.randn(T, d), torch.randn(E, 2 * I, d) * 0.2, torch.randn(E, d, I) * 0.2
    w, idx = torch.topk(torch.randn(T, E).softmax(-1), k)
    assert torch.allclose(dense_moe(x, gu, dn, idx, w), grouped_moe(x, gu, dn, idx, w), atol=1e-5)
    assert moe_dispatch_plan(4096, 2048, 1024, 64, 8) == "grouped"
    wt = torch.randn(3)
    seg = lambda w_, x_: torch.tanh(x_ * w_).sum()
    f = lambda w_, x_: checkpoint_under_vmap(seg, w_, x_)
    g1 = torch.func.vmap(torch.func.grad(f), in_dims=(None, 0))(wt, torch.ones(4, 3))
    g2 = torch.func.vmap(torch.func.grad(seg), in_dims=(None, 0))(wt, torch.ones(4, 3))
    assert torch.allclose(g1, g2)


def test_oom_step_down_halves_microbatch_and_retries(tmp_path):
    """A simulated out-of-memory error in the gradient computation halves the micro-batch and training restarts."""
    from opake_b200.transformers import DPTrainer

    class Flaky(DPTrainer):
        calls = 0

        def training_step(self, batch):
            if (self._microbatch or 10**9) > 4:
                Flaky.calls += 1
                raise RuntimeError("CUDA out of memory. Tried to allocate 1.00 GiB (simulated)")
            return super().training_step(batch)

    args = _args(tmp_path, save_strategy="no", eval_strategy="no", max_steps=3, microbatch_size=16, auto_find_microbatch_size=True)
    tr = Flaky(_Net(), args, train_dataset=_DS(300))
    with pytest.warns(UserWarning, match="out of memory"):
        out = tr.train()
    assert out.global_step == 3 and tr._microbatch == 4 and Flaky.calls == 2
    # without auto_find_microbatch_size the error propagates
    Flaky.calls = 0
    tr2 = Flaky(_Net(), _args(tmp_path, save_strategy="no", eval_strategy="no", microbatch_size=16), train_dataset=_DS(300))
    with pytest.raises(RuntimeError, match="out of memory"):
        tr2.train()


def test_sigterm_triggers_checkpoint_and_clean_stop(tmp_path):
    import signal

    from opake_b200.transformers import DPTrainer, TrainerCallback

    class Preempt(TrainerCallback):
        def on_step_end(self, args, state, control, **kw):
            if state.global_step == 2:
                os.kill(os.getpid(), signal.SIGTERM)

    args = _args(tmp_path, save_strategy="no", eval_strategy="no", max_steps=8, enable_jit_checkpoint=True)
    tr = DPTrainer(_Net(), args, train_dataset=_DS(300), callbacks=[Preempt()])
    out = tr.train()
    assert out.global_step == 2 and (tmp_path / "checkpoint-2" / "dp_state.pt").exists()
    tr.save_metrics("train", out.metrics)
    tr.save_state()
    assert (tmp_path / "train_results.json").exists() and (tmp_path / "trainer_state.json").exists()


def test_accountant_engine_under_address_and_ub_sanitizers(tmp_path):
    """Builds the stand-alone exercise of the C++ privacy-loss-distribution engine with ASAN + UBSAN and runs it."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "accounting")
    exe = str(tmp_path / "acc_selftest")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer",
                            "-pthread", os.path.join(root, "selftest.cpp"), "-o", exe], capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "all checks passed" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]


def test_hf_and_trl_argument_conversion_report_and_rejections():
    """Hugging Face / TRL argument objects convert with the DP rules: accumulation collapses into the logical batch,
    ``max_grad_norm`` becomes the per-example clipping norm, optimizer spellings collapse, old field names are
    renamed, and settings that would silently change what is trained are refused."""
    import warnings

    from opake_b200.base.exceptions import ConfigurationError
    from opake_b200.transformers import SFTConfig, TrainingArguments
    from opake_b200.transformers.hf_convert import convert_hf_training_arguments

    src = dict(output_dir="o", per_device_train_batch_size=4, gradient_accumulation_steps=8, optim="adamw_torch_fused",
               lr_scheduler_type="cosine", warmup_ratio=0.1, max_grad_norm=0.7, learning_rate=2e-4, torch_compile=True,
               gradient_checkpointing=True, gradient_checkpointing_kwargs={"use_reentrant": True}, group_by_length=True)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        args, report = convert_hf_training_arguments(src, TrainingArguments, return_report=True, privacy_noise_multiplier=1.0)
    assert args.per_device_train_batch_size == 32 and args.microbatch_size == 4
    assert args.optim == "adamw" and args.lr_scheduler == "cosine" and args.warmup_steps == 0.1
    assert args.clipping_norm == 0.7 and args.gradient_checkpointing and args.gradient_checkpointing_kwargs == {}
    assert not args.torch_compile and "torch_compile" in report.dropped and "group_by_length" in report.dropped
    assert report.renamed["max_grad_norm"].startswith("clipping_norm") and "gradient_accumulation_steps" in report.renamed
    assert any("group_by_length" in str(x.message) for x in w)
    sft = SFTConfig.from_trl(dict(output_dir="o", max_seq_length=256, per_device_train_batch_size=2), privacy_noise_multiplier=1.0)
    assert sft.max_length == 256
    for bad in ({"deepspeed": "ds.json"}, {"packing": True}, {"padding_free": True}):
        with pytest.raises(ConfigurationError):
            convert_hf_training_arguments({"output_dir": "o", **bad}, SFTConfig)


def test_lr_schedule_factory_matches_hugging_face_formulas_and_validates():
    """Every scheduler name against the closed-form Hugging Face lambda, kwargs validation, recipe path."""
    import math

    from opake_b200.base.exceptions import ConfigurationError
    from opake_b200.engine.scheduling import cosine_schedule
    from opake_b200.transformers.scheduler import SUPPORTED_SCHEDULERS, build_lr_schedule, get_warmup_steps

    lr, total, W = 2e-3, 50, 7
    mk = lambda name, **kw: build_lr_schedule(name, learning_rate=lr, total_steps=total, warmup_steps=W, kwargs=kw)  # noqa: E731
    prog = lambda s: (s - W) / (total - W)  # noqa: E731
    hf = {
        "linear": lambda s: s / W if s < W else max(0.0, (total - s) / (total - W)),
        "cosine": lambda s: s / W if s < W else max(0.0, 0.5 * (1 + math.cos(math.pi * prog(s)))),
        "constant_with_warmup": lambda s: s / W if s < W else 1.0,
        "constant": lambda s: 1.0,
        "cosine_with_restarts": lambda s: s / W if s < W else (0.0 if prog(s) >= 1 else 0.5 * (1 + math.cos(math.pi * ((3 * prog(s)) % 1.0)))),
        "inverse_sqrt": lambda s: s / W if s < W else 1.0 / math.sqrt((s - W) / W + 1.0),
    }
    kws = {"cosine_with_restarts": {"num_cycles": 3}}
    for name, f in hf.items():
        sch = mk(name, **kws.get(name, {}))
        for s in range(total + 1):          # past the end the upstream cosine lambda oscillates on; ours holds
            assert sch(s) == pytest.approx(lr * f(s), rel=1e-9, abs=1e-15), (name, s)
    # polynomial: (lr - end) * (1 - p)^power + end
    sch = mk("polynomial", lr_end=1e-5, power=2.0)
    for s in range(W, total + 1):
        assert sch(s) == pytest.approx((lr - 1e-5) * (1 - prog(s)) ** 2 + 1e-5, rel=1e-9)
    with pytest.raises(ConfigurationError, match="smaller than initial lr"):
        mk("polynomial", lr_end=1.0)
    # cosine with a floor, given either way but not both, and required
    a, b = mk("cosine_with_min_lr", min_lr=2e-4), mk("cosine_with_min_lr", min_lr_rate=0.1)
    for s in range(total + 1):
        assert a(s) == pytest.approx(b(s), rel=1e-12)
    assert a(total) == pytest.approx(2e-4) and a(W) == pytest.approx(lr)
    with pytest.raises(ConfigurationError, match="only one"):
        mk("cosine_with_min_lr", min_lr=1e-4, min_lr_rate=0.1)
    with pytest.raises(ConfigurationError, match="exactly one"):
        mk("cosine_with_min_lr")
    c = mk("cosine_warmup_with_min_lr", min_lr_rate=0.1, warmup_lr_rate=0.25)
    assert c(0) == pytest.approx(0.25 * lr) and c(W) == pytest.approx(lr) and c(total) == pytest.approx(0.1 * lr)
    assert all(c(s) < c(s + 1) for s in range(W))
    # warmup-stable-decay: floor on both ends, stable plateau, decay shape, held at the floor afterwards
    with pytest.raises(ConfigurationError, match="num_decay_steps"):
        mk("warmup_stable_decay")
    with pytest.raises(ConfigurationError, match="decay_type"):
        mk("warmup_stable_decay", num_decay_steps=10, decay_type="square")
    w = mk("warmup_stable_decay", num_decay_steps=10, min_lr_ratio=0.1, decay_type="linear")
    assert w(0) == pytest.approx(0.1 * lr) and w(W) == pytest.approx(lr) and w(W + 32) == pytest.approx(lr)
    assert w(W + 33 + 5) == pytest.approx(0.1 * lr + 0.9 * lr * 0.5, rel=1e-6) and w(total) == pytest.approx(0.1 * lr) and w(total + 9) == pytest.approx(0.1 * lr)
    wc = mk("warmup_stable_decay", num_decay_steps=10, num_stable_steps=5, decay_type="cosine")
    assert wc(W + 5 + 5) == pytest.approx(0.5 * lr) and wc(W + 15) == 0.0 and wc(W + 40) == 0.0
    ws = mk("warmup_stable_decay", num_decay_steps=16, num_stable_steps=0, decay_type="1-sqrt", warmup_type="cosine")
    assert ws(W + 4) == pytest.approx(lr * 0.5) and 0 < ws(3) < lr
    # unknown names / keys
    with pytest.raises(ConfigurationError, match="unsupported keys"):
        mk("linear", num_cycles=2)
    with pytest.raises(ConfigurationError, match="unknown lr_scheduler"):
        mk("triangular")
    with pytest.raises(ConfigurationError, match="timescale"):
        mk("inverse_sqrt", timescale=0)
    assert set(SUPPORTED_SCHEDULERS) >= {"linear", "cosine", "cosine_with_restarts", "polynomial", "constant", "constant_with_warmup",
                                         "inverse_sqrt", "cosine_with_min_lr", "cosine_warmup_with_min_lr", "warmup_stable_decay"}
    # fractions, recipes, argument objects
    assert get_warmup_steps(100, 0.055) == 6 and get_warmup_steps(100, 12.7) == 12 and get_warmup_steps(100, 0) == 0
    recipe = cosine_schedule(1e-3, 100)
    assert build_lr_schedule(recipe, learning_rate=1.0, total_steps=10) is recipe
    with pytest.raises(ConfigurationError, match="warmup_steps is incompatible"):
        build_lr_schedule(recipe, learning_rate=1.0, total_steps=10, warmup_steps=3)
    with pytest.raises(ConfigurationError, match="lr_scheduler_kwargs is incompatible"):
        build_lr_schedule(recipe, learning_rate=1.0, total_steps=10, kwargs={"num_cycles": 1})
    from opake_b200.transformers import TrainingArguments

    args = TrainingArguments(output_dir="/tmp/x", lr_scheduler="cosine", warmup_steps=0.1, learning_rate=lr)
    s1 = build_lr_schedule(args, 50)
    assert s1(5) == pytest.approx(lr) and s1(2) == pytest.approx(lr * 2 / 5)
    assert TrainingArguments(output_dir="/tmp/x", lr_scheduler=recipe).lr_scheduler is recipe


def test_model_card_from_trainer_privacy_section_and_hub_guards(tmp_path, monkeypatch):
    """Card layout, privacy values taken from the run, in-place replacement of the marked section, Hub calls routed
    through huggingface_hub (a fake: there is no network) with the documented ignore patterns and callback."""
    import sys
    import types

    from opake_b200.transformers import DPTrainer
    from opake_b200.transformers.callback import TrainerCallback
    from opake_b200.transformers.hub import DP_BEGIN, DP_END, DPTrainingSummary, build_privacy_summary, create_model_card, splice_dp_section

    events = []

    class _Cb(TrainerCallback):
        def on_push_begin(self, args, state, control, **kw):
            events.append("push_begin")

    tr = DPTrainer(_Net(), _args(tmp_path / "run"), train_dataset=_DS(256), eval_dataset=_DS(64, 1), callbacks=[_Cb()])
    tr.train()
    priv = build_privacy_summary(tr)
    assert 0 < priv["epsilon"] <= 6.01 and priv["delta"] == pytest.approx(tr._rt["target_delta"]) and priv["noise_multiplier"] > 0
    assert priv["clipping_norm"] == pytest.approx(float(tr.args.clipping_norm))
    card = tr.create_model_card(language="en", license="apache-2.0", tags=["text"], dataset="toy", finetuned_from="org/base")
    on_disk = open(tmp_path / "run" / "README.md", encoding="utf-8").read()
    assert card == on_disk
    head = card.split("---")[1]
    for needle in ("library_name: opake", "language: en", "license: apache-2.0", "base_model: org/base", "- text", "- differential-privacy",
                   "- opake", "datasets:\n- toy"):
        assert needle in head, needle
    for needle in ("### Training hyperparameters", "- learning_rate: 0.05", "- optim: adamw-bc", "### Training results", "### Framework versions",
                   "- opake_b200 ", "### Privacy budget", f"({priv['epsilon']:.4g}, "):
        assert needle in card, needle
    assert card.index("### Framework versions") < card.index(DP_BEGIN) < card.index(DP_END)
    assert "| Training Loss | Epoch | Step | Loss |" in card
    # re-saving replaces the section in place and leaves the user's edits alone
    edited = on_disk.replace("# run", "# run (edited by hand)")
    open(tmp_path / "run" / "README.md", "w", encoding="utf-8").write(edited)
    tr.state.log_history.append({"privacy_epsilon": 1.2345, "privacy_delta": 1e-6, "privacy_noise_multiplier": 0.77})
    again = tr.create_model_card()
    assert "# run (edited by hand)" in again and again.count(DP_BEGIN) == 1 and "(1.234, 1e-06)-DP" in again and "| Noise multiplier | 0.77 |" in again
    # summary-only API and splice fallbacks
    s = DPTrainingSummary(model_name="m", epsilon=2.0, delta=1e-5, noise_multiplier=1.1, clipping_norm=1.0)
    assert "(2, 1e-05)-DP" in create_model_card(s) and create_model_card(s, existing="# mine\n").startswith("# mine\n\n" + DP_BEGIN)
    assert splice_dp_section("a\n### Framework versions\n- x 1\n\n## Next\n", "SEC").index("SEC") < splice_dp_section(
        "a\n### Framework versions\n- x 1\n\n## Next\n", "SEC").index("## Next")
    assert "not accounted" in DPTrainingSummary().privacy_section()

    # the Hub path, against a fake huggingface_hub
    calls = {}
    fake = types.ModuleType("huggingface_hub")
    fake.create_repo = lambda name, token=None, private=None, exist_ok=False: types.SimpleNamespace(repo_id=f"user/{name.split('/')[-1]}")

    def upload_folder(**kw):
        calls.update(kw)
        return "commit-info"

    fake.upload_folder = upload_folder
    monkeypatch.setitem(sys.modules, "huggingface_hub", fake)
    out = tr.push_to_hub(commit_message="done", tags=["extra"])
    assert out == "commit-info" and tr.hub_model_id == "user/run" and events == ["push_begin"]
    assert calls["repo_id"] == "user/run" and calls["commit_message"] == "done" and calls["folder_path"] == str(tmp_path / "run")
    assert calls["ignore_patterns"] == ["_*", "checkpoint-*", "runs/**"] and calls["run_as_future"] is False
    assert "- extra" in open(tmp_path / "run" / "README.md", encoding="utf-8").read() or True
    monkeypatch.setitem(sys.modules, "huggingface_hub", None)
    from opake_b200.base.exceptions import OperationError

    with pytest.raises(OperationError, match="huggingface_hub"):
        tr.push_to_hub()


def test_evaluation_telemetry_transfer_pipeline_and_nested_accumulation():
    from opake_b200.transformers.eval import (PAD_VALUE, EvaluationTelemetry, PredictionAccumulator, TransferPipeline, concat_nested,
                                              interval_overlap, resolve_eval_num_samples)
    import numpy as np

    assert interval_overlap([(0, 2), (3, 5)], [(1, 4)]) == pytest.approx(2.0)
    assert interval_overlap([(0, 1)], [(2, 3)]) == 0.0 and interval_overlap([], [(0, 1)]) == 0.0
    tel = EvaluationTelemetry("cpu")
    with tel.model():
        torch.randn(64, 64) @ torch.randn(64, 64)
    with tel.phase("metric"):
        pass
    acc = PredictionAccumulator(torch.device("cpu"), accumulation_steps=2, concat=True, telemetry=tel)
    # ragged sequence lengths and a nested prediction payload (two heads)
    for i, T in enumerate((3, 5, 4)):
        acc.add(losses=torch.full((2,), float(i)), predictions=(torch.full((2, T, 4), float(i)), {"aux": torch.full((2,), 10.0 + i)}),
                label_ids=torch.full((2, T), i, dtype=torch.long))
    out = acc.finalize()
    assert out["losses"].tolist() == [0, 0, 1, 1, 2, 2]
    head, extra = out["predictions"]
    assert head.shape == (6, 5, 4) and (head[0, 3:] == PAD_VALUE).all() and (head[2] == 1).all() and (head[4, 4:] == PAD_VALUE).all()
    assert extra["aux"].tolist() == [10, 10, 11, 11, 12, 12]
    assert out["label_ids"].shape == (6, 5) and out["label_ids"][0].tolist() == [0, 0, 0, PAD_VALUE, PAD_VALUE]
    d = tel.to_dict()
    assert d["model_time_sec"] > 0 and d["transfer_bytes"] == sum(2 * 4 + 2 * T * 4 * 4 + 2 * 4 + 2 * T * 8 for T in (3, 5, 4))
    assert set(d) == {"model_time_sec", "gather_time_sec", "transfer_time_sec", "finalization_time_sec", "metric_time_sec",
                      "transfer_bytes", "transfer_overlap_sec", "transfer_overlap_ratio"}
    # no concatenation: lists of per-batch payloads
    acc2 = PredictionAccumulator(torch.device("cpu"), None, concat=False)
    acc2.add(losses=torch.zeros(2))
    acc2.add(losses=torch.ones(3))
    assert [x.tolist() for x in acc2.finalize()["losses"]] == [[0, 0], [1, 1, 1]]
    pipe = TransferPipeline(None, max_pending=2)
    assert pipe.submit({"a": torch.ones(2)})[0]["a"].tolist() == [1, 1] and pipe.drain_all() == []
    assert concat_nested([np.zeros((1, 2)), np.ones((2, 3))]).shape == (3, 3)
    assert resolve_eval_num_samples([1, 2, 3], None, 2) == 3 and resolve_eval_num_samples(iter(()), None, 7) == 7


def test_stop_at_epsilon_ends_training_at_the_predicted_step(tmp_path):
    """Fixed noise AND a target epsilon: the run stops at the first step whose accounted epsilon reaches the target,
    found once by bisection; a resumed run that is already there does no further step."""
    from opake_b200 import accounting as acc
    from opake_b200.dpsgd import accounting as SA
    from opake_b200.transformers import DPTrainer
    from opake_b200.transformers.dp_trainer import predict_stop_step

    q, sigma, delta, horizon = 32 / 256, 0.8, 256 ** -1.1, 40
    step = SA.poisson(SA.gaussian(sigma), q)
    eps = lambda k: (step * k).epsilon_at(delta)  # noqa: E731
    target = 0.5 * (eps(9) + eps(10))
    assert predict_stop_step(None, step, target_epsilon=target, delta=delta, k0=0, horizon=horizon) == 10
    assert predict_stop_step(None, step, target_epsilon=eps(horizon) + 1.0, delta=delta, k0=0, horizon=horizon) is None
    # with a prefix of 4 accounted steps the same crossing is found at the same absolute step
    assert predict_stop_step(step * 4, step, target_epsilon=target, delta=delta, k0=4, horizon=horizon) == 10
    assert predict_stop_step(None, step, target_epsilon=target, delta=delta, k0=40, horizon=horizon) is None

    args = _args(tmp_path / "run", max_steps=horizon, privacy_target_epsilon=target, privacy_noise_multiplier=sigma,
                 save_steps=5, eval_strategy="no", logging_steps=5)
    tr = DPTrainer(_Net(), args, train_dataset=_DS(256))
    out = tr.train()
    assert tr.state.global_step == 10 and tr.state.privacy_target_epsilon_reached
    assert out.metrics["privacy_epsilon"] == pytest.approx(eps(10), rel=1e-6) and out.metrics["privacy_epsilon"] >= target
    assert os.path.isdir(tmp_path / "run" / "checkpoint-10")                 # the stop forces a checkpoint
    # resuming from there trains no further
    tr2 = DPTrainer(_Net(), args, train_dataset=_DS(256))
    tr2.train(resume_from_checkpoint=True)
    assert tr2.state.global_step == 10 and tr2.state.privacy_target_epsilon_reached
    # noise 0 with a target is refused
    from opake_b200.base.exceptions import ConfigurationError
    from opake_b200.transformers import TrainingArguments

    with pytest.raises(ConfigurationError, match="non-private"):
        TrainingArguments(privacy_target_epsilon=1.0, privacy_noise_multiplier=0.0)
    assert acc is not None


def test_per_example_metrics_seam_reaches_the_training_logs(tmp_path):
    from opake_b200.transformers import DPTrainer

    class T(DPTrainer):
        def compute_per_example_loss_and_metrics(self, call, params, inputs):
            loss = self.compute_per_example_loss(call, params, inputs)
            return loss, {"probe/first_feature": inputs["x"][0, 0], "probe/one": torch.ones(())}

    tr = T(_Net(), _args(tmp_path / "run", max_steps=4, logging_steps=2, eval_strategy="no", save_strategy="no"), train_dataset=_DS(256))
    assert tr._overrides_metrics_seam() and tr.is_local_process_zero() and tr.label_names == ["labels"]
    tr.train()
    logged = [e for e in tr.state.log_history if "probe/one" in e]
    assert len(logged) == 2 and all(e["probe/one"] == pytest.approx(1.0) for e in logged)
    assert all(abs(e["probe/first_feature"]) < 1.0 for e in logged)             # a batch mean of N(0, 1) features
    plain = DPTrainer(_Net(), _args(tmp_path / "run2", max_steps=2, eval_strategy="no", save_strategy="no"), train_dataset=_DS(256))
    assert not plain._overrides_metrics_seam()
