"""The vmap-safety and performance components behind ``apply_model_patches`` / ``apply_runtime_patches``, one by one
(the layout of packages/opake-patches/tests/transformers/components/ and runtime/ in the reference)."""
import copy

import pytest
import torch
from torch.func import functional_call, grad, vmap

transformers = pytest.importorskip("transformers")


def _llama(**kw):
    cfg = transformers.LlamaConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64, tie_word_embeddings=False, **kw)
    return transformers.LlamaForCausalLM(cfg)


def test_kv_cache_wrapper_only_acts_in_training_without_cache_content():
    from opake_b200.patches.transformers.components import disable_kv_cache_in_training

    seen = {}

    class M:
        training = True

        def forward(self, x, past_key_values=None, use_cache=None):
            seen["use_cache"] = use_cache
            return x

    fwd = disable_kv_cache_in_training(M.forward)
    assert disable_kv_cache_in_training(fwd) is fwd                      # idempotent
    m = M()
    fwd(m, 1, use_cache=True)
    assert seen["use_cache"] is False
    m.training = False
    fwd(m, 1, use_cache=True)
    assert seen["use_cache"] is True
    m.training = True
    with torch.no_grad():
        fwd(m, 1, use_cache=True)
    assert seen["use_cache"] is True

    class Cache:
        def get_seq_length(self):
            return 5

    fwd(m, 1, past_key_values=Cache(), use_cache=True)
    assert seen["use_cache"] is True                                     # a cache with content: generation, hands off
    fwd(m, 1, past_key_values=[], use_cache=True)
    assert seen["use_cache"] is False


def test_patched_model_accepts_unbatched_inputs_and_generates():
    from opake_b200 import patches

    torch.manual_seed(0)
    model = _llama().eval()
    ids = torch.randint(1, 97, (2, 9))
    with torch.no_grad():
        want = model(ids[:1]).logits[0]
    rep = patches.apply_model_patches(model)
    fwd = type(model).forward            # class-level wrappers (counts in the report are "newly installed by this call")
    assert all(getattr(fwd, mark, False) for mark in ("_opake_batchified", "_opake_cache_disabled", "_opake_fused_ce"))
    assert rep["loss_function"] == 1 and rep["fused_linear_cross_entropy"] is True
    with torch.no_grad():
        got = model(ids[0]).logits                                       # [T] in, [T, V] out
        out = model(ids[0], labels=ids[0])
    assert got.shape == (9, 97) and torch.allclose(got, want, atol=1e-5)
    assert out.loss.dim() == 0
    # generation still uses (and fills) a cache
    gen = model.generate(ids[:1, :4], max_new_tokens=3, do_sample=False, pad_token_id=0)
    assert gen.shape == (1, 7)
    # a second application changes nothing
    rep2 = patches.apply_model_patches(model)
    assert rep2["batchify"] == 0 and rep2["kv_cache"] == 0 and rep2["norms"] == 0


def test_padded_examples_under_vmap_grad_match_loop():
    """Padding masks need the vmap-safe mask builders: the stock ones branch on ``padding_mask.all()``."""
    from opake_b200 import patches

    torch.manual_seed(1)
    model = _llama().eval()
    patches.apply_model_patches(model)
    B, T = 3, 10
    ids = torch.randint(1, 97, (B, T))
    mask = torch.ones(B, T, dtype=torch.long)
    mask[0, 7:] = 0
    mask[2, 4:] = 0
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    params = {k: v.detach() for k, v in model.named_parameters()}

    def loss(p, x, m, y):
        return functional_call(model, p, (x,), {"attention_mask": m, "labels": y}).loss

    g_v = vmap(grad(loss), in_dims=(None, 0, 0, 0))(params, ids, mask, labels)
    for b in range(B):
        n = int(mask[b].sum())
        g_1 = grad(lambda p: functional_call(model, p, (ids[b : b + 1, :n],), {"labels": ids[b : b + 1, :n]}).loss)(params)
        for k in g_1:
            assert torch.allclose(g_v[k][b], g_1[k], rtol=2e-4, atol=2e-6), (k, b)


def test_causal_lm_loss_function_matches_stock_and_refuses_batch_normalisation():
    from opake_b200.patches.transformers.components import opake_causal_lm_loss
    from transformers.loss.loss_utils import ForCausalLMLoss

    torch.manual_seed(2)
    logits = torch.randn(2, 7, 31)
    labels = torch.randint(0, 31, (2, 7))
    labels[0, 3:5] = -100
    got, want = opake_causal_lm_loss(logits, labels, 31), ForCausalLMLoss(logits, labels, 31)
    assert torch.allclose(got, want, atol=1e-6)
    sm = opake_causal_lm_loss(logits, labels, 31, label_smoothing=0.1)
    assert sm > got - 1.0 and sm != got
    with pytest.raises(ValueError, match="num_items_in_batch"):
        opake_causal_lm_loss(logits, labels, 31, num_items_in_batch=5)


@pytest.mark.parametrize("family_kw", [{}, {"final": 30.0}])
def test_fused_linear_cross_entropy_forward_is_conditional_and_exact(family_kw):
    from opake_b200 import patches

    torch.manual_seed(3)
    if family_kw:
        cfg = transformers.Gemma2Config(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                        num_key_value_heads=2, head_dim=8, max_position_embeddings=64, final_logit_softcapping=30.0,
                                        query_pre_attn_scalar=8, sliding_window=6, tie_word_embeddings=False)
        model = transformers.Gemma2ForCausalLM(cfg).eval()
    else:
        model = _llama().eval()
    stock = copy.deepcopy(model)
    patches.apply_model_patches(model)
    ids = torch.randint(1, 97, (3, 11))
    labels = ids.clone()
    labels[1, :4] = -100
    with torch.no_grad():
        want = torch.stack([stock(ids[b : b + 1], labels=labels[b : b + 1]).loss for b in range(3)])
        full = model(ids[:1], labels=labels[:1])                                   # not loss_only: logits materialised
        fused = [model(ids[b : b + 1], labels=labels[b : b + 1], loss_only=True) for b in range(3)]
    assert full.logits is not None and all(o.logits is None for o in fused)
    assert torch.allclose(torch.stack([o.loss for o in fused]), want, rtol=1e-4, atol=1e-5)
    # calls the fused branch cannot serve fall back to the stock forward
    with torch.no_grad():
        kept = model(ids[:1], loss_only=True, logits_to_keep=2)                    # no labels: nothing to fuse
        smooth = model(ids[:1], labels=labels[:1], loss_only=True, label_smoothing=0.1)
    assert kept.logits is not None and kept.logits.shape[1] == 2 and smooth.logits is not None
    # per-example gradients through the fused branch
    params = {k: v.detach() for k, v in model.named_parameters()}

    def loss(p, x, y):
        return functional_call(model, p, (x,), {"labels": y, "loss_only": True}).loss

    g_v = vmap(grad(loss), in_dims=(None, 0, 0))(params, ids, labels)
    sparams = {k: v.detach() for k, v in stock.named_parameters()}
    for b in range(3):
        g_1 = grad(lambda p: functional_call(stock, p, (ids[b : b + 1],), {"labels": labels[b : b + 1]}).loss)(sparams)
        for k in g_1:
            assert torch.allclose(g_v[k][b], g_1[k], rtol=5e-4, atol=5e-6), (k, b)


@pytest.mark.parametrize("window", [0, 5])
def test_softcapped_attention_recompute_matches_autograd_and_vmaps(window):
    from opake_b200.patches.transformers.components import eager_attention_forward, softcapped_attention_recompute

    torch.manual_seed(4)
    H, KV, T, hd = 4, 2, 13, 8
    q = torch.randn(1, H, T, hd, dtype=torch.float64, requires_grad=True)
    k = torch.randn(1, KV, T, hd, dtype=torch.float64, requires_grad=True)
    v = torch.randn(1, KV, T, hd, dtype=torch.float64, requires_grad=True)
    w = torch.randn(1, H, T, hd, dtype=torch.float64)
    ref, _ = eager_attention_forward(None, q, k, v, softcap=7.0, sliding_window=window or None)
    (ref.transpose(1, 2) * w).sum().backward()
    want = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    got = softcapped_attention_recompute(q, k, v, 7.0, sliding_window=window or None, chunk=4)
    assert torch.allclose(got, ref.transpose(1, 2), atol=1e-5)           # the eager form takes its softmax in fp32
    (got * w).sum().backward()
    for a, b in zip((q.grad, k.grad, v.grad), want):
        assert torch.allclose(a, b, atol=1e-5)
    # per-example gradients under vmap(grad)
    qb, kb, vb = (torch.randn(3, 1, n, T, hd, dtype=torch.float64) for n in (H, KV, KV))
    f = lambda a, b, c: softcapped_attention_recompute(a, b, c, 7.0, sliding_window=window or None, chunk=4).pow(2).sum()  # noqa: E731
    gv = vmap(grad(f, argnums=(0, 1, 2)))(qb, kb, vb)
    for i in range(3):
        g1 = grad(f, argnums=(0, 1, 2))(qb[i], kb[i], vb[i])
        for a, b in zip(gv, g1):
            assert torch.allclose(a[i], b, atol=1e-9)


def test_rope_replacement_keeps_stock_semantics_off_the_fast_path():
    from opake_b200.patches.transformers.components import apply_rope_patch, opake_apply_rotary_pos_emb
    import transformers.models.llama.modeling_llama as ml

    model = _llama()
    stock = ml.apply_rotary_pos_emb
    stock = getattr(stock, "__wrapped__", stock)
    n = apply_rope_patch(model)
    assert n in (0, 1) and getattr(ml.apply_rotary_pos_emb, "_opake_rope", False) and apply_rope_patch(model) == 0
    q, k = torch.randn(2, 4, 6, 8), torch.randn(2, 2, 6, 8)
    ang = torch.randn(2, 6, 4)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    for fn in (ml.apply_rotary_pos_emb, opake_apply_rotary_pos_emb):
        a, b = fn(q, k, cos, sin)
        wa, wb = stock(q, k, cos, sin)
        assert torch.allclose(a, wa) and torch.allclose(b, wb)


def test_runtime_patches_collators_grouped_gemm_and_dropout():
    from opake_b200 import patches
    from opake_b200.patches.transformers.components import disable_dropout
    import transformers.integrations.moe as hf_moe

    rep = patches.apply_runtime_patches()
    assert patches.is_runtime_patched() and set(rep) >= {"masking", "collators", "grouped_mm"}
    assert getattr(hf_moe._can_use_grouped_mm, "_opake_vmap_safe", False)
    import transformers.masking_utils as mu

    assert getattr(mu.create_causal_mask, "_opake_vmap_safe", False) and getattr(mu._ignore_causal_mask_sdpa, "_opake_vmap_safe", False)
    assert mu._ignore_causal_mask_sdpa(torch.ones(1, 4, dtype=torch.bool), 4, 4, 0) is False

    class Tok:
        pad_token_id, pad_token, padding_side = 0, "<pad>", "right"

        def pad(self, examples, return_tensors=None, pad_to_multiple_of=None, **_kw):
            n = max(len(e["input_ids"]) for e in examples)
            return {"input_ids": torch.tensor([e["input_ids"] + [0] * (n - len(e["input_ids"])) for e in examples])}

        def get_special_tokens_mask(self, ids, already_has_special_tokens=True):
            return [0] * len(ids)

        def __len__(self):
            return 50

    coll = transformers.DataCollatorForLanguageModeling(Tok(), mlm=False)
    first = coll([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}])
    empty = coll([])                                                   # a Poisson draw that selected nobody
    assert set(empty) == set(first) and empty["input_ids"].shape[0] == 0 and empty["input_ids"].dtype == first["input_ids"].dtype

    model = _llama(attention_dropout=0.1)
    model.model.layers[0].self_attn.attention_dropout = 0.1
    drop = torch.nn.Dropout(0.3)
    model.extra = drop
    assert disable_dropout(model) >= 2
    assert drop.p == 0.0 and model.model.layers[0].self_attn.attention_dropout == 0.0 and model.config.attention_dropout == 0.0


def test_user_registered_family_goes_through_the_factories():
    """A model type that is not built in: module-level patches from ``make_apply_family_patches``, per-role forwards by
    kind from ``make_apply_model_patches`` (activation, RMSNorm, fused add + RMSNorm decoder layer, loss), routed by
    ``register_family``; losses and per-example gradients agree with the stock model."""
    from opake_b200 import patches
    from opake_b200.base.exceptions import ConfigurationError
    from opake_b200.patches import transformers as PT

    class MyConfig(transformers.LlamaConfig):
        model_type = "my_llama"

    torch.manual_seed(5)
    model = transformers.LlamaForCausalLM(MyConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                                   tie_word_embeddings=False)).eval()
    assert PT.family_name(model) == "my_llama" and "my_llama" not in PT.supported_families()
    stock = copy.deepcopy(model)
    seen = []

    def my_act(original):                                    # a custom kind: same math, observable
        def forward(self, x):
            seen.append("act")
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))
        return forward

    PT.register_activation_kind("my_swiglu", my_act)
    path = "transformers.models.llama.modeling_llama"
    fam = PT.make_apply_family_patches(family="my_llama", module_path=path)
    with pytest.raises(ConfigurationError, match="unknown kind"):
        PT.make_apply_model_patches(family="my_llama", family_apply=fam, module_path=path, classes={}, activation_kind="nope")
    apply = PT.make_apply_model_patches(family="my_llama", family_apply=fam, module_path=path,
                                        classes={"mlp": "LlamaMLP", "rms_norm": "LlamaRMSNorm", "decoder_layer": "LlamaDecoderLayer",
                                                 "causal_lm": "LlamaForCausalLM"},
                                        activation_kind="my_swiglu", rms_norm_kind="llama", fused_add_rms_kind="llama")
    PT.register_family("my_llama", apply)
    assert "my_llama" in PT.supported_families() and apply.__name__ == "apply_my_llama_patches"
    rep = patches.apply_model_patches(model)
    assert rep["family"] == "my_llama" and rep["mlps"] == 2 and rep["norms"] == 5 and rep["decoder_layers"] == 2
    assert rep["loss_function"] == 1
    ids = torch.randint(1, 97, (3, 10))
    with torch.no_grad():
        want = torch.stack([stock(ids[b : b + 1], labels=ids[b : b + 1]).loss for b in range(3)])
        got = torch.stack([model(ids[b : b + 1], labels=ids[b : b + 1]).loss for b in range(3)])
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5) and seen
    params = {k: v.detach() for k, v in model.named_parameters()}
    loss = lambda p, x: functional_call(model, p, (x,), {"labels": x}).loss  # noqa: E731
    g_v = vmap(grad(loss), in_dims=(None, 0))(params, ids)
    sparams = {k: v.detach() for k, v in stock.named_parameters()}
    for b in range(3):
        g_1 = grad(lambda p: functional_call(stock, p, (ids[b : b + 1],), {"labels": ids[b : b + 1]}).loss)(sparams)
        for k in g_1:
            assert torch.allclose(g_v[k][b], g_1[k], rtol=5e-4, atol=5e-6), (k, b)
    # second application: nothing new
    rep2 = patches.apply_model_patches(model)
    assert rep2["mlps"] == 0 and rep2["norms"] == 0 and rep2["decoder_layers"] == 0


def test_public_namespaces_match_the_reference_layout():
    """``from opake import random, scheduling, ...`` style imports resolve under this package's name."""
    import importlib

    surface = {
        "exceptions": "ConfigurationError OpakeError PrivacyBudgetError", "serialization": "state_dict from_state_dict register_serializer",
        "random": "key fold_in split generator_from_key", "scheduling": "cosine_schedule with_warmup warmup_stable_decay",
        "functional": "make_functional with_batch_dim empty_collate", "distributed": "sum_gradients_ local_shard sync is_main_process",
        "profiling": "step_perf PerfTracker get_memory_stats", "device": "device_capabilities fused_kernels_available",
        "accounting": "amplification calibration composition mechanisms Accountant calibrate epsilon_budget",
        "dpftrl": "clipping clipped_grad BallsInBinsSampler blt_strategy mf_gaussian_noise", "dpftrl.clipping": "clipped_grad per_group",
        "dpftrl.noise": "band_mf_strategy mf_gaussian_noise", "dpsgd": "clipped_grad gaussian_noise PoissonSampler",
        "alignment.dpo.loss": "sequence_logp fused_sequence_logp sigmoid_loss", "patches.torch": "apply_checkpoint_patch is_checkpoint_patched",
        "patches.kernels": "opake_rope opake_slow_rope opake_lora_qkv opake_geglu_exact ACTIVATION_SWIGLU opake_cross_entropy_loss",
        "patches.transformers": "register_family make_apply_model_patches supported_families family_name",
        "patches.transformers.runtime": "apply_collator_patches apply_grouped_mm_patches apply_masking_patches",
        "transformers": "DPTrainer TrainingArguments trl", "transformers.trl": "SFTTrainer DPOTrainer SFTConfig DPOConfig",
    }
    for mod, names in surface.items():
        m = importlib.import_module("opake_b200." + mod)
        assert not [n for n in names.split() if not hasattr(m, n)], mod


def test_checkpoint_patch_routes_only_inside_transforms():
    import torch.utils.checkpoint as tuc

    from opake_b200.patches.torch import apply_checkpoint_patch, is_checkpoint_patched

    apply_checkpoint_patch()
    assert is_checkpoint_patched() and apply_checkpoint_patch() is False
    lin = torch.nn.Linear(6, 6)
    f = lambda x: torch.tanh(lin(x)).pow(2).sum()  # noqa: E731
    x = torch.randn(4, 6)
    # outside a transform: the stock checkpoint
    y = tuc.checkpoint(lambda t: torch.tanh(lin(t)), x[0].clone().requires_grad_(), use_reentrant=False)
    assert y.requires_grad
    # inside vmap(grad): the functional recomputation
    g_ck = vmap(grad(lambda t: tuc.checkpoint(lambda u: torch.tanh(lin(u)), t, use_reentrant=False).pow(2).sum()))(x)
    g_pl = vmap(grad(f))(x)
    assert torch.allclose(g_ck, g_pl, atol=1e-6)
