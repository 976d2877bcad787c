"""Hugging Face model families under ``apply_model_patches``: a tiny random-init model of each family must (1) give
the stock model's loss after patching (the replacement attention honours grouped heads, sliding windows, logit
soft-capping, q/k norms, biases, fused projections, expert routing), and (2) yield per-example gradients under
``vmap(grad)`` equal to a per-example loop (the layout of packages/opake-patches/tests/transformers/models/ in the
reference)."""
import copy

import pytest
import torch
from torch.func import functional_call, grad, vmap

transformers = pytest.importorskip("transformers")

_COMMON = dict(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               max_position_embeddings=64, tie_word_embeddings=False)
_FAMILIES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", {}),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", {}),                                   # q/k/v bias
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", {"head_dim": 8}),                      # per-head q/k RMSNorm
    "mistral": ("MistralConfig", "MistralForCausalLM", {"sliding_window": 6}),
    "gemma": ("GemmaConfig", "GemmaForCausalLM", {"head_dim": 8}),                      # weight - 1 norms, tanh GeLU gate
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM", {"head_dim": 8, "sliding_window": 6, "query_pre_attn_scalar": 8}),
    "gemma3_text": ("Gemma3TextConfig", "Gemma3ForCausalLM", {"head_dim": 8, "sliding_window": 6, "query_pre_attn_scalar": 8}),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", {"pad_token_id": 0}),                     # fused qkv and gate_up
    "glm4": ("Glm4Config", "Glm4ForCausalLM", {"head_dim": 8, "pad_token_id": 0}),
    "olmo2": ("Olmo2Config", "Olmo2ForCausalLM", {}),                                   # post-norm, q/k norm
    "granite": ("GraniteConfig", "GraniteForCausalLM", {}),
    "cohere": ("CohereConfig", "CohereForCausalLM", {}),                                # parallel block
    "smollm3": ("SmolLM3Config", "SmolLM3ForCausalLM", {"pad_token_id": 0}),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", {"num_local_experts": 4, "num_experts_per_tok": 2}),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", {"head_dim": 8, "num_experts": 4, "num_experts_per_tok": 2,
                                                            "moe_intermediate_size": 16}),
    "olmoe": ("OlmoeConfig", "OlmoeForCausalLM", {"num_experts": 4, "num_experts_per_tok": 2}),
}


def _tiny(family: str):
    if family == "gpt2":
        return transformers.GPT2LMHeadModel(transformers.GPT2Config(vocab_size=97, n_embd=32, n_layer=2, n_head=4, n_positions=64))
    cn, mn, extra = _FAMILIES[family]
    if not hasattr(transformers, cn):
        pytest.skip(f"this transformers version has no {cn}")
    return getattr(transformers, mn)(getattr(transformers, cn)(**{**_COMMON, **extra}))


@pytest.mark.parametrize("family", [*_FAMILIES, "gpt2"])
def test_family_patched_loss_and_per_example_gradients(family):
    from opake_b200 import patches
    torch.manual_seed(0)
    model = _tiny(family).eval()
    B, T = 3, 12
    ids = torch.randint(1, 97, (B, T))
    stock = copy.deepcopy(model)
    with torch.no_grad():
        want = torch.stack([stock(ids[b : b + 1], labels=ids[b : b + 1]).loss for b in range(B)])
    report = patches.apply_model_patches(model)
    assert report["family"] is not None, "family not registered"
    with torch.no_grad():
        got = torch.stack([model(ids[b : b + 1], labels=ids[b : b + 1]).loss for b in range(B)])
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (got, want)
    params = {k: v.detach() for k, v in model.named_parameters()}

    def loss(p, x):
        return functional_call(model, p, (x.unsqueeze(0),), {"labels": x.unsqueeze(0)}).loss

    g_v = vmap(grad(loss), in_dims=(None, 0))(params, ids)
    for b in range(B):
        g_1 = grad(loss)(params, ids[b])
        for k in g_1:
            assert torch.allclose(g_v[k][b], g_1[k], rtol=1e-4, atol=1e-6), (family, k, b)
    # sanity: the examples do have different gradients
    some = next(k for k in g_v if g_v[k].abs().sum() > 0)
    assert not torch.allclose(g_v[some][0], g_v[some][1])


@pytest.mark.parametrize("offload", [False, True])
def test_gradient_checkpointing_under_vmap_grad(offload):
    """Layer checkpointing of a Hugging Face model inside ``vmap(grad)``: same per-example gradients, and every decoder
    layer runs twice (forward, then recomputation in the backward pass)."""
    from opake_b200 import patches
    from opake_b200.patches.torch_checkpoint import apply_gradient_checkpointing
    torch.manual_seed(0)
    model = _tiny("qwen3")
    patches.apply_model_patches(model)
    model.train()
    params = {k: v.detach() for k, v in model.named_parameters()}
    ids = torch.randint(1, 97, (3, 12))

    def loss(p, x):
        return functional_call(model, p, (x.unsqueeze(0),), {"labels": x.unsqueeze(0)}).loss

    want = vmap(grad(loss), in_dims=(None, 0))(params, ids)
    assert apply_gradient_checkpointing(model, offload=offload)
    calls = {"n": 0}
    layer = model.model.layers[1]
    inner = layer.forward

    def counting(*a, **k):
        calls["n"] += 1
        return inner(*a, **k)

    layer.forward = counting
    got = vmap(grad(loss), in_dims=(None, 0))(params, ids)
    assert calls["n"] == 2
    for k in want:
        assert torch.allclose(got[k], want[k], rtol=1e-5, atol=1e-7), k
