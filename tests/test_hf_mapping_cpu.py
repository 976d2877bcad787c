"""Hugging Face state-dict mapping of the native decoder layouts (CPU): export then import is the identity, for the
dense Llama layout, the GPT-2 layout and the OLMoE layout with query / key norms and interleaved expert weights."""
import pytest
import torch

from opake_b200.models import config as C
from opake_b200.models.flat import build_layout
from opake_b200.models.native import config_from_hf, flat_views_to_hf, hf_to_flat_views


def _cfg(name):
    if name == "llama":
        return C.tiny_llama()
    if name == "llama-tied":
        return C.tiny_llama(tie_embeddings=True)
    if name == "qwen2":
        return C.tiny_llama(qkv_bias=True, family="qwen2", name="tiny-qwen2")
    if name == "qwen3":
        return C.tiny_llama(qk_norm="head", family="qwen3", name="tiny-qwen3")
    if name == "olmoe":
        return C.tiny_llama(n_experts=4, top_k=2, expert_ffn=64, ffn=0, qk_norm=True, family="olmoe", name="tiny-olmoe")
    return C.gpt2_small(n_layers=2, d_model=64, n_heads=2, n_kv_heads=2, head_dim=32, ffn=128, vocab_size=101, max_seq=16,
                        name="tiny-gpt2")


@pytest.mark.parametrize("name", ["llama", "llama-tied", "qwen2", "qwen3", "olmoe", "gpt2"])
def test_export_then_import_is_identity(name):
    cfg = _cfg(name)
    layout = build_layout(cfg)
    g = torch.Generator().manual_seed(0)
    buf = torch.randn(layout.total, generator=g)
    w = layout.views(buf)
    sd = {k: v.clone() for k, v in flat_views_to_hf(cfg, w).items()}
    buf2 = torch.zeros(layout.total)
    w2 = layout.views(buf2)
    hf_to_flat_views(cfg, sd, w2)
    for s in layout.slots:
        assert torch.equal(w2[s.name], w[s.name]), s.name
    if name == "olmoe":
        # expert gate / up projections are stored interleaved (row 2j = gate j, row 2j + 1 = up j)
        e0 = w["layers.0.experts.wgu"][0]
        assert torch.equal(sd["model.layers.0.mlp.experts.0.gate_proj.weight"], e0[0::2])
        assert torch.equal(sd["model.layers.0.mlp.experts.0.up_proj.weight"], e0[1::2])
        assert "model.layers.1.self_attn.q_norm.weight" in sd and "model.layers.1.self_attn.k_norm.weight" in sd
        assert sd["model.layers.0.self_attn.k_norm.weight"].shape == (cfg.n_kv_heads * cfg.head_dim,)


def test_config_from_hf_recognises_families():
    llama = config_from_hf(dict(model_type="llama", vocab_size=128256, hidden_size=4096, num_hidden_layers=32,
                                num_attention_heads=32, num_key_value_heads=8, intermediate_size=14336, rope_theta=500000.0,
                                max_position_embeddings=8192, rms_norm_eps=1e-5))
    assert (llama.d_model, llama.n_kv_heads, llama.head_dim, llama.ffn, llama.act, llama.qk_norm) == (4096, 8, 128, 14336, "swiglu", False)
    olmoe = config_from_hf(dict(model_type="olmoe", vocab_size=50304, hidden_size=2048, num_hidden_layers=16,
                                num_attention_heads=16, num_key_value_heads=16, intermediate_size=1024, num_experts=64,
                                num_experts_per_tok=8, norm_topk_prob=False))
    assert olmoe.qk_norm and olmoe.n_experts == 64 and olmoe.top_k == 8 and olmoe.expert_ffn == 1024
    gpt2 = config_from_hf(dict(model_type="gpt2", vocab_size=50257, n_embd=768, n_layer=12, n_head=12))
    assert gpt2.norm == "layer" and gpt2.pos == "learned" and gpt2.bias and gpt2.tie_embeddings and gpt2.ffn == 3072


@pytest.mark.parametrize("family", ["qwen2", "qwen3"])
def test_native_reference_math_matches_hugging_face_model(family):
    """A tiny random-init Hugging Face Qwen2 (q/k/v bias) / Qwen3 (per-head q/k norm) lowered to the native layout:
    the fp32 reference math of the native runtime gives the Hugging Face loss, and the exported state dict loads back
    into the Hugging Face class."""
    transformers = pytest.importorskip("transformers")
    from opake_b200.models.reference_torch import example_loss
    from opake_b200.ops.kernels import rope_table

    torch.manual_seed(0)
    common = dict(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=64, tie_word_embeddings=False, rope_theta=10000.0)
    if family == "qwen2":
        hf = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**common))
    else:
        hf = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(head_dim=8, **common))
    for n, p in hf.named_parameters():          # non-trivial biases and norm weights
        if p.dim() == 1:
            p.data.add_(0.1 * torch.randn_like(p))
    hf = hf.eval()
    cfg = config_from_hf(hf.config)
    assert cfg.qkv_bias == (family == "qwen2") and cfg.qk_norm == ("head" if family == "qwen3" else False)
    layout = build_layout(cfg)
    buf = torch.zeros(layout.total)
    w = layout.views(buf)
    hf_to_flat_views(cfg, hf.state_dict(), w)
    T = 12
    ids = torch.randint(1, 97, (T,))
    with torch.no_grad():
        want = hf(ids[None], labels=ids[None]).loss.item()
    labels = torch.roll(ids, -1)
    labels[-1] = -100
    table = rope_table(T, cfg.head_dim, cfg.rope_theta, torch.device("cpu"))
    got = example_loss(cfg, w, ids.int(), labels.int(), table).item()          # mean over the T - 1 targets
    assert got == pytest.approx(want, rel=2e-4)
    back = flat_views_to_hf(cfg, w)
    missing, unexpected = hf.load_state_dict({k: v.clone() for k, v in back.items()}, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing)
