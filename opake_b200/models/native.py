"""``NativeCausalLM``: the ``nn.Module`` face of a decoder whose parameters live in one flat buffer.

The same object serves both execution paths of the trainer. The sm_100a runtime (``DecoderRuntime`` /
``ShardedDPEngine``) consumes the flat buffer directly; ``forward`` is the plain-PyTorch restatement (CPU, evaluation,
``vmap(grad)`` clipping), so a model trained natively can be evaluated or fine-tuned generically and vice versa.
Weights convert to and from Hugging Face checkpoints of the supported families (Llama-like, GPT-2): q / k / v are
fused into one projection and gate / up rows are interleaved, which is what the fused GEMM epilogues expect.
"""
from __future__ import annotations

from typing import Any, Mapping

import torch
from torch import nn

from ..ops.kernels import rope_table
from .config import DecoderConfig
from .flat import build_layout
from .reference_torch import decoder_hidden

__all__ = ["NativeCausalLM", "config_from_hf", "hf_to_flat_views", "flat_views_to_hf"]


class NativeCausalLM(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype: torch.dtype = torch.float32, device=None, init_seed: int | None = 0):
        super().__init__()
        self.cfg = cfg
        self.layout = build_layout(cfg)
        self.flat = nn.Parameter(torch.zeros(self.layout.total, dtype=dtype, device=device))
        self._rope = None
        if init_seed is not None:
            from .decoder import init_params_
            with torch.no_grad():
                init_params_(cfg, self.flat.data, self.layout, seed=init_seed)

    # the Hugging Face attribute trainers look at
    @property
    def config(self) -> DecoderConfig:
        return self.cfg

    def views(self, flat: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        return self.layout.views(self.flat if flat is None else flat)

    def _rope_table(self, T: int, device) -> torch.Tensor | None:
        if self.cfg.pos != "rope":
            return None
        if self._rope is None or self._rope.shape[0] < T or self._rope.device != device:
            self._rope = rope_table(max(T, self.cfg.max_seq), self.cfg.head_dim, self.cfg.rope_theta, device=device,
                                    scaling=self.cfg.rope_scaling)
        return self._rope

    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Final-norm hidden states ``[..., T, d]``."""
        w = self.views()
        if input_ids.dim() == 1:
            return decoder_hidden(self.cfg, w, input_ids, self._rope_table(input_ids.shape[-1], self.flat.device))
        return torch.stack([self.hidden_states(row) for row in input_ids])

    def lm_head_weight(self) -> torch.Tensor:
        w = self.views()
        return w["embed"] if self.cfg.tie_embeddings else w["lm_head"]

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, attention_mask=None,
                output_hidden_states: bool = False, **_unused) -> dict[str, Any]:
        """Hugging Face calling convention: ``labels`` equal to ``input_ids`` with ``-100`` on ignored positions;
        position t predicts t+1. Padding must be on the right (causal attention never looks at it)."""
        h = self.hidden_states(input_ids)
        logits = h @ self.lm_head_weight().T
        out: dict[str, Any] = {"logits": logits}
        if output_hidden_states:
            out["last_hidden_state"] = h
        if labels is not None:
            from ..alignment.sft.loss import nll_loss
            per_seq = nll_loss(logits, labels)
            out["loss"] = per_seq.mean() if per_seq.dim() else per_seq
        return out

    # ------------------------------------------------------------------ Hugging Face interchange
    @classmethod
    def from_hf(cls, hf_model_or_state: Any, hf_config: Any | None = None, dtype: torch.dtype = torch.float32, device=None):
        """Builds the model from a Hugging Face causal LM (module or ``state_dict`` + config)."""
        if isinstance(hf_model_or_state, Mapping):
            sd, conf = hf_model_or_state, hf_config
        else:
            sd, conf = hf_model_or_state.state_dict(), hf_model_or_state.config
        if conf is None:
            raise ValueError("a Hugging Face config is needed to map a bare state dict")
        cfg = conf if isinstance(conf, DecoderConfig) else config_from_hf(conf)
        model = cls(cfg, dtype=dtype, device=device, init_seed=None)
        with torch.no_grad():
            hf_to_flat_views(cfg, sd, model.views(model.flat.data))
        return model

    def to_hf_state_dict(self) -> dict[str, torch.Tensor]:
        return flat_views_to_hf(self.cfg, self.views(self.flat.data))

    def save_pretrained(self, path: str, safe_serialization: bool = True) -> None:
        import dataclasses
        import json
        import os
        os.makedirs(path, exist_ok=True)
        sd = {k: v.detach().cpu().contiguous().clone() for k, v in self.to_hf_state_dict().items()}
        if safe_serialization:
            from safetensors.torch import save_file
            save_file(sd, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
        else:
            torch.save(sd, os.path.join(path, "pytorch_model.bin"))
        with open(os.path.join(path, "native_config.json"), "w", encoding="utf-8") as f:
            json.dump(dataclasses.asdict(self.cfg), f, indent=2, sort_keys=True)

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.float32, device=None) -> "NativeCausalLM":
        import json
        import os
        with open(os.path.join(path, "native_config.json"), encoding="utf-8") as f:
            cfg = DecoderConfig(**json.load(f))
        st = os.path.join(path, "model.safetensors")
        if os.path.exists(st):
            from safetensors.torch import load_file
            sd = load_file(st)
        else:
            sd = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True)
        return cls.from_hf(sd, cfg, dtype=dtype, device=device)


# ---------------------------------------------------------------------------------------------- config mapping
def config_from_hf(conf: Any) -> DecoderConfig:
    """Maps a Hugging Face config (Llama-like families and GPT-2) to a ``DecoderConfig``."""
    get = (lambda k, d=None: conf.get(k, d)) if isinstance(conf, Mapping) else (lambda k, d=None: getattr(conf, k, d))
    mt = get("model_type", "llama")
    if mt == "gpt2":
        d, L, H = get("n_embd"), get("n_layer"), get("n_head")
        return DecoderConfig(name="gpt2", vocab_size=get("vocab_size"), d_model=d, n_layers=L, n_heads=H, n_kv_heads=H,
                             head_dim=d // H, ffn=get("n_inner") or 4 * d, max_seq=get("n_positions", 1024), norm="layer",
                             norm_eps=get("layer_norm_epsilon", 1e-5), act="gelu", pos="learned", tie_embeddings=True,
                             bias=True, family="gpt2")
    d, H = get("hidden_size"), get("num_attention_heads")
    act = get("hidden_act", get("hidden_activation", "silu"))
    return DecoderConfig(
        name=mt, vocab_size=get("vocab_size"), d_model=d, n_layers=get("num_hidden_layers"), n_heads=H,
        n_kv_heads=get("num_key_value_heads") or H, head_dim=get("head_dim") or d // H, ffn=get("intermediate_size"),
        max_seq=get("max_position_embeddings", 2048), norm="rms", norm_eps=get("rms_norm_eps", 1e-5),
        act="geglu" if "gelu" in str(act) else "swiglu", pos="rope", rope_theta=float(get("rope_theta", 10000.0) or 10000.0),
        rope_scaling=get("rope_scaling"), tie_embeddings=bool(get("tie_word_embeddings", False)), bias=False,
        n_experts=int(get("num_local_experts", get("num_experts", 0)) or 0), top_k=int(get("num_experts_per_tok", 0) or 0),
        expert_ffn=int(get("moe_intermediate_size", get("intermediate_size", 0)) or 0) if get("num_local_experts", get("num_experts", 0)) else 0,
        norm_topk_prob=bool(get("norm_topk_prob", False)),
        qk_norm=True if mt == "olmoe" else ("head" if mt in ("qwen3", "qwen3_moe") else False),
        qkv_bias=(mt == "qwen2") or (mt in ("qwen3", "qwen3_moe") and bool(get("attention_bias", False))), family=mt)


def _interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])


def hf_to_flat_views(cfg: DecoderConfig, sd: Mapping[str, torch.Tensor], w: dict[str, torch.Tensor]) -> None:
    """Copies a Hugging Face state dict into the flat views ``w`` (in place)."""
    def put(name, t):
        w[name].copy_(t.to(w[name].dtype).reshape(w[name].shape))

    if cfg.family == "gpt2":
        pre = "transformer." if any(k.startswith("transformer.") for k in sd) else ""
        put("embed", sd[pre + "wte.weight"])
        put("wpe", sd[pre + "wpe.weight"][: cfg.max_seq])
        for i in range(cfg.n_layers):
            s, p = f"{pre}h.{i}.", f"layers.{i}."
            put(p + "norm1.weight", sd[s + "ln_1.weight"]); put(p + "norm1.bias", sd[s + "ln_1.bias"])
            put(p + "norm2.weight", sd[s + "ln_2.weight"]); put(p + "norm2.bias", sd[s + "ln_2.bias"])
            put(p + "wqkv", sd[s + "attn.c_attn.weight"].T); put(p + "bqkv", sd[s + "attn.c_attn.bias"])   # Conv1D: [in, out]
            put(p + "wo", sd[s + "attn.c_proj.weight"].T); put(p + "bo", sd[s + "attn.c_proj.bias"])
            put(p + "wfc", sd[s + "mlp.c_fc.weight"].T); put(p + "bfc", sd[s + "mlp.c_fc.bias"])
            put(p + "wproj", sd[s + "mlp.c_proj.weight"].T); put(p + "bproj", sd[s + "mlp.c_proj.bias"])
        put("norm_f.weight", sd[pre + "ln_f.weight"]); put("norm_f.bias", sd[pre + "ln_f.bias"])
        return
    pre = "model." if any(k.startswith("model.") for k in sd) else ""
    put("embed", sd[pre + "embed_tokens.weight"])
    if not cfg.tie_embeddings:
        put("lm_head", sd.get("lm_head.weight", sd[pre + "embed_tokens.weight"]))
    for i in range(cfg.n_layers):
        s, p = f"{pre}layers.{i}.", f"layers.{i}."
        put(p + "norm1.weight", sd[s + "input_layernorm.weight"])
        put(p + "norm2.weight", sd[s + "post_attention_layernorm.weight"])
        put(p + "wqkv", torch.cat([sd[s + "self_attn.q_proj.weight"], sd[s + "self_attn.k_proj.weight"],
                                   sd[s + "self_attn.v_proj.weight"]], dim=0))
        put(p + "wo", sd[s + "self_attn.o_proj.weight"])
        if cfg.qkv_bias:
            put(p + "bqkv", torch.cat([sd[s + "self_attn.q_proj.bias"], sd[s + "self_attn.k_proj.bias"],
                                       sd[s + "self_attn.v_proj.bias"]], dim=0))
        if cfg.qk_norm:
            put(p + "q_norm.weight", sd[s + "self_attn.q_norm.weight"])
            put(p + "k_norm.weight", sd[s + "self_attn.k_norm.weight"])
        if cfg.n_experts:
            put(p + "router", sd[s + "mlp.gate.weight"] if s + "mlp.gate.weight" in sd else sd[s + "block_sparse_moe.gate.weight"])
            for e in range(cfg.n_experts):
                ep = f"{s}mlp.experts.{e}."
                w[p + "experts.wgu"][e].copy_(_interleave(sd[ep + "gate_proj.weight"], sd[ep + "up_proj.weight"]).to(w[p + "experts.wgu"].dtype))
                w[p + "experts.wd"][e].copy_(sd[ep + "down_proj.weight"].to(w[p + "experts.wd"].dtype))
        else:
            put(p + "wgu", _interleave(sd[s + "mlp.gate_proj.weight"], sd[s + "mlp.up_proj.weight"]))
            put(p + "wd", sd[s + "mlp.down_proj.weight"])
    put("norm_f.weight", sd[pre + "norm.weight"])


def flat_views_to_hf(cfg: DecoderConfig, w: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Inverse of ``hf_to_flat_views``: a state dict loadable by the matching Hugging Face class."""
    out: dict[str, torch.Tensor] = {}
    H, KV, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    if cfg.family == "gpt2":
        out["transformer.wte.weight"] = w["embed"]
        out["transformer.wpe.weight"] = w["wpe"]
        for i in range(cfg.n_layers):
            s, p = f"transformer.h.{i}.", f"layers.{i}."
            out[s + "ln_1.weight"], out[s + "ln_1.bias"] = w[p + "norm1.weight"], w[p + "norm1.bias"]
            out[s + "ln_2.weight"], out[s + "ln_2.bias"] = w[p + "norm2.weight"], w[p + "norm2.bias"]
            out[s + "attn.c_attn.weight"], out[s + "attn.c_attn.bias"] = w[p + "wqkv"].T, w[p + "bqkv"]
            out[s + "attn.c_proj.weight"], out[s + "attn.c_proj.bias"] = w[p + "wo"].T, w[p + "bo"]
            out[s + "mlp.c_fc.weight"], out[s + "mlp.c_fc.bias"] = w[p + "wfc"].T, w[p + "bfc"]
            out[s + "mlp.c_proj.weight"], out[s + "mlp.c_proj.bias"] = w[p + "wproj"].T, w[p + "bproj"]
        out["transformer.ln_f.weight"], out["transformer.ln_f.bias"] = w["norm_f.weight"], w["norm_f.bias"]
        out["lm_head.weight"] = w["embed"]
        return out
    out["model.embed_tokens.weight"] = w["embed"]
    out["lm_head.weight"] = w["embed"] if cfg.tie_embeddings else w["lm_head"]
    for i in range(cfg.n_layers):
        s, p = f"model.layers.{i}.", f"layers.{i}."
        out[s + "input_layernorm.weight"] = w[p + "norm1.weight"]
        out[s + "post_attention_layernorm.weight"] = w[p + "norm2.weight"]
        qkv = w[p + "wqkv"]
        out[s + "self_attn.q_proj.weight"] = qkv[: H * hd]
        out[s + "self_attn.k_proj.weight"] = qkv[H * hd:(H + KV) * hd]
        out[s + "self_attn.v_proj.weight"] = qkv[(H + KV) * hd:]
        out[s + "self_attn.o_proj.weight"] = w[p + "wo"]
        if cfg.qkv_bias:
            b = w[p + "bqkv"]
            out[s + "self_attn.q_proj.bias"], out[s + "self_attn.k_proj.bias"] = b[: H * hd], b[H * hd:(H + KV) * hd]
            out[s + "self_attn.v_proj.bias"] = b[(H + KV) * hd:]
        if cfg.qk_norm:
            out[s + "self_attn.q_norm.weight"] = w[p + "q_norm.weight"]
            out[s + "self_attn.k_norm.weight"] = w[p + "k_norm.weight"]
        if cfg.n_experts:
            out[s + "mlp.gate.weight"] = w[p + "router"]
            for e in range(cfg.n_experts):
                ep = f"{s}mlp.experts.{e}."
                out[ep + "gate_proj.weight"], out[ep + "up_proj.weight"] = w[p + "experts.wgu"][e][0::2], w[p + "experts.wgu"][e][1::2]
                out[ep + "down_proj.weight"] = w[p + "experts.wd"][e]
        else:
            out[s + "mlp.gate_proj.weight"], out[s + "mlp.up_proj.weight"] = w[p + "wgu"][0::2], w[p + "wgu"][1::2]
            out[s + "mlp.down_proj.weight"] = w[p + "wd"]
    out["model.norm.weight"] = w["norm_f.weight"]
    return out
