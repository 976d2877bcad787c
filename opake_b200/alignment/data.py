"""Chat-template data preparation shared by SFT and DPO (packages/opake-alignment/src/opake/api/alignment/data/
_chat_template.py:41-588, _completion_mask.py:22-142).

``get_training_chat_template`` makes a tokenizer's Jinja chat template usable for completion-only loss by putting
``{% generation %}`` / ``{% endgeneration %}`` markers around what the assistant says. Instead of one rewrite rule
per known template family, this implementation enumerates candidate rewrites (every expression that prints message
content, wrapped plainly or behind an ``assistant`` role guard), renders each candidate on a probe conversation with
a span-recording Jinja extension, and accepts the first whose marked spans contain the assistant probe text and none
of the system or user probe text. A template that cannot be validated raises instead of guessing.
"""
from __future__ import annotations

import re
from typing import Any

import torch

from ..base.exceptions import ConfigurationError

__all__ = ["SyntheticLM", "SyntheticPreferences", "apply_chat_template_with_mask", "clone_chat_template", "get_training_chat_template"]

_GEN_START, _GEN_END = "{% generation %}", "{% endgeneration %}"
_MARKER_RE = re.compile(r"\{%-?\s*generation\s*-?%\}")
_PROBE = [
    {"role": "system", "content": "SYSPROBE-7c1"},
    {"role": "user", "content": "USERPROBE-a92"},
    {"role": "assistant", "content": "ASSTPROBE-e04"},
    {"role": "user", "content": "USERPROBE-b13"},
    {"role": "assistant", "content": "ASSTPROBE-f55"},
]


def _has_generation_marker(template: str) -> bool:
    return bool(_MARKER_RE.search(template))


def _resolve_chat_template(tokenizer, chat_template: str | None = None, tools=None) -> str:
    if chat_template is not None and ("{" in chat_template):
        return chat_template
    tpl = getattr(tokenizer, "chat_template", None)
    if isinstance(tpl, dict):                      # named templates
        name = chat_template or ("tool_use" if tools and "tool_use" in tpl else "default")
        tpl = tpl.get(name)
    if not tpl:
        raise ConfigurationError("tokenizer.chat_template is not set. Assign a Jinja2 template string first.")
    return tpl


def _render_with_spans(template: str, messages, **ctx) -> tuple[str, list[tuple[int, int]]]:
    """Renders ``template`` and returns the text plus the character spans produced inside generation blocks."""
    import jinja2
    from jinja2.ext import Extension
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    spans: list[tuple[int, int]] = []

    class _Generation(Extension):
        tags = {"generation"}

        def parse(self, parser):
            lineno = next(parser.stream).lineno
            body = parser.parse_statements(["name:endgeneration"], drop_needle=True)
            return jinja2.nodes.CallBlock(self.call_method("_mark"), [], [], body).set_lineno(lineno)

        def _mark(self, caller):
            text = caller()
            return "\x00G" + text + "\x00E"

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=[_Generation])
    env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(jinja2.exceptions.TemplateError(msg))
    env.globals["strftime_now"] = lambda fmt: "1970-01-01"
    env.filters.setdefault("tojson", lambda x, **kw: __import__("json").dumps(x, **kw))
    raw = env.from_string(template).render(messages=messages, add_generation_prompt=False, **ctx)
    out, depth_start, i = [], None, 0
    n = 0
    while i < len(raw):
        if raw.startswith("\x00G", i):
            depth_start = n
            i += 2
        elif raw.startswith("\x00E", i):
            if depth_start is not None:
                spans.append((depth_start, n))
            depth_start = None
            i += 2
        else:
            out.append(raw[i])
            n += 1
            i += 1
    return "".join(out), spans


def _special_token_context(tokenizer) -> dict:
    ctx = {}
    for name in ("bos_token", "eos_token", "pad_token", "unk_token"):
        ctx[name] = getattr(tokenizer, name, None) or ""
    return ctx


def _marks_only_assistant(template: str, tokenizer) -> bool:
    try:
        text, spans = _render_with_spans(template, _PROBE, **_special_token_context(tokenizer))
    except Exception:
        try:                                        # templates that reject a system turn
            text, spans = _render_with_spans(template, _PROBE[1:], **_special_token_context(tokenizer))
        except Exception:
            return False
    marked = "".join(text[a:b] for a, b in spans)
    if "ASSTPROBE-e04" not in marked or "ASSTPROBE-f55" not in marked:
        return False
    return not any(p in marked for p in ("SYSPROBE-7c1", "USERPROBE-a92", "USERPROBE-b13"))


_EXPR_RE = re.compile(r"\{\{-?[^{}]*?-?\}\}")


def _candidates(template: str):
    """Candidate rewrites, most specific first."""
    token_expr = "{{ generation_token }}"
    if token_expr in template:
        yield template.replace(token_expr, f"{_GEN_START}{token_expr}{_GEN_END}", 1)
    exprs = [m for m in _EXPR_RE.finditer(template) if re.search(r"\bcontent\b|\bmessage\b|\bmsg\b", m.group(0))]
    # plain wrap of one expression (assistant-only branches), last occurrence first
    for m in reversed(exprs):
        yield template[:m.start()] + _GEN_START + m.group(0) + _GEN_END + template[m.end():]
    # role-guarded wrap (templates that print every role through one shared expression)
    for var in ("message", "msg", "m"):
        if not re.search(rf"\b{var}\b", template):
            continue
        for m in reversed(exprs):
            guard = (f"{{% if {var}['role'] == 'assistant' %}}{_GEN_START}{m.group(0)}{_GEN_END}"
                     f"{{% else %}}{m.group(0)}{{% endif %}}")
            yield template[:m.start()] + guard + template[m.end():]


def get_training_chat_template(tokenizer) -> str:
    """Returns the tokenizer's chat template with validated assistant-only generation markers (idempotent)."""
    template = _resolve_chat_template(tokenizer)
    if _has_generation_marker(template):
        if _marks_only_assistant(template, tokenizer):
            return template
        raise ConfigurationError("get_training_chat_template: existing generation markers do not identify a "
                                 "validated assistant-only render path; ensure they exclude system and user content.")
    for cand in _candidates(template):
        if _marks_only_assistant(cand, tokenizer):
            return cand
    raise ConfigurationError("get_training_chat_template: could not identify and validate an assistant-only render "
                             "path in the chat template. Provide a template with explicit '{% generation %}' / "
                             "'{% endgeneration %}' markers.")


def clone_chat_template(model, tokenizer, source_tokenizer_or_path):
    """Copies chat template and missing special tokens from a source tokenizer; resizes the model's embeddings.
    Returns ``(model, tokenizer, added_token_ids)``. Call before taking any functional snapshot of the parameters."""
    source = source_tokenizer_or_path
    if isinstance(source, str):
        from transformers import AutoTokenizer
        source = AutoTokenizer.from_pretrained(source, trust_remote_code=False)
    tokenizer.chat_template = source.chat_template
    have = set(tokenizer.get_vocab())
    new = [str(tok) for tok in getattr(source, "added_tokens_decoder", {}).values()
           if getattr(tok, "special", False) and str(tok) not in have]
    if new:
        tokenizer.add_special_tokens({"additional_special_tokens": new}, replace_additional_special_tokens=False)
    for name in ("bos_token", "eos_token", "pad_token"):
        if getattr(tokenizer, name, None) is None and getattr(source, name, None) is not None:
            setattr(tokenizer, name, getattr(source, name))
    model.resize_token_embeddings(len(tokenizer))
    return model, tokenizer, [tokenizer.convert_tokens_to_ids(t) for t in new]


def apply_chat_template_with_mask(tokenizer, conversation: list[dict[str, Any]], **kwargs: Any) -> dict[str, Any]:
    """Tokenizes a conversation and returns ``input_ids`` plus ``completion_mask`` (1 on assistant tokens)."""
    active = _resolve_chat_template(tokenizer, chat_template=kwargs.get("chat_template"), tools=kwargs.get("tools"))
    hint = ("Install the markers first:\n\n    tokenizer.chat_template = get_training_chat_template(tokenizer)\n")
    if not _has_generation_marker(active):
        raise ConfigurationError("apply_chat_template_with_mask: the active chat template has no '{% generation %}' / "
                                 "'{% endgeneration %}' markers, so no assistant-token mask can be produced. " + hint)
    enc = tokenizer.apply_chat_template(conversation, tokenize=True, return_assistant_tokens_mask=True,
                                        return_dict=True, **kwargs)
    masks = enc.get("assistant_masks")
    empty = masks is None or not (bool(masks.any()) if hasattr(masks, "any") else any(masks))
    if empty:
        raise ConfigurationError("apply_chat_template_with_mask: the tokenizer returned no assistant-token mask. " + hint)
    out = {"input_ids": enc["input_ids"], "completion_mask": masks}
    if enc.get("attention_mask") is not None:
        out["attention_mask"] = enc["attention_mask"]
    return out


# ------------------------------------------------------------------------------------------------ synthetic data
class SyntheticLM(torch.utils.data.Dataset):
    """Zipf-distributed token sequences with a completion mask on the last 75 % of every sequence."""

    def __init__(self, n: int, vocab: int, seq: int, seed: int = 0):
        self.n, self.vocab, self.seq, self.seed = n, vocab, seq, seed
        ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
        self.p = (ranks ** -1.1 / (ranks ** -1.1).sum()).float()
        self._fingerprint = f"synthetic-lm-{n}-{vocab}-{seq}-{seed}"

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.multinomial(self.p, self.seq, replacement=True, generator=g).tolist()
        cut = self.seq // 4
        return {"input_ids": ids, "completion_mask": [0] * cut + [1] * (self.seq - cut)}


class SyntheticPreferences(torch.utils.data.Dataset):
    def __init__(self, n: int, vocab: int, prompt: int = 16, completion: int = 16, seed: int = 0):
        self.n, self.vocab, self.prompt, self.completion, self.seed = n, vocab, prompt, completion, seed
        self._fingerprint = f"synthetic-pref-{n}-{vocab}-{prompt}-{completion}-{seed}"

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        p, c, r = (torch.randint(0, self.vocab, (k,), generator=g).tolist() for k in (self.prompt, self.completion, self.completion))
        return {"chosen_input_ids": p + c, "rejected_input_ids": p + r, "chosen_completion_mask": [0] * len(p) + [1] * len(c),
                "rejected_completion_mask": [0] * len(p) + [1] * len(r)}
