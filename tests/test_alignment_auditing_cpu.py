"""Alignment losses / collators / log-probabilities and the auditing package (CPU)."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F


def test_sft_losses_match_manual():
    from opake_b200.alignment.sft import dft_loss, fused_dft_loss, fused_nll_loss, nll_loss
    torch.manual_seed(0)
    h, W = torch.randn(3, 9, 16), torch.randn(40, 16)
    lab = torch.randint(0, 40, (3, 9))
    lab[0, :4] = -100
    logits = h @ W.t()
    lp = logits[:, :-1].log_softmax(-1).gather(-1, lab[:, 1:].clamp(min=0)[..., None])[..., 0]
    m = (lab[:, 1:] != -100).float()
    want = -(lp * m).sum(-1) / m.sum(-1)
    assert torch.allclose(nll_loss(logits, lab), want, atol=1e-5)
    assert torch.allclose(fused_nll_loss(h, W, lab), want, atol=1e-4)
    want_dft = -(lp.exp() * lp * m).sum(-1) / m.sum(-1)
    assert torch.allclose(dft_loss(logits, lab), want_dft, atol=1e-5)
    assert torch.allclose(fused_dft_loss(h, W, lab), want_dft, atol=1e-4)
    # the DFT weight is detached: gradient equals p * d(nll)
    hh = h.clone().requires_grad_()
    dft_loss(hh @ W.t(), lab).sum().backward()
    assert hh.grad.abs().sum() > 0


def test_sequence_logp_and_ld_weighting():
    from opake_b200.alignment.dpo import fused_sequence_logp, ld_dpo_split, sequence_logp
    torch.manual_seed(1)
    h, W = torch.randn(2, 8, 12), torch.randn(30, 12)
    ids = torch.randint(0, 30, (2, 8))
    cm = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 0], [0, 1, 1, 1, 1, 1, 0, 0]])
    logits = h @ W.t()
    lp = logits[:, :-1].log_softmax(-1).gather(-1, ids[:, 1:, None])[..., 0]
    want = (lp * cm[:, 1:]).sum(-1)
    assert torch.allclose(sequence_logp(logits, ids, cm), want, atol=1e-5)
    assert torch.allclose(fused_sequence_logp(h, W, ids, cm), want, atol=1e-4)
    norm = sequence_logp(logits, ids, cm, length_normalized=True)
    assert torch.allclose(norm, want / cm[:, 1:].sum(-1), atol=1e-5)
    ld = sequence_logp(logits, ids, cm, ld_alpha=0.5, shared_prefix_len=2)
    w = torch.where(cm[:, 1:].cumsum(-1) <= 2, 1.0, 0.5) * cm[:, 1:]
    assert torch.allclose(ld, (lp * w).sum(-1), atol=1e-5)
    assert torch.allclose(ld_dpo_split(lp, cm[:, 1:], 2, 0.5), ld, atol=1e-5)


def test_dpo_heads_values():
    from opake_b200.alignment.dpo import loss as L
    c, r = torch.tensor([0.3, -0.2]), torch.tensor([-0.1, 0.4])
    z = 0.5 * (c - r)
    assert torch.allclose(L.sigmoid_loss(c, r, beta=0.5), -F.logsigmoid(z))
    assert torch.allclose(L.sigmoid_loss(c, r, beta=0.5, label_smoothing=0.1), -0.9 * F.logsigmoid(z) - 0.1 * F.logsigmoid(-z))
    assert torch.allclose(L.hinge_loss(c, r, beta=0.5), torch.relu(1 - z))
    assert torch.allclose(L.ipo_loss(c, r, beta=0.5), (c - r - 1.0) ** 2)
    assert torch.allclose(L.sppo_loss(c, r, beta=0.5), (c - 1.0) ** 2 + (r + 1.0) ** 2)
    assert torch.allclose(L.robust_loss(c, r, beta=0.5, label_smoothing=0.1), (-0.9 * F.logsigmoid(z) + 0.1 * F.logsigmoid(-z)) / 0.8)
    assert torch.allclose(L.apo_zero_loss(c, r, beta=0.5), 1 - torch.sigmoid(0.5 * c) + torch.sigmoid(0.5 * r))
    assert torch.allclose(L.nca_loss(c, r, beta=1.0), -F.logsigmoid(c) - 0.5 * F.logsigmoid(-c) - 0.5 * F.logsigmoid(-r))
    assert torch.allclose(L.simpo_loss(c, r, beta=2.0, gamma=0.5), -F.logsigmoid(2 * (c - r) - 0.5))
    lp_c, lp_r = torch.tensor([-0.5, -1.0]), torch.tensor([-1.5, -0.7])
    odds = lambda p: p - torch.log1p(-p.exp())
    assert torch.allclose(L.odds_ratio_loss(lp_c, lp_r), -F.logsigmoid(odds(lp_c) - odds(lp_r)), atol=1e-6)
    assert torch.allclose(L.f_divergence_logits(c, r, f_divergence_type="js_divergence"), F.logsigmoid(c) - F.logsigmoid(r))
    assert torch.allclose(L.mpo_combine({"a": c, "b": r}, {"a": 1.0, "b": 0.5}), c + 0.5 * r)
    assert set(L.LOSS_HEADS) >= {"sigmoid", "hinge", "ipo", "robust", "exo_pair", "nca_pair", "bco_pair", "sppo_hard", "apo_zero",
                                 "apo_down", "discopop", "simpo", "orpo", "sft"}
    assert torch.isfinite(L.discopop_loss(torch.tensor([-500.0]), torch.tensor([0.0]), beta=1.0)).all()
    assert torch.isfinite(L.exo_loss(c, r, beta=0.5, label_smoothing=0.0)).all()


def test_collators():
    from opake_b200.alignment.dpo import preference_collator
    from opake_b200.alignment.sft import language_modeling_collator
    col = language_modeling_collator(0, 6, completion_only_loss=True, pad_to_multiple_of=4)
    b = col([{"input_ids": [5, 6, 7, 8, 9, 10, 11], "completion_mask": [0, 0, 1, 1, 1, 1, 1]}, {"input_ids": [3, 4]}])
    assert b["input_ids"].shape == (2, 8) and b["attention_mask"].sum().item() == 8
    assert b["labels"][0].tolist() == [-100, -100, 7, 8, 9, 10, -100, -100]
    assert b["labels"][1].tolist() == [3, 4] + [-100] * 6 and b["completion_mask"][1].tolist() == [1, 1, 0, 0, 0, 0, 0, 0]
    assert col([])["input_ids"].shape == (0, 0)
    pc = preference_collator(0, 5)
    ex = {"chosen_input_ids": [1, 2, 3], "rejected_input_ids": [1, 2, 4, 5, 6, 7], "chosen_completion_mask": [0, 1, 1],
          "rejected_completion_mask": [0, 1, 1, 1, 1, 1], "ref_chosen_logps": -1.0, "ref_rejected_logps": -2.0}
    out = pc([ex, ex])
    assert out["chosen_input_ids"].shape == (2, 3) and out["rejected_input_ids"].shape == (2, 5)
    assert out["ref_chosen_logps"].tolist() == [-1.0, -1.0]


def test_training_chat_template_markers():
    from opake_b200.alignment.data import get_training_chat_template
    from opake_b200.base.exceptions import ConfigurationError

    class Tok:
        bos_token, eos_token, pad_token, unk_token = "<s>", "</s>", None, None
        chat_template = ("{% for message in messages %}{{'<|im_start|>' + message['role'] + '\n' + message['content'] + "
                         "'<|im_end|>\n'}}{% endfor %}")
    t = get_training_chat_template(Tok())
    assert "{% generation %}" in t and t.count("{% generation %}") == 1
    Tok.chat_template = t
    assert get_training_chat_template(Tok()) == t          # idempotent
    Tok.chat_template = "{{ bos_token }}static text only"
    with pytest.raises(ConfigurationError):
        get_training_chat_template(Tok())


def test_coin_flip_and_one_run_estimators():
    from opake_b200.auditing import canary_scores, coin_flip, one_run
    from opake_b200.base.exceptions import ConfigurationError, InputTypeError
    from opake_b200.engine.random import key
    ds = list(range(1000))
    cf = coin_flip(ds, num_canaries=400, key=key(7))
    cf2 = coin_flip(ds, num_canaries=400, key=key(7))
    assert np.array_equal(cf.canary_indices, cf2.canary_indices) and np.array_equal(cf.in_indices, cf2.in_indices)
    assert len(set(cf.train_indices())) == 1000 - len(cf.out_indices)
    rng = np.random.default_rng(0)
    member = np.isin(cf.canary_indices, cf.in_indices)
    strong = canary_scores(rng.normal(size=400) + 3.0 * member, canary_indices=cf.canary_indices)
    null = canary_scores(rng.normal(size=400), canary_indices=cf.canary_indices)
    perm = rng.permutation(400)                # identifiers travel with the scores: order does not matter
    shuffled = canary_scores(strong.scores[perm], canary_indices=cf.canary_indices[perm])
    e1, e2, e0 = one_run(strong, coin_flip=cf), one_run(shuffled, coin_flip=cf), one_run(null, coin_flip=cf)
    assert e1.attack_auc() == pytest.approx(e2.attack_auc()) and e1.attack_auc() > 0.95 and abs(e0.attack_auc() - 0.5) < 0.1
    eps_strong = e1.eps_delta().epsilon_at(delta=1e-5)
    assert eps_strong > 1.0 and e0.eps_delta().epsilon_at(delta=1e-5) < 0.5
    assert e1.epsilon_at(delta=1e-5) > e0.epsilon_at(delta=1e-5)
    assert 0 <= e0.advantage() < e1.advantage() <= 1
    lo, hi = e1.attack_auc(confidence=0.9, num_samples=50, key=key(1))
    assert lo <= e1.attack_auc() <= hi + 1e-9
    with pytest.raises(InputTypeError):
        cf.split_scores(np.zeros(400))
    with pytest.raises(ConfigurationError):
        cf.split_scores(canary_scores(np.zeros(3), canary_indices=[1, 2, 3]))


def test_loss_and_gradient_scores_bind_identifiers():
    from opake_b200.auditing import coin_flip, gradient_scores, loss_scores
    from opake_b200.engine.random import key
    ds = torch.utils.data.TensorDataset(torch.randn(120, 4), torch.randn(120))
    cf = coin_flip(ds, num_canaries=50, key=key(3))
    w = torch.randn(4)
    fn = lambda w, x, y: ((x @ w) - y) ** 2
    s = loss_scores(fn, w, batch_argnums=(1, 2), coin_flip=cf, dataset=ds, batch_size=16)
    x, y = ds.tensors
    want = -((x[cf.canary_indices] @ w) - y[cf.canary_indices]) ** 2
    assert np.allclose(s.scores, want.numpy(), atol=1e-5) and np.array_equal(s.canary_indices, cf.canary_indices)
    g = gradient_scores(fn, w, batch_argnums=(1, 2), coin_flip=cf, dataset=ds, batch_size=16)
    gw = 2 * ((x[cf.canary_indices] @ w) - y[cf.canary_indices])[:, None] * x[cf.canary_indices]
    assert np.allclose(g.scores, -(gw ** 2).sum(-1).numpy(), rtol=1e-4)
    cal = loss_scores(fn, w, batch_argnums=(1, 2), coin_flip=cf, dataset=ds, reference_scores=s)
    assert np.allclose(cal.scores, 0.0, atol=1e-6)


def test_fused_lora_qkv_and_mlp_match_autograd_under_vmap():
    """The fused LoRA functions (three projections of one input; the adapted gated MLP) against plain autograd, both as
    ordinary calls and as per-example gradients under ``vmap(grad)``."""
    import torch
    import torch.nn.functional as F

    from opake_b200.patches.kernels.lora import lora_mlp, lora_qkv

    torch.manual_seed(0)
    n, T, d, r, f = 3, 5, 8, 2, 12
    x = torch.randn(n, T, d)

    def mk(o, i):
        return [torch.randn(o, i) * 0.3, torch.randn(r, i) * 0.3, torch.randn(o, r) * 0.3, 0.5]

    q, k, v = mk(d, d), mk(4, d), mk(4, d)
    gate, up, down = mk(f, d), mk(f, d), mk(d, f)
    adapters = {"q": (q[1], q[2]), "k": (k[1], k[2]), "v": (v[1], v[2]), "g": (gate[1], gate[2]), "u": (up[1], up[2]), "d": (down[1], down[2])}

    def plain(p, W, xx):
        return xx @ W[0].t() + W[3] * (xx @ p[0].t()) @ p[1].t()

    def loss_fused(ad, xe):
        qq, kk, vv = lora_qkv(xe, (q[0], *ad["q"], q[3]), (k[0], *ad["k"], k[3]), (v[0], *ad["v"], v[3]))
        y = lora_mlp(xe, (gate[0], *ad["g"], gate[3]), (up[0], *ad["u"], up[3]), (down[0], *ad["d"], down[3]))
        return (qq.sum() + (kk * vv).sum() + (y ** 2).sum())

    def loss_plain(ad, xe):
        qq, kk, vv = plain(ad["q"], q, xe), plain(ad["k"], k, xe), plain(ad["v"], v, xe)
        h = F.silu(plain(ad["g"], gate, xe)) * plain(ad["u"], up, xe)
        y = plain(ad["d"], down, h)
        return (qq.sum() + (kk * vv).sum() + (y ** 2).sum())

    assert torch.allclose(loss_fused(adapters, x[0]), loss_plain(adapters, x[0]), rtol=1e-5)
    g1 = torch.func.vmap(torch.func.grad(loss_fused), in_dims=(None, 0))(adapters, x)
    g2 = torch.func.vmap(torch.func.grad(loss_plain), in_dims=(None, 0))(adapters, x)
    for name in adapters:
        for a, b in zip(g1[name], g2[name]):
            assert a.shape == b.shape and torch.allclose(a, b, rtol=1e-4, atol=1e-5), name
    # input gradient of the un-batched call
    xr = x[0].clone().requires_grad_()
    loss_fused(adapters, xr).backward()
    gx = xr.grad.clone()
    xr.grad = None
    loss_plain(adapters, xr).backward()
    assert torch.allclose(gx, xr.grad, rtol=1e-4, atol=1e-5)
    # tanh-GELU gate
    y1 = lora_mlp(x[0], (gate[0], *adapters["g"], gate[3]), (up[0], *adapters["u"], up[3]), (down[0], *adapters["d"], down[3]), act="gelu_tanh")
    h = F.gelu(plain(adapters["g"], gate, x[0]), approximate="tanh") * plain(adapters["u"], up, x[0])
    assert torch.allclose(y1, plain(adapters["d"], down, h), rtol=1e-5, atol=1e-6)
