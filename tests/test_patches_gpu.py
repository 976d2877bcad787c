"""CUDA paths added for the generic (vmap) route: multi-tensor clip-and-sum, vmap-safe kernel wrappers, fused linear
cross-entropy, and the trainer's native engine path."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_fused_clip_sum_matches_portable_path(cuda):
    from opake_b200.engine.clipping import numerics as N
    from opake_b200.ops.clip_sum import fused_clip_sum
    torch.manual_seed(0)
    B = 9
    leaves = [(torch.randn(B, 300, 70, device=cuda) * 0.05).to(torch.bfloat16), torch.randn(B, 5000, device=cuda) * 0.02,
              (torch.randn(B, 17, device=cuda)).to(torch.bfloat16)]
    leaves[0][3] *= 40.0            # one example far above the bound
    leaves[1][5, 7] = float("nan")  # sanitised to zero
    C = 1.5
    sums, norms, mask, post = fused_clip_sum(leaves, C, with_postsq=True)
    clean = [N.sanitize(l) for l in leaves]
    sq = sum(N.per_example_sq(l, torch.float64) for l in clean)
    fac, rn, rmask = N.clip_factors(sq, C, clean)
    assert torch.allclose(norms, rn, rtol=1e-12) and torch.equal(mask, rmask)
    for s, l, f in zip(sums, clean, fac):
        want = N.scale_leaf(l, f).sum(0, dtype=torch.float32)
        assert torch.allclose(s, want, rtol=1e-5, atol=1e-6)
    want_post = torch.sqrt(sum(N.per_example_sq(N.scale_leaf(l, f), torch.float64) for l, f in zip(clean, fac)))
    assert torch.allclose(post, want_post, rtol=1e-9) and (post <= C * (1 + 1e-9)).all()


def test_clipped_grad_uses_fused_backend(cuda):
    from opake_b200 import patches
    from opake_b200.dpsgd.clipping import clipped_grad
    from opake_b200.engine.clipping import kernel_backend
    torch.manual_seed(0)
    w = {"a": torch.randn(64, 32, device=cuda), "b": torch.randn(32, device=cuda)}
    x = torch.randn(12, 64, device=cuda)
    loss = lambda p, xe: ((xe @ p["a"] + p["b"]) ** 2).sum()
    saved = kernel_backend.get_fused_clip_backend()
    try:
        kernel_backend.register_fused_clip_backend(None)
        fn, st = clipped_grad(loss, clipping_norm=1.0, normalize_by=12.0)
        ref, _ = fn(w, x, state=st)
        patches.apply_runtime_patches()
        fn2, st2 = clipped_grad(loss, clipping_norm=1.0, normalize_by=12.0)
        got, _ = fn2(w, x, state=st2)
    finally:
        kernel_backend.register_fused_clip_backend(saved)
    for k in w:
        assert torch.allclose(got.pytree[k], ref.pytree[k], rtol=1e-5, atol=1e-7), k


def test_rowwise_wrappers_under_vmap_grad(cuda):
    from opake_b200.patches.kernels import opake_cross_entropy, opake_geglu, opake_rms_norm, opake_swiglu
    torch.manual_seed(0)
    B, T, D = 3, 40, 64
    x = (torch.randn(B, T, D, device=cuda) * 0.8).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, device=cuda)).to(torch.bfloat16)
    u = (torch.randn(B, T, D, device=cuda) * 0.8).to(torch.bfloat16)
    lab = torch.randint(0, D, (B, T), device=cuda)
    lab[0, :5] = -100

    def model(norm, glu, ce):
        def f(w_, xe, ue, le):
            h = norm(xe, w_)
            return ce(glu(h, ue), le).sum()
        return f

    ours = model(lambda a, b: opake_rms_norm(a, b, 1e-6), opake_swiglu, opake_cross_entropy)
    ref = model(lambda a, b: (a.float() * torch.rsqrt(a.float().pow(2).mean(-1, keepdim=True) + 1e-6) * b.float()),
                lambda g, v: F.silu(g.float()) * v.float(),
                lambda z, l: F.cross_entropy(z.float(), l, ignore_index=-100, reduction="none"))
    g1 = torch.func.vmap(torch.func.grad(ours, argnums=(0, 1)), in_dims=(None, 0, 0, 0))(w, x, u, lab)
    g2 = torch.func.vmap(torch.func.grad(ref, argnums=(0, 1)), in_dims=(None, 0, 0, 0))(w.float(), x.float(), u.float(), lab)
    for a, b in zip(g1, g2):
        assert a.shape == b.shape
        assert (a.float() - b).abs().max() <= 4e-2 * b.abs().max() + 1e-3
    a = opake_geglu(x, u).float()
    assert (a - F.gelu(x.float(), approximate="tanh") * u.float()).abs().max() < 5e-2


def test_fused_add_rms_norm_under_vmap_grad(cuda):
    """One-kernel ``s = x + r; y = rmsnorm(s)`` with the residual gradient folded into the norm backward, under
    ``vmap(grad)``: per-example weight gradients come from the per-example reduction kernel."""
    from opake_b200.patches.kernels import opake_fused_add_rms_norm
    torch.manual_seed(1)
    B, T, D = 4, 50, 128
    x = (torch.randn(B, T, D, device=cuda) * 0.7).to(torch.bfloat16)
    r = (torch.randn(B, T, D, device=cuda) * 0.7).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, device=cuda)).to(torch.bfloat16)
    t1 = torch.randn(T, D, device=cuda)
    t2 = torch.randn(T, D, device=cuda)

    def ours(w_, xe, re):
        y, s = opake_fused_add_rms_norm(xe, re, w_, 1e-6)
        return (y.float() * t1).sum() + (s.float() * t2).sum()

    def ref(w_, xe, re):
        s = xe + re
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w_
        return (y * t1).sum() + (s * t2).sum()

    g1 = torch.func.vmap(torch.func.grad(ours, argnums=(0, 1, 2)), in_dims=(None, 0, 0))(w, x, r)
    g2 = torch.func.vmap(torch.func.grad(ref, argnums=(0, 1, 2)), in_dims=(None, 0, 0))(w.float(), x.float(), r.float())
    for a, b in zip(g1, g2):
        assert a.shape == b.shape
        assert (a.float() - b).abs().max() <= 4e-2 * b.abs().max() + 1e-3
    # un-batched call
    y, s = opake_fused_add_rms_norm(x[0], r[0], w, 1e-6)
    sf = x[0].float() + r[0].float()
    assert (s.float() - sf).abs().max() <= 2 ** -7 * sf.abs().max()
    yf = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (y.float() - yf).abs().max() <= 3e-2 * yf.abs().max()


def test_linear_cross_entropy_native_matches_portable(cuda):
    from opake_b200.ops.lce import linear_cross_entropy
    torch.manual_seed(0)
    T, D, V = 300, 128, 1000
    h = (torch.randn(T, D, device=cuda) * 0.5).to(torch.bfloat16).requires_grad_()
    W = (torch.randn(V, D, device=cuda) * 0.1).to(torch.bfloat16).requires_grad_()
    lab = torch.randint(0, V, (T,), device=cuda)
    lab[:20] = -1
    got = linear_cross_entropy(h, W, lab)
    got.sum().backward()
    gh, gw = h.grad.clone(), W.grad.clone()
    h.grad = W.grad = None
    want = linear_cross_entropy(h, W, lab, force_portable=True)
    want.sum().backward()
    assert torch.allclose(got, want, atol=3e-2, rtol=1e-2)
    assert (gh.float() - h.grad.float()).abs().max() < 3e-2 * h.grad.float().abs().max() + 1e-3
    assert (gw.float() - W.grad.float()).abs().max() < 3e-2 * W.grad.float().abs().max() + 1e-3
    # per-example weight gradients under vmap
    hb = h.detach().view(3, 100, D)
    lb = lab.view(3, 100)
    f = lambda W_, he, le: linear_cross_entropy(he, W_, le).sum()
    gb = torch.func.vmap(torch.func.grad(f), in_dims=(None, 0, 0))(W.detach(), hb, lb)
    fp = lambda W_, he, le: linear_cross_entropy(he, W_, le, force_portable=True).sum()
    gp = torch.func.vmap(torch.func.grad(fp), in_dims=(None, 0, 0))(W.detach(), hb, lb)
    assert gb.shape == (3, V, D) and (gb.float() - gp.float()).abs().max() < 3e-2 * gp.float().abs().max() + 1e-3


def test_trainer_native_engine_path(cuda, tmp_path):
    from opake_b200.models.config import tiny_llama
    from opake_b200.models.native import NativeCausalLM
    from opake_b200.transformers import SFTConfig, SFTTrainer
    cfg = tiny_llama()

    class LM(torch.utils.data.Dataset):
        def __len__(self):
            return 64

        def __getitem__(self, i):
            g = torch.Generator().manual_seed(i)
            return {"input_ids": torch.randint(0, cfg.vocab_size, (64,), generator=g).tolist()}

    m = NativeCausalLM(cfg, dtype=torch.bfloat16, device=cuda)
    before = m.flat.detach().clone()
    a = SFTConfig(output_dir=str(tmp_path), per_device_train_batch_size=8, max_steps=3, privacy_noise_multiplier=0.8, save_steps=3,
                  max_length=64, learning_rate=1e-3, logging_steps=1, native_engine=True, optim="adamw-bc")
    tr = SFTTrainer(m, a, train_dataset=LM())
    out = tr.train()
    assert tr._native is not None and out.global_step == 3 and out.metrics["train_loss"] > 0
    assert not torch.equal(before, m.flat.detach())
    assert (tmp_path / "checkpoint-3" / "native_engine_rank0.pt").exists()
