"""Bandwidth-bound kernels and DP primitives against fp32 PyTorch / NumPy references."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, dev, scale=1.0):
    return (torch.randn(shape, device=dev) * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    assert (a - b).abs().max().item() <= tol * (b.abs().max().item() + 1e-6)


@pytest.mark.parametrize("T,D", [(300, 1024), (77, 4096), (130, 2048), (65, 768)])
def test_rmsnorm_fwd_bwd(cuda, T, D):
    """Widths 1024 / 2048 / 4096 take the warp-per-row forward kernel, the others the block-per-row one."""
    from opake_b200.ops import kernels as K

    x, w, dy, dres = _rand((T, D), cuda), _rand((D,), cuda), _rand((T, D), cuda), _rand((T, D), cuda)
    y, rstd = K.rmsnorm_fwd(x, w, eps=1e-5)
    xf = x.float().requires_grad_()
    wf = w.float().requires_grad_()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    _close(y, ref)
    ref.backward(dy.float())
    dw = torch.zeros(D, device=cuda)
    dx = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres, dw=dw)
    _close(dx, xf.grad + dres.float())
    _close(dw, wf.grad)
    s, y2, _ = K.add_rmsnorm_fwd(x, dres, w, eps=1e-5)
    _close(s, x.float() + dres.float())
    sf = s.float()
    _close(y2, sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())


def test_layernorm_fwd_bwd(cuda):
    from opake_b200.ops import kernels as K

    T, D = 130, 768
    x, w, b, dy = _rand((T, D), cuda), _rand((D,), cuda), _rand((D,), cuda), _rand((T, D), cuda)
    y, mean, rstd = K.layernorm_fwd(x, w, b)
    xf, wf, bf = x.float().requires_grad_(), w.float().requires_grad_(), b.float().requires_grad_()
    ref = torch.nn.functional.layer_norm(xf, (D,), wf, bf, 1e-5)
    _close(y, ref)
    ref.backward(dy.float())
    dw, db = torch.zeros(D, device=cuda), torch.zeros(D, device=cuda)
    dx = K.layernorm_bwd(dy, x, w, mean, rstd, dw=dw, db=db)
    _close(dx, xf.grad)
    _close(dw, wf.grad)
    _close(db, bf.grad)


def test_rope_roundtrip_and_reference(cuda):
    from opake_b200.ops import kernels as K

    T, H, hd = 64, 6, 128
    qk = _rand((T, H * hd + 256), cuda)
    orig = qk.clone()
    tab = K.rope_table(T, hd, 500000.0, device=cuda)
    K.rope_(qk, tab, H, hd)
    x = orig[:, : H * hd].float().view(T, H, hd)
    cos = torch.cat([tab[..., 0], tab[..., 0]], -1)[:, None, :]
    sin = torch.cat([tab[..., 1], tab[..., 1]], -1)[:, None, :]
    rot = torch.cat([-x[..., hd // 2:], x[..., : hd // 2]], -1)
    _close(qk[:, : H * hd].view(T, H, hd), x * cos + rot * sin)
    assert torch.equal(qk[:, H * hd:], orig[:, H * hd:])
    K.rope_(qk, tab, H, hd, backward=True)
    _close(qk, orig, 3e-2)


def test_swiglu_geglu_gelu(cuda):
    from opake_b200.ops import kernels as K

    T, F = 100, 512
    gu, dact = _rand((T, 2 * F), cuda), _rand((T, F), cuda)
    for fwd, bwd, fn in [
        (K.swiglu_fwd, K.swiglu_bwd, torch.nn.functional.silu),
        (lambda t: K.geglu_fwd(t, True), lambda d, t: K.geglu_bwd(d, t, True),
         lambda t: torch.nn.functional.gelu(t, approximate="tanh")),
        (lambda t: K.geglu_fwd(t, False), lambda d, t: K.geglu_bwd(d, t, False), torch.nn.functional.gelu),
    ]:
        guf = gu.float().requires_grad_()
        ref = fn(guf[:, 0::2]) * guf[:, 1::2]
        _close(fwd(gu), ref)
        ref.backward(dact.float())
        _close(bwd(dact, gu), guf.grad)
    x = _rand((1000,), cuda)
    xf = x.float().requires_grad_()
    ref = torch.nn.functional.gelu(xf, approximate="tanh")
    _close(K.gelu_fwd(x), ref)
    ref.backward(torch.ones_like(ref))
    _close(K.gelu_bwd(torch.ones_like(x), x), xf.grad)


def test_embedding_compact_grad(cuda):
    from opake_b200.ops import kernels as K

    V, T, D = 1000, 256, 128
    table = _rand((V, D), cuda)
    tok = torch.randint(0, 50, (T,), device=cuda, dtype=torch.int32)  # many collisions
    out = K.embedding_fwd(tok, table)
    assert torch.equal(out, table[tok.long()])
    dx = _rand((T, D), cuda)
    ws = K.EmbeddingGradWorkspace(V, T, D, cuda)
    ss = torch.zeros(1, dtype=torch.float64, device=cuda)
    K.embedding_bwd_compact(tok, dx, ws, ss)
    dense = torch.zeros(V, D, device=cuda).index_add_(0, tok.long(), dx.float())
    want = dense.to(torch.bfloat16).double().pow(2).sum().item()
    assert abs(ss.item() - want) / want < 1e-3
    assert (ws.first_pos == 2**31 - 1).all()
    acc = torch.zeros(V, D, device=cuda)
    scale = torch.tensor([0.5], device=cuda)
    K.embedding_accumulate(tok, ws, scale, acc, T)
    _close(acc, dense * 0.5, 1e-2)


def test_cross_entropy_rowwise(cuda):
    from opake_b200.ops import kernels as K

    T, V = 50, 3000
    logits = torch.randn(T, V, device=cuda) * 3
    labels = torch.randint(0, V, (T,), device=cuda, dtype=torch.int32)
    labels[::5] = -100
    nll, lse = K.cross_entropy_fwd(logits, labels, scale=0.5, softcap=30.0)
    z = 30.0 * torch.tanh(logits * 0.5 / 30.0)
    ref = torch.nn.functional.cross_entropy(z, labels.long(), ignore_index=-100, reduction="none")
    assert (nll - ref).abs().max().item() < 1e-3
    zf = logits.clone().requires_grad_()
    zz = 30.0 * torch.tanh(zf * 0.5 / 30.0)
    coef = (labels >= 0).float()
    (torch.nn.functional.cross_entropy(zz, labels.long(), ignore_index=-100, reduction="none") * coef).sum().backward()
    d = K.cross_entropy_bwd(logits, labels, lse, coef, scale=0.5, softcap=30.0)
    assert (d - zf.grad).abs().max().item() < 1e-4


def test_philox_matches_cpu_restatement_and_is_shard_invariant(cuda):
    from opake_b200.ops import kernels as K
    from opake_b200.ops.philox_ref import normal

    n, seed, step = 10007, 0x1234_5678_9ABC_DEF0, 7
    full = K.philox_normal_(torch.empty(n, device=cuda), seed, step, sigma=1.0)
    ref = normal(n, seed, step)
    assert np.abs(full.cpu().numpy() - ref).max() < 1e-4
    # any shard of the global index space reproduces the same values (exactly-once noise under sharding)
    part = K.philox_normal_(torch.empty(1001, device=cuda), seed, step, offset=3002, sigma=1.0)
    assert torch.equal(part, full[3002:4003])
    big = K.philox_normal_(torch.empty(4_000_000, device=cuda), seed, 3, sigma=2.0)
    assert abs(big.mean().item()) < 5e-3 and abs(big.std().item() - 2.0) < 5e-3
    from scipy import stats

    assert stats.kstest(big[:200000].cpu().numpy() / 2.0, "norm").pvalue > 1e-3


def test_clip_scale_and_accumulate(cuda):
    from opake_b200.ops import kernels as K

    n = 100003 * 8
    g = _rand((n,), cuda)
    ss = torch.zeros(1, dtype=torch.float64, device=cuda)
    K.sumsq_(g, ss)
    assert abs(ss.item() - g.double().pow(2).sum().item()) / ss.item() < 1e-7
    scale, norm = torch.empty(1, device=cuda), torch.empty(1, device=cuda)
    cnt = torch.zeros(1, dtype=torch.int32, device=cuda)
    K.clip_scale(ss, 1.0, scale_out=scale, norm_out=norm, counters=cnt, n_leaves=1, widest_leaf=n)
    assert ss.item() == 0.0 and cnt.item() == 1
    true_norm = g.double().norm().item()
    assert abs(norm.item() - true_norm) / true_norm < 1e-6
    s = scale.item()
    assert 0.99 / true_norm < s <= 1.0 / true_norm
    acc = torch.zeros(n, device=cuda)
    K.clip_accumulate(g, scale, acc, overwrite=True)
    K.clip_accumulate(g, scale, acc)
    stored = (g.float() * s).to(torch.bfloat16)
    assert stored.double().norm().item() <= 1.0  # the stored clipped gradient respects the bound
    assert torch.equal(acc, stored.float() * 2)
    # not clipped when the norm is below the bound
    K.sumsq_(g, ss)
    K.clip_scale(ss, 1e9, scale_out=scale, counters=cnt)
    assert scale.item() == 1.0 and cnt.item() == 1


@pytest.mark.parametrize("group", [1, 2, 3, 5, 8])
def test_clip_accumulate_group_equals_one_by_one(cuda, group):
    """One pass over the sums for a whole group of examples gives the sum of the individually stored clipped gradients."""
    from opake_b200.ops import kernels as K

    n = 100003 * 8 + 5                     # vector body plus a ragged tail
    gs = [_rand((n,), cuda) for _ in range(group)]
    scales = [torch.full((1,), 0.1 + 0.07 * j, device=cuda) for j in range(group)]
    acc = torch.randn(n, device=cuda)
    want = acc.clone()
    f = torch.zeros(n, device=cuda)
    for g, s in zip(gs, scales):
        ref = torch.zeros(n, device=cuda)
        K.clip_accumulate(g, s, ref, overwrite=True)     # stored(g * s) exactly as the single-example kernel rounds it
        f += ref
    want += f
    K.clip_accumulate_group(gs, scales, acc)
    assert torch.equal(acc, want)
    K.clip_accumulate_group(gs, scales, acc, overwrite=True)
    assert torch.equal(acc, f)


def test_dp_step_single_rank_matches_reference_math(cuda):
    from opake_b200.ops import kernels as K
    from opake_b200.ops.philox_ref import normal

    n, B = 4096 + 8, 16.0
    acc = torch.randn(n, device=cuda) * 16.0
    acc0 = acc.clone()
    p = _rand((n,), cuda, 0.05)
    p0 = p.clone()
    m, v = torch.zeros(n, device=cuda), torch.zeros(n, device=cuda)
    lr, b1, b2, eps, wd, sigma, seed, step = 1e-2, 0.9, 0.999, 1e-8, 0.01, 0.05, 99, 3
    phi = (1 - b2) * sigma**2
    K.dp_step(grad_src=[acc.data_ptr()], shard_begin=0, shard_len=n, inv_batch=1 / B, sigma=sigma, seed=seed, step=step,
              m=m, v=v, master=None, param_dst=[p.data_ptr()], param_src=p, lr=lr, beta1=b1, beta2=b2, eps=eps,
              weight_decay=wd, bc1=1 - b1, bc2=1 - b2, phi_hat=phi / (1 - b2), zero_grad=True)
    z = torch.from_numpy(normal(n, seed, step)).to(cuda)
    g = acc0 / B + sigma * z
    m_ref, v_ref = (1 - b1) * g, (1 - b2) * g * g
    vh = v_ref / (1 - b2)
    d = vh - sigma**2
    den = torch.sqrt(torch.where(d > 0, d, vh)) + eps
    upd = (m_ref / (1 - b1)) / den + wd * p0.float()
    p_ref = (p0.float() - lr * upd).to(torch.bfloat16)
    assert (m - m_ref).abs().max().item() < 1e-5
    stable = (d.abs() > 1e-2 * vh)  # away from the branch point of the bias correction
    diff = (p.float() - p_ref.float()).abs()[stable]
    assert stable.float().mean().item() > 0.9
    assert diff.max().item() <= 2 * 2**-8 * p_ref.float().abs().max().item()
    assert acc.abs().max().item() == 0.0


def test_bounded_wait_expires_and_reports(cuda):
    """A pipeline wait on a barrier that nothing completes gives up after its cycle budget, raises the CTA abort flag and
    sets the error word; the kernel returns and the context keeps working."""
    from opake_b200.ops import _lib
    L = _lib.lib()
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    waited = torch.zeros(1, dtype=torch.int64, device=cuda)
    budget = 200_000_000      # about 0.1 s
    assert L.opk_wait_selftest(err.data_ptr(), budget, waited.data_ptr(), _lib.stream_ptr(cuda)) == 0
    torch.cuda.synchronize()
    assert err.item() == 3 and budget <= waited.item() < 20 * budget
    x = torch.ones(1024, device=cuda)
    assert x.sum().item() == 1024.0          # context still usable


def test_dp_step_banded_toeplitz_ring_matches_streaming_inverse(cuda):
    """Band-MF / banded-square-root correlated noise in the fused step: with zero gradients, SGD, lr = 1 and fp32 master
    weights the parameter moves by exactly -sigma * zhat_t, where zhat = C^{-1} z is the banded Toeplitz recursion
    ``zhat_t = (z_t - sum_k c_k zhat_{t-k}) / c_0`` (packages/opake-dpftrl/src/opake/api/dpftrl/noise/_toeplitz.py:177-326)."""
    import numpy as np

    from opake_b200.ops import kernels as K
    from opake_b200.ops.philox_ref import normal

    n, off = 1024 + 8, 64              # a shard that does not start at element 0 (state rows stay 16-byte aligned)
    coef = [1.25, 0.5, -0.25, 0.125]
    nlag = len(coef) - 1
    acc = torch.zeros(off + n, device=cuda)
    p = torch.zeros(off + n, dtype=torch.bfloat16, device=cuda)
    master = torch.zeros(n, device=cuda)
    ring = torch.zeros(nlag, n, device=cuda)
    c_dev = torch.tensor(coef, device=cuda)
    sigma, seed, pos = 0.5, 7, 0
    hist, want = [], np.zeros(n, dtype=np.float64)
    for step in range(6):
        K.dp_step(grad_src=[acc.data_ptr()], shard_begin=off, shard_len=n, inv_batch=1.0, sigma=sigma, seed=seed, step=step,
                  m=None, v=None, master=master, param_dst=[p.data_ptr()], param_src=p, lr=1.0, beta1=0.9, beta2=0.999,
                  eps=1e-8, weight_decay=0.0, bc1=1.0, bc2=1.0, phi_hat=0.0, toep_state=ring, toep_coef=c_dev, toep_pos=pos,
                  sgd_mode=True, device=cuda)
        pos = (pos - 1) % nlag
        z = normal(n, seed, step, offset=off).astype(np.float64)
        zhat = (z - sum(coef[k] * hist[-k] for k in range(1, min(nlag, len(hist)) + 1))) / coef[0]
        hist.append(zhat)
        want -= sigma * zhat
        got = master.double().cpu().numpy()
        assert np.abs(got - want).max() < 5e-5 * (step + 1), step
    assert p[off:].float().sub(master).abs().max().item() <= 2 ** -8 * master.abs().max().item()


def test_sharded_sum_push_matches_local_group_pass(cuda):
    """The reduce-scatter form of the group accumulation (reductions into per-owner shards) gives the sums of the local
    one-pass kernel; here both 'owners' live on this GPU."""
    from opake_b200.ops import kernels as K

    n, k = 8 * 1000 + 8 * 37, 3
    gs = [_rand((n,), cuda, 2.0) for _ in range(k)]
    scales = [torch.tensor([s], device=cuda) for s in (0.5, 1.0, 0.125)]
    want = torch.randn(n, device=cuda)
    base = want.clone()
    K.clip_accumulate_group(gs, scales, want)
    bounds = [0, 8 * 600, n]
    shards = [base[bounds[o]:bounds[o + 1]].clone() for o in range(2)]
    for rank in (0, 1):         # the starting owner changes the walk, not the result
        cur = [s.clone() for s in shards]
        K.clip_accumulate_group_push(gs, scales, [t.data_ptr() for t in cur], bounds, rank, n)
        torch.cuda.synchronize()
        got = torch.cat(cur)
        assert (got - want).abs().max().item() <= 1e-5 * want.abs().max().item()


def test_copy_bytes_and_shared_embedding_accumulate(cuda):
    from opake_b200.ops import kernels as K

    src = torch.randn(1 << 16, device=cuda)
    dst = torch.zeros_like(src)
    K.copy_bytes(dst.data_ptr(), src.data_ptr(), src.numel() * 4, cuda)
    assert torch.equal(dst, src)
    V, T, D = 300, 96, 64
    g = torch.Generator(device=cuda).manual_seed(5)
    tok = torch.randint(0, V, (T,), generator=g, device=cuda, dtype=torch.int32)
    dx = torch.randn(T, D, generator=g, device=cuda).to(torch.bfloat16)
    ws = K.EmbeddingGradWorkspace(V, T, D, cuda)
    K.embedding_bwd_compact(tok, dx, ws, None)
    scale = torch.tensor([0.37], device=cuda)
    a, b = torch.zeros(V, D, device=cuda), torch.zeros(V, D, device=cuda)
    K.embedding_accumulate(tok, ws, scale, a, T)
    K.embedding_accumulate(tok, ws, scale, b, T, shared=True)
    assert torch.equal(a, b)


def test_debug_library_records_and_skips_bad_indices():
    """The checked library variant (child process: a process loads one variant) records an out-of-range token id,
    label and expert id with file / line / index / bound, skips the access, and leaves the context usable."""
    import os
    import subprocess
    import sys

    code = r'''
import torch
from opake_b200.ops import kernels as K
from opake_b200.ops._lib import debug_bounds_report
dev = torch.device("cuda", 0)
assert debug_bounds_report() == {"failures": 0, "file": "", "line": 0, "index": 0, "bound": 0}
table = torch.randn(50, 64, device=dev).bfloat16()
tok = torch.tensor([1, 2, 77, 3], dtype=torch.int32, device=dev)
out = K.embedding_fwd(tok, table)
torch.cuda.synchronize()
assert torch.equal(out[0], table[1]) and torch.equal(out[3], table[3]) and float(out[2].abs().max()) == 0.0
rep = debug_bounds_report()
assert rep["failures"] >= 1 and rep["index"] == 77 and rep["bound"] == 50 and rep["file"].endswith("elementwise.cu"), rep
assert debug_bounds_report()["failures"] == 0          # the read cleared it
idx = torch.tensor([0, 3, 9, 1, 2, 2], dtype=torch.int32, device=dev)        # 9 >= E = 4
plan = K.MoePlan(3, 4, 2, dev)
plan.build(idx)
torch.cuda.synchronize()
rep = debug_bounds_report()
assert rep["failures"] >= 1 and rep["index"] == 9 and rep["bound"] == 4 and rep["file"].endswith("moe.cu"), rep
assert int(plan.dest.flatten()[2]) == -1
x = torch.ones(4, device=dev)
assert float((x + 1).sum()) == 8.0          # the context is alive
print("DEBUG-BOUNDS-OK")
'''
    env = dict(os.environ, OPAKE_B200_DEBUG_KERNELS="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert "DEBUG-BOUNDS-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_release_library_drops_bad_ids_without_touching_memory():
    from opake_b200.ops import kernels as K
    from opake_b200.ops._lib import debug_bounds_report

    assert debug_bounds_report() is None            # release build: no record
    dev = torch.device("cuda", 0)
    table = torch.randn(50, 64, device=dev).bfloat16()
    tok = torch.tensor([1, -4, 50, 3], dtype=torch.int32, device=dev)
    out = K.embedding_fwd(tok, table)
    assert torch.equal(out[0], table[1]) and float(out[1:3].abs().max()) == 0.0
    idx = torch.tensor([0, 3, 9, 1, 2, 2], dtype=torch.int32, device=dev)
    plan = K.MoePlan(3, 4, 2, dev)
    plan.build(idx)
    y = torch.randn(plan.R, 64, device=dev).bfloat16()
    wts = torch.ones(3, 2, device=dev)
    o = K.moe_combine(y, plan, torch.empty(3, 64, dtype=torch.bfloat16, device=dev), wts)
    torch.cuda.synchronize()
    assert int(plan.dest.flatten()[2]) == -1
    ref = y[plan.dest.flatten()[3].long()].float()           # token 1: slot 0 dropped, slot 1 kept
    torch.testing.assert_close(o[1].float(), ref, atol=2e-2, rtol=2e-2)


def test_engine_step_leaves_every_guard_band_intact():
    """A whole DP step (forward, backward, clip, accumulate, fused update) with gradient slots and workspaces
    allocated between guard bands: no kernel writes outside its buffers."""
    from opake_b200.models.config import tiny_llama
    from opake_b200.parallel.engine import EngineConfig, ShardedDPEngine

    dev = torch.device("cuda", 0)
    cfg = tiny_llama()
    for graph in (False, True):
        eng = ShardedDPEngine(cfg, EngineConfig(logical_batch=4, noise_multiplier=0.5, use_cuda_graph=graph, debug_canaries=True), dev)
        tok = torch.randint(0, cfg.vocab_size, (4, 96), dtype=torch.int32).pin_memory()
        labels = torch.roll(tok, -1, 1).clone()
        labels[:, -1] = -100
        for _ in range(2):
            loss = eng.step(tok, labels).item()
        assert loss == loss and len(eng.canaries) > 20
        assert eng.canaries.check() == []
