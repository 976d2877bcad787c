"""Mixture-of-experts routing kernels and grouped GEMM modes against PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_route_plan_gather_combine(cuda):
    from opake_b200.ops import kernels as K
    torch.manual_seed(0)
    T, E, k, D = 300, 12, 3, 64
    logits = torch.randn(T, E, device=cuda).to(torch.bfloat16)
    plan = K.MoePlan(T, E, k, cuda)
    K.moe_route(logits, plan, norm_topk=True)
    probs = logits.float().softmax(-1)
    w, _ = torch.topk(probs, k, dim=-1)
    idx = plan.idx.long()                      # bf16 logits have ties; compare selected values, not indices
    assert torch.allclose(probs.gather(1, idx), w, atol=1e-6) and torch.allclose(plan.probs, probs, atol=1e-6)
    assert (idx.sort(-1).values.diff(dim=-1) > 0).all()          # k distinct experts per token
    assert torch.allclose(plan.wts, w / w.sum(-1, keepdim=True), atol=1e-6)
    counts = torch.bincount(idx.reshape(-1), minlength=E)
    assert torch.equal(plan.counts.long(), counts)
    padded = torch.where(counts == 0, torch.full_like(counts, 128), (counts + 127) // 128 * 128)
    offs = torch.cumsum(padded, 0) - padded
    assert torch.equal(plan.group_k[:, 0].long(), offs) and torch.equal(plan.group_k[:, 1].long(), padded // 64)
    # stable: inside an expert's segment the entries appear in increasing entry order
    dest, flat = plan.dest.reshape(-1).long(), idx.reshape(-1)
    for e in range(E):
        rows = dest[flat == e]
        assert torch.equal(rows, offs[e] + torch.arange(rows.numel(), device=cuda))
    src = plan.src_entry.long()
    assert torch.equal(src[dest], torch.arange(T * k, device=cuda)) and (src >= 0).sum().item() == T * k
    tg = plan.tile_group.long()
    n_tiles = int(padded.sum().item()) // 128
    assert torch.equal(tg[:n_tiles], torch.repeat_interleave(torch.arange(E, device=cuda), padded // 128)) and (tg[n_tiles:] == -1).all()
    x = torch.randn(T, D, device=cuda).to(torch.bfloat16)
    xs = K.moe_gather(x, plan, torch.empty(plan.R, D, device=cuda, dtype=torch.bfloat16))
    want = torch.zeros(plan.R, D, device=cuda, dtype=torch.bfloat16)
    want[dest] = x[torch.arange(T * k, device=cuda) // k]
    assert torch.equal(xs, want)
    res = torch.randn(T, D, device=cuda).to(torch.bfloat16)
    out = K.moe_combine(xs, plan, torch.empty_like(x), wts=plan.wts, residual=res)
    ref = res.float() + (plan.wts[..., None] * xs[plan.dest.long()].float()).sum(1)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    dw = K.moe_combine_bwd(res, xs, plan, torch.empty(T, k, device=cuda))
    assert torch.allclose(dw, (res.float()[:, None, :] * xs[plan.dest.long()].float()).sum(-1), atol=1e-2, rtol=1e-2)
    # router backward against autograd
    lg = logits.float().requires_grad_()
    p2 = lg.softmax(-1)
    w2 = p2.gather(1, idx)
    (w2 / w2.sum(-1, keepdim=True) * dw).sum().backward()
    drl = K.moe_route_bwd(plan, dw, torch.empty(T, E, device=cuda, dtype=torch.bfloat16), norm_topk=True)
    assert (drl.float() - lg.grad).abs().max() < 2e-2 * lg.grad.abs().max() + 1e-4


def test_grouped_gemm_modes(cuda):
    from opake_b200.ops import gemm as G, kernels as K
    torch.manual_seed(1)
    T, E, k, D, N = 500, 6, 2, 128, 256
    logits = torch.randn(T, E, device=cuda).to(torch.bfloat16)
    logits[:, 4] = -30.0                       # one expert without any token
    plan = K.moe_route(logits, K.MoePlan(T, E, k, cuda))
    x = (torch.randn(T, D, device=cuda) * 0.5).to(torch.bfloat16)
    xs = K.moe_gather(x, plan, torch.empty(plan.R, D, device=cuda, dtype=torch.bfloat16))
    W = (torch.randn(E, N, D, device=cuda) * 0.1).to(torch.bfloat16)
    y = torch.zeros(plan.R, N, device=cuda, dtype=torch.bfloat16)
    G.gemm(xs, W, out=y, tile_group=plan.tile_group)
    tg = plan.tile_group.long()
    for tl in range(plan.R // 128):
        rows = slice(tl * 128, tl * 128 + 128)
        if tg[tl] >= 0:
            want = xs[rows].float() @ W[tg[tl]].float().t()
            assert (y[rows].float() - want).abs().max() < 2e-2 * want.abs().max() + 1e-3
        else:
            assert (y[rows] == 0).all()        # skipped tiles are left untouched
    # dgrad: dx = dy @ W[e]
    dxs = torch.zeros(plan.R, D, device=cuda, dtype=torch.bfloat16)
    G.gemm(y, W, b_mn=True, out=dxs, tile_group=plan.tile_group)
    tl = 0
    want = y[:128].float() @ W[tg[0]].float()
    assert (dxs[:128].float() - want).abs().max() < 3e-2 * want.abs().max() + 1e-3
    # wgrad per expert with the shared squared-norm accumulator
    dW = torch.empty(E, N, D, device=cuda, dtype=torch.bfloat16)
    ss = torch.zeros(1, dtype=torch.float64, device=cuda)
    G.gemm(y, xs, a_mn=True, b_mn=True, out=dW, epilogue=G.EPI_SUMSQ, sumsq=ss, group_k=plan.group_k, sumsq_shared=True)
    gk = plan.group_k.long()
    for e in range(E):
        seg = slice(int(gk[e, 0]), int(gk[e, 0] + 64 * gk[e, 1]))
        want = y[seg].float().t() @ xs[seg].float()
        assert (dW[e].float() - want).abs().max() < 3e-2 * want.abs().max() + 1e-3
    assert (dW[4] == 0).all()
    assert abs(ss.item() - dW.double().pow(2).sum().item()) < 1e-3 * ss.item()
    from opake_b200.ops._lib import raise_if_device_error
    raise_if_device_error(cuda)


def test_expert_parallel_fused_single_rank(cuda):
    """The expert-parallel kernels with a group of one rank (every peer pointer is the rank's own buffer): dispatch,
    grouped GEMMs, combine, per-source norms and clipped accumulation against a dense fp32 oracle."""
    from tests.multi_gpu_selftest import ep_fused_check

    res = ep_fused_check(0, 1, cuda)
    for name in ("out", "dx", "d_router", "acc_wgu", "acc_wd", "norms"):
        assert res[name] < 3e-2, (name, res)
