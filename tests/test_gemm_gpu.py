"""tcgen05 GEMM against an fp32 PyTorch reference for every operand layout and epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["pair", "single"])
def _kernel_variant(request):
    """Every case runs on the two-CTA kernel (where the shape is eligible) and on the single-CTA kernel."""
    from opake_b200.ops import gemm as G

    before = G.pair_mode()
    G.set_pair_mode(request.param == "pair")
    yield
    G.set_pair_mode(before)


def _rand(shape, dev, scale=1.0):
    return (torch.randn(shape, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(out, ref, rtol=2e-2):
    err = (out.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < rtol, f"max err {err} vs scale {den}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 136, 96), (2048, 1024, 512), (77, 50264, 64)])
def test_gemm_nt(cuda, M, N, K):
    from opake_b200.ops import gemm as G
    from opake_b200.ops._lib import raise_if_device_error

    a, b = _rand((M, K), cuda), _rand((N, K), cuda)
    out = G.gemm(a, b)
    raise_if_device_error(cuda)
    _close(out, a.float() @ b.float().T)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 320, 200), (2048, 512, 1024)])
def test_gemm_dgrad_layout(cuda, M, N, K):
    from opake_b200.ops import gemm as G
    from opake_b200.ops._lib import raise_if_device_error

    dy, w = _rand((M, K), cuda), _rand((K, N), cuda)  # reduce over K = rows of w
    out = G.gemm(dy, w, b_mn=True)
    raise_if_device_error(cuda)
    _close(out, dy.float() @ w.float())


@pytest.mark.parametrize("T,N,K", [(64, 128, 256), (200, 384, 264), (2048, 512, 768)])
def test_gemm_wgrad_layout_and_sumsq(cuda, T, N, K):
    from opake_b200.ops import gemm as G
    from opake_b200.ops._lib import raise_if_device_error

    dy, x = _rand((T, N), cuda, 0.1), _rand((T, K), cuda)
    ss = torch.zeros(1, dtype=torch.float64, device=cuda)
    out = G.linear_wgrad(dy, x, sumsq=ss)
    raise_if_device_error(cuda)
    ref = dy.float().T @ x.float()
    _close(out, ref)
    want = out.double().pow(2).sum().item()
    assert abs(ss.item() - want) / want < 1e-4
    out2 = G.linear_wgrad(dy, x)
    assert torch.equal(out, out2)


def test_gemm_bias_residual_alpha(cuda):
    from opake_b200.ops import gemm as G

    a, b = _rand((256, 128), cuda), _rand((512, 128), cuda)
    bias, res = _rand((512,), cuda), _rand((256, 512), cuda)
    out = G.gemm(a, b, bias=bias, residual=res, alpha=0.5)
    _close(out, 0.5 * (a.float() @ b.float().T) + bias.float() + res.float())
    # in-place residual accumulate
    acc = res.clone()
    G.gemm(a, b, out=acc, residual=acc)
    _close(acc, (a.float() @ b.float().T) + res.float())


def test_gemm_batched_shared_b(cuda):
    from opake_b200.ops import gemm as G

    a = _rand((8, 256, 128), cuda)
    b = _rand((2, 384, 128), cuda)
    out = G.gemm(a, b, b_batch_div=4)
    ref = torch.einsum("bmk,bnk->bmn", a.float(), b.float().repeat_interleave(4, 0))
    _close(out, ref)


def test_gemm_swiglu(cuda):
    from opake_b200.ops import gemm as G

    x, w = _rand((256, 128), cuda), _rand((1024, 128), cuda, 0.1)
    act = torch.empty(256, 512, dtype=torch.bfloat16, device=cuda)
    raw = G.gemm(x, w, epilogue=G.EPI_SWIGLU, act=act)
    ref = x.float() @ w.float().T
    _close(raw, ref)
    g, u = raw.float()[:, 0::2], raw.float()[:, 1::2]
    _close(act, torch.nn.functional.silu(g) * u)


@pytest.mark.parametrize("T,F,D", [(256, 512, 128), (300, 200, 72), (2048, 1024, 256)])
def test_gemm_swiglu_backward_epilogue(cuda, T, F, D):
    """d(act) = dy @ w_down stays in the accumulator; the epilogue emits interleaved (d_gate, d_up)."""
    from opake_b200.ops import gemm as G
    from opake_b200.ops._lib import raise_if_device_error

    dy, wd = _rand((T, D), cuda), _rand((D, F), cuda, 0.1)
    gu = _rand((T, 2 * F), cuda)
    out = torch.empty_like(gu)
    G.swiglu_dgrad(dy, wd, gu, out=out)
    raise_if_device_error(cuda)
    g, u = gu.float()[:, 0::2], gu.float()[:, 1::2]
    dact = (dy.float() @ wd.float())
    sg = torch.sigmoid(g)
    ref = torch.stack([dact * u * sg * (1 + g * (1 - sg)), dact * g * sg], dim=-1).reshape(T, 2 * F)
    _close(out, ref)


def test_gemm_lce(cuda):
    from opake_b200.ops import gemm as G

    T, V, D = 300, 1000, 128
    h, w = _rand((T, D), cuda), _rand((V, D), cuda, 0.2)
    labels = torch.randint(0, V, (T,), device=cuda, dtype=torch.int32)
    labels[::7] = -100
    nt = G.lce_tiles(V)
    pmax = torch.empty(T, nt, device=cuda)
    psum = torch.empty(T, nt, device=cuda)
    tgt = torch.zeros(T, device=cuda)
    G.gemm(h, w, epilogue=G.EPI_LCE_FWD, labels=labels, pmax=pmax, psum=psum, tgt=tgt)
    m = pmax.max(dim=1).values
    lse = m + torch.log((psum * torch.exp(pmax - m[:, None])).sum(1))
    logits = h.float() @ w.float().T
    ref_lse = torch.logsumexp(logits, dim=1)
    assert (lse - ref_lse).abs().max().item() < 2e-3
    valid = labels >= 0
    ref_t = logits[valid, labels[valid].long()]
    assert (tgt[valid] - ref_t).abs().max().item() < 2e-3
    coef = valid.float() / valid.sum()
    d = G.gemm(h, w, epilogue=G.EPI_LCE_BWD, labels=labels, lse=lse, coef=coef)
    p = torch.softmax(logits, dim=1)
    onehot = torch.zeros_like(p)
    onehot[valid, labels[valid].long()] = 1
    ref_d = (p - onehot) * coef[:, None]
    assert (d.float() - ref_d).abs().max().item() < 2e-2 * ref_d.abs().max().item() + 1e-6


@pytest.mark.parametrize("swiglu", [False, True])
def test_staged_weight_fetch_inside_the_gemm(cuda, swiglu):
    """The staged two-CTA GEMM copies its weight operand into a local destination band by band while it multiplies
    (the all-gather of a sharded weight fused into its first consumer): same product as the plain kernel, and the
    destination ends up holding the weight. The 'remote' source is local memory here."""
    from opake_b200.ops import gemm as G

    if not G.pair_mode():
        pytest.skip("staging runs on the two-CTA kernel")
    M, N, K_ = 512, 4608, 320
    g = torch.Generator(device=cuda).manual_seed(11)
    x = (torch.randn(M, K_, generator=g, device=cuda) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g, device=cuda) * 0.1).to(torch.bfloat16)
    dst = torch.zeros_like(w)
    ready = torch.zeros(64, dtype=torch.int32, device=cuda)
    if swiglu:
        act_a = torch.empty(M, N // 2, dtype=torch.bfloat16, device=cuda)
        act_b = torch.empty_like(act_a)
        want = G.gemm(x, w, epilogue=G.EPI_SWIGLU, act=act_a)
        got = G.gemm(x, w, epilogue=G.EPI_SWIGLU, act=act_b, stage=(dst, ready))
        assert torch.equal(act_a, act_b)
    else:
        want = G.gemm(x, w)
        got = G.gemm(x, w, stage=(dst, ready))
    torch.cuda.synchronize()
    from opake_b200.ops._lib import raise_if_device_error

    raise_if_device_error(cuda)
    assert torch.equal(got, want)
    assert torch.equal(dst, w)
