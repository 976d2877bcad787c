"""tcgen05 flash attention (forward and backward) against an fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, H, KV, hd):
    T = qkv.shape[0]
    x = qkv.float().detach().requires_grad_()
    q = x[:, : H * hd].view(T, H, hd)
    k = x[:, H * hd : (H + KV) * hd].view(T, KV, hd).repeat_interleave(H // KV, 1)
    v = x[:, (H + KV) * hd :].view(T, KV, hd).repeat_interleave(H // KV, 1)
    s = torch.einsum("thd,shd->hts", q, k) * hd**-0.5
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * hd)
    return x, o, lse


# the last two cases have more (query tile, head) items than the GPU has SMs: every persistent CTA walks several items
@pytest.mark.parametrize("T,H,KV,hd", [(128, 2, 1, 128), (384, 4, 2, 128), (300, 4, 4, 64), (1024, 8, 2, 128),
                                       (2048, 16, 4, 128), (1100, 24, 8, 64)])
def test_flash_forward(cuda, T, H, KV, hd):
    from opake_b200.ops.flash import flash_fwd
    from opake_b200.ops._lib import raise_if_device_error

    torch.manual_seed(0)
    qkv = (torch.randn(T, (H + 2 * KV) * hd, device=cuda) * 0.7).to(torch.bfloat16)
    out, lse = flash_fwd(qkv, H, KV, hd)
    raise_if_device_error(cuda)
    _, o_ref, lse_ref = _ref(qkv, H, KV, hd)
    assert (lse - lse_ref).abs().max().item() < 2e-2
    assert (out.float() - o_ref).abs().max().item() < 3e-2 * o_ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("T,H,KV,hd", [(1024, 4, 2, 128), (640, 4, 4, 64), (1536, 16, 4, 128)])
def test_flash_forward_growing_scores(cuda, T, H, KV, hd):
    """Keys whose magnitude grows with the position: the row maxima jump by far more than the lazy-rescale
    threshold from one key tile to the next, so the running maximum is replaced, the accumulators are rescaled and
    a tile whose exponentials were taken against a stale maximum is done again."""
    from opake_b200.ops.flash import flash_fwd
    from opake_b200.ops._lib import raise_if_device_error

    torch.manual_seed(2)
    x = torch.randn(T, (H + 2 * KV) * hd, device=cuda)
    ramp = torch.linspace(1.0, 30.0, T, device=cuda)[:, None]
    x[:, H * hd : (H + KV) * hd] *= ramp
    qkv = x.to(torch.bfloat16)
    out, lse = flash_fwd(qkv, H, KV, hd)
    raise_if_device_error(cuda)
    _, o_ref, lse_ref = _ref(qkv, H, KV, hd)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert (lse - lse_ref).abs().max().item() < 2e-2 + 2e-3 * lse_ref.abs().max().item()
    assert (out.float() - o_ref).abs().max().item() < 3e-2 * o_ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("T,H,KV,hd", [(128, 2, 1, 128), (384, 4, 2, 128), (300, 4, 4, 64), (1024, 8, 2, 128)])
def test_flash_backward(cuda, T, H, KV, hd, split):
    from opake_b200.ops import attention as A
    from opake_b200.ops._lib import raise_if_device_error

    if not A.have_flash():
        pytest.skip("backward kernels not built")
    from opake_b200.ops.flash import flash_bwd, flash_fwd

    torch.manual_seed(1)
    qkv = (torch.randn(T, (H + 2 * KV) * hd, device=cuda) * 0.7).to(torch.bfloat16)
    dout = (torch.randn(T, H * hd, device=cuda) * 0.5).to(torch.bfloat16)
    out, lse = flash_fwd(qkv, H, KV, hd)
    dqkv = torch.full_like(qkv, float("nan"))
    flash_bwd(dout, qkv, out, lse, H, KV, hd, dqkv, split_heads=split)
    raise_if_device_error(cuda)
    x, o_ref, _ = _ref(qkv, H, KV, hd)
    o_ref.backward(dout.float())
    err = (dqkv.float() - x.grad).abs().max().item()
    assert err < 4e-2 * x.grad.abs().max().item() + 1e-3, err
