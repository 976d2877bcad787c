"""Fused LoRA linear layers with explicit backward and vmap rules (packages/opake-patches/src/opake/api/patches/
kernels/lora.py:206,499,1063: ``Opake_LoRA_W``, ``_QKV``, ``_MLP``).

``y = x W^T + s (x A^T) B^T (+ bias)`` with frozen ``W`` and trainable ``A [r, in]``, ``B [out, r]``. The backward is
written out (instead of letting autograd trace five matmuls) so that under ``vmap`` only the two small adapter
gradients are materialised per example: ``dA_b = s (dy_b B)^T x_b`` and ``dB_b = s dy_b^T (x_b A^T)``; ``dx`` is one
flattened GEMM chain for the whole batch. ``lora_grad_sq_norms`` gives the per-example squared norms of ``dA`` and
``dB`` without forming them (Gram identity), for clipping LoRA-only fine-tuning without any per-example tensor.
On CUDA bf16 the large products run on the tcgen05 GEMM; everything else uses ``torch.matmul``.
"""
from __future__ import annotations

import torch

__all__ = ["lora_linear", "lora_qkv", "lora_mlp", "lora_grad_sq_norms"]


def _mm(a: torch.Tensor, b_nk: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ b_nk[N, K]^T``."""
    if a.is_cuda and a.dtype == torch.bfloat16 and b_nk.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0 and b_nk.shape[0] % 8 == 0 \
            and a.shape[0] >= 128:
        from ...ops import gemm as G
        return G.gemm(a.contiguous(), b_nk.contiguous())
    return a @ b_nk.t()


def _mm_nn(a: torch.Tensor, b_kn: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ b_kn[K, N]``."""
    if a.is_cuda and a.dtype == torch.bfloat16 and b_kn.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0 and b_kn.shape[1] % 8 == 0 \
            and a.shape[0] >= 128:
        from ...ops import gemm as G
        return G.gemm(a.contiguous(), b_kn.contiguous(), b_mn=True)
    return a @ b_kn


class _LoRABwd(torch.autograd.Function):
    @staticmethod
    def forward(dy, x, xa, W, A, B, s):
        # dy [M, out], x [M, in], xa [M, r]
        dyB = _mm_nn(dy, B)                                  # [M, r]
        dx = _mm_nn(dy, W) + s * _mm_nn(dyB, A)              # [M, in]
        dA = s * (dyB.t() @ x)                               # [r, in]
        dB = s * (dy.t() @ xa)                               # [out, r]
        return dx, dA, dB

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused LoRA linear is not supported")

    @staticmethod
    def vmap(info, in_dims, dy, x, xa, W, A, B, s):
        if any(d is not None for d in in_dims[3:6]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        dy, x, xa = (t.movedim(d, 0) if d is not None else t.unsqueeze(0).expand(n, *t.shape) for t, d in zip((dy, x, xa), in_dims[:3]))
        M = dy.shape[1]
        dyf = dy.reshape(n * M, -1)
        dyB = _mm_nn(dyf, B)
        dx = (_mm_nn(dyf, W) + s * _mm_nn(dyB, A)).view(n, M, -1)
        dA = s * torch.bmm(dyB.view(n, M, -1).transpose(1, 2), x)        # [n, r, in]
        dB = s * torch.bmm(dy.transpose(1, 2), xa)                       # [n, out, r]
        return (dx, dA, dB), (0, 0, 0)


class _LoRA(torch.autograd.Function):
    @staticmethod
    def forward(x, W, A, B, s):
        xa = _mm(x, A)                                       # [M, r]
        y = _mm(x, W) + s * _mm(xa, B)
        return y, xa

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, W, A, B, s = inputs
        ctx.save_for_backward(x, output[1], W, A, B)
        ctx.mark_non_differentiable(output[1])
        ctx.s = s

    @staticmethod
    def backward(ctx, dy, _dxa):
        x, xa, W, A, B = ctx.saved_tensors
        dx, dA, dB = _LoRABwd.apply(dy.contiguous(), x, xa, W, A, B, ctx.s)
        return dx, None, dA, dB, None

    @staticmethod
    def vmap(info, in_dims, x, W, A, B, s):
        if any(d is not None for d in in_dims[1:4]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        x = x.movedim(in_dims[0], 0) if in_dims[0] is not None else x.unsqueeze(0).expand(n, *x.shape)
        M = x.shape[1]
        y, xa = _LoRA.apply(x.reshape(n * M, -1), W, A, B, s)
        return (y.view(n, M, -1), xa.view(n, M, -1)), (0, 0)


def lora_linear(x, weight, lora_a, lora_b, scaling: float, bias=None):
    """``x [..., in]`` -> ``[..., out]``."""
    lead = x.shape[:-1]
    y = _LoRA.apply(x.reshape(-1, x.shape[-1]), weight, lora_a, lora_b, float(scaling))[0]
    if bias is not None:
        y = y + bias
    return y.view(*lead, -1)


def lora_qkv(x, q, k, v):
    """Three adapted projections of the same input; each of ``q, k, v`` is ``(weight, A, B, scaling, bias)``."""
    return tuple(lora_linear(x, *p) for p in (q, k, v))


def lora_mlp(x, gate, up, down, act: str = "silu"):
    """Gated MLP with adapters on all three projections (``act``: ``silu`` or ``gelu_tanh``)."""
    from .functions import opake_geglu, opake_swiglu
    g, u = lora_linear(x, *gate), lora_linear(x, *up)
    h = opake_swiglu(g, u) if act == "silu" else opake_geglu(g, u)
    return lora_linear(h, *down)


def lora_grad_sq_norms(x, dy, lora_a, lora_b, scaling: float):
    """Per-example ``(||dA_b||^2, ||dB_b||^2)`` for ``x [n, T, in]``, ``dy [n, T, out]`` without materialising the
    gradients: ``||U^T V||_F^2 = sum((U U^T) * (V V^T))`` with T x T Gram matrices (cheap when ``T << in, out``)."""
    s2 = float(scaling) ** 2
    xf, dyf = x.float(), dy.float()
    dyB = dyf @ lora_b.float()                      # [n, T, r]
    xa = xf @ lora_a.float().t()                    # [n, T, r]
    gx = torch.bmm(xf, xf.transpose(1, 2))          # [n, T, T]
    gdy = torch.bmm(dyf, dyf.transpose(1, 2))
    na = s2 * (torch.bmm(dyB, dyB.transpose(1, 2)) * gx).sum((1, 2))
    nb = s2 * (gdy * torch.bmm(xa, xa.transpose(1, 2))).sum((1, 2))
    return na, nb
