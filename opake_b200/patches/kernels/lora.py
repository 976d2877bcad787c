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


def _front(t, d, n):
    return t.movedim(d, 0) if d is not None else t.unsqueeze(0).expand(n, *t.shape)


def _adapter_grads(dy, x, xa, A, B, s, n=None):
    """``(dy B, dA, dB)`` for one adapted projection; with ``n`` the row dimension is ``n`` examples of ``M`` rows and the
    adapter gradients stay per example."""
    dyB = _mm_nn(dy, B)
    if n is None:
        return dyB, s * (dyB.t() @ x), s * (dy.t() @ xa)
    M = dy.shape[0] // n
    dA = s * torch.bmm(dyB.view(n, M, -1).transpose(1, 2), x.view(n, M, -1))
    dB = s * torch.bmm(dy.view(n, M, -1).transpose(1, 2), xa.view(n, M, -1))
    return dyB, dA, dB


class _LoRAQKVBwd(torch.autograd.Function):
    """Backward of three adapted projections of ONE input: the input gradient is a single accumulated chain, the six
    adapter gradients are the only per-example tensors under vmap (``Opake_LoRA_QKV``, lora.py:499 of the reference)."""

    @staticmethod
    def forward(dq, dk, dv, x, xaq, xak, xav, Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv, sq, sk, sv):
        return _LoRAQKVBwd._run(None, dq, dk, dv, x, xaq, xak, xav, Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv, sq, sk, sv)

    @staticmethod
    def _run(n, dq, dk, dv, x, xaq, xak, xav, Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv, sq, sk, sv):
        dx, grads = None, []
        for dy, xa, W, A, B, s in ((dq, xaq, Wq, Aq, Bq, sq), (dk, xak, Wk, Ak, Bk, sk), (dv, xav, Wv, Av, Bv, sv)):
            dyB, dA, dB = _adapter_grads(dy, x, xa, A, B, s, n)
            part = _mm_nn(dy, W) + s * _mm_nn(dyB, A)
            dx = part if dx is None else dx + part
            grads += [dA, dB]
        return (dx, *grads)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused LoRA projections is not supported")

    @staticmethod
    def vmap(info, in_dims, dq, dk, dv, x, xaq, xak, xav, *rest):
        if any(d is not None for d in in_dims[7:16]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        acts = [_front(t, d, n) for t, d in zip((dq, dk, dv, x, xaq, xak, xav), in_dims[:7])]
        M = acts[0].shape[1]
        flat = [t.reshape(n * M, -1) for t in acts]
        out = _LoRAQKVBwd._run(n, *flat, *rest)
        return (out[0].view(n, M, -1), *out[1:]), (0,) * 7


class _LoRAQKV(torch.autograd.Function):
    @staticmethod
    def forward(x, Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv, sq, sk, sv):
        outs, xas = [], []
        for W, A, B, s in ((Wq, Aq, Bq, sq), (Wk, Ak, Bk, sk), (Wv, Av, Bv, sv)):
            xa = _mm(x, A)
            outs.append(_mm(x, W) + s * _mm(xa, B))
            xas.append(xa)
        return (*outs, *xas)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv, sq, sk, sv = inputs
        ctx.save_for_backward(x, *output[3:], Wq, Aq, Bq, Wk, Ak, Bk, Wv, Av, Bv)
        ctx.mark_non_differentiable(*output[3:])
        ctx.s = (sq, sk, sv)

    @staticmethod
    def backward(ctx, dq, dk, dv, *_):
        x, xaq, xak, xav, *w = ctx.saved_tensors
        dx, dAq, dBq, dAk, dBk, dAv, dBv = _LoRAQKVBwd.apply(dq.contiguous(), dk.contiguous(), dv.contiguous(), x, xaq, xak, xav,
                                                             *w, *ctx.s)
        return dx, None, dAq, dBq, None, dAk, dBk, None, dAv, dBv, None, None, None

    @staticmethod
    def vmap(info, in_dims, x, *rest):
        if any(d is not None for d in in_dims[1:10]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        x = _front(x, in_dims[0], n)
        M = x.shape[1]
        out = _LoRAQKV.apply(x.reshape(n * M, -1), *rest)
        return tuple(t.view(n, M, -1) for t in out), (0,) * 6


def lora_qkv(x, q, k, v):
    """Three adapted projections of the same input in one autograd node; each of ``q, k, v`` is
    ``(weight, A, B, scaling, bias)``. The input is saved once and its gradient accumulated in one chain."""
    lead = x.shape[:-1]
    out = _LoRAQKV.apply(x.reshape(-1, x.shape[-1]), q[0], q[1], q[2], k[0], k[1], k[2], v[0], v[1], v[2],
                         float(q[3]), float(k[3]), float(v[3]))[:3]
    res = []
    for y, p in zip(out, (q, k, v)):
        if len(p) > 4 and p[4] is not None:
            y = y + p[4]
        res.append(y.view(*lead, -1))
    return tuple(res)


def _act_fwd(g, u, act: str):
    gf = g.float()
    a = torch.nn.functional.silu(gf) if act == "silu" else torch.nn.functional.gelu(gf, approximate="tanh")
    return (a * u.float()).to(g.dtype)


def _act_bwd(dh, g, u, act: str):
    gf, uf, dhf = g.float(), u.float(), dh.float()
    if act == "silu":
        sig = torch.sigmoid(gf)
        a, da = gf * sig, sig * (1 + gf * (1 - sig))
    else:
        c = 0.7978845608028654
        t = torch.tanh(c * (gf + 0.044715 * gf ** 3))
        a = 0.5 * gf * (1 + t)
        da = 0.5 * (1 + t) + 0.5 * gf * (1 - t * t) * c * (1 + 3 * 0.044715 * gf * gf)
    return (dhf * uf * da).to(g.dtype), (dhf * a).to(g.dtype)


class _LoRAMLPBwd(torch.autograd.Function):
    """Backward of the adapted gated MLP (``Opake_LoRA_MLP``, lora.py:1063 of the reference): the activation is
    recomputed from the saved pre-activations, the three adapted projections are differentiated by hand."""

    @staticmethod
    def forward(dy, x, g, u, xag, xau, had, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd, sg, su, sd, act):
        return _LoRAMLPBwd._run(None, dy, x, g, u, xag, xau, had, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd, sg, su, sd, act)

    @staticmethod
    def _run(n, dy, x, g, u, xag, xau, had, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd, sg, su, sd, act):
        h = _act_fwd(g, u, act)
        dyB, dAd, dBd = _adapter_grads(dy, h, had, Ad, Bd, sd, n)
        dh = _mm_nn(dy, Wd) + sd * _mm_nn(dyB, Ad)
        dg, du = _act_bwd(dh, g, u, act)
        dgB, dAg, dBg = _adapter_grads(dg, x, xag, Ag, Bg, sg, n)
        duB, dAu, dBu = _adapter_grads(du, x, xau, Au, Bu, su, n)
        dx = _mm_nn(dg, Wg) + sg * _mm_nn(dgB, Ag) + _mm_nn(du, Wu) + su * _mm_nn(duB, Au)
        return dx, dAg, dBg, dAu, dBu, dAd, dBd

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused LoRA MLP is not supported")

    @staticmethod
    def vmap(info, in_dims, dy, x, g, u, xag, xau, had, *rest):
        if any(d is not None for d in in_dims[7:16]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        acts = [_front(t, d, n) for t, d in zip((dy, x, g, u, xag, xau, had), in_dims[:7])]
        M = acts[0].shape[1]
        out = _LoRAMLPBwd._run(n, *[t.reshape(n * M, -1) for t in acts], *rest)
        return (out[0].view(n, M, -1), *out[1:]), (0,) * 7


class _LoRAMLP(torch.autograd.Function):
    @staticmethod
    def forward(x, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd, sg, su, sd, act):
        xag, xau = _mm(x, Ag), _mm(x, Au)
        g = _mm(x, Wg) + sg * _mm(xag, Bg)
        u = _mm(x, Wu) + su * _mm(xau, Bu)
        h = _act_fwd(g, u, act)
        had = _mm(h, Ad)
        y = _mm(h, Wd) + sd * _mm(had, Bd)
        return y, g, u, xag, xau, had

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd, sg, su, sd, act = inputs
        ctx.save_for_backward(x, *output[1:], Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd)
        ctx.mark_non_differentiable(*output[1:])
        ctx.consts = (sg, su, sd, act)

    @staticmethod
    def backward(ctx, dy, *_):
        x, g, u, xag, xau, had, *w = ctx.saved_tensors
        dx, dAg, dBg, dAu, dBu, dAd, dBd = _LoRAMLPBwd.apply(dy.contiguous(), x, g, u, xag, xau, had, *w, *ctx.consts)
        return dx, None, dAg, dBg, None, dAu, dBu, None, dAd, dBd, None, None, None, None

    @staticmethod
    def vmap(info, in_dims, x, *rest):
        if any(d is not None for d in in_dims[1:10]):
            raise NotImplementedError("per-example LoRA weights are not supported")
        n = info.batch_size
        x = _front(x, in_dims[0], n)
        M = x.shape[1]
        out = _LoRAMLP.apply(x.reshape(n * M, -1), *rest)
        return tuple(t.view(n, M, -1) for t in out), (0,) * 6


def lora_mlp(x, gate, up, down, act: str = "silu"):
    """Gated MLP with adapters on all three projections in one autograd node (``act``: ``silu`` or ``gelu_tanh``); each
    of ``gate, up, down`` is ``(weight, A, B, scaling[, bias])``. Projection biases take the composed path."""
    if any(len(p) > 4 and p[4] is not None for p in (gate, up, down)):
        from .functions import opake_geglu, opake_swiglu
        g, u = lora_linear(x, *gate), lora_linear(x, *up)
        h = opake_swiglu(g, u) if act == "silu" else opake_geglu(g, u)
        return lora_linear(h, *down)
    lead = x.shape[:-1]
    y = _LoRAMLP.apply(x.reshape(-1, x.shape[-1]), gate[0], gate[1], gate[2], up[0], up[1], up[2], down[0], down[1], down[2],
                       float(gate[3]), float(up[3]), float(down[3]), "silu" if act == "silu" else "gelu_tanh")[0]
    return y.view(*lead, -1)


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
