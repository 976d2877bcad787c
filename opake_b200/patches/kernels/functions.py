"""vmap-safe autograd wrappers around the sm_100a row kernels (packages/opake-patches/src/opake/api/patches/kernels/
rms_norm.py:74-373, fused_add_rms_norm.py:68-134, swiglu.py:31-130, geglu.py:39-330, cross_entropy.py:29-236,629-704,
rope_embedding.py:50-215).

Every op is two ``torch.autograd.Function`` objects, forward and backward, each with a ``vmap`` rule, so that
``vmap(grad(loss))`` and double vmap work. The kernels act on rows, so a vmapped batch is handled by folding the batch
dimension into the row dimension: ONE launch for the whole batch. Only parameter gradients differ under vmap: they
must stay per example, and are reduced per example instead of over all rows. Inputs that are not CUDA bf16 take the
plain-PyTorch formulas (same math, used on CPU and as the numerical reference in the tests).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = ["opake_rms_norm", "opake_fused_add_rms_norm", "opake_swiglu", "opake_geglu", "opake_cross_entropy",
           "opake_selective_log_softmax", "opake_rope_qk", "native_rows"]


def native_rows(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def _front(x, d, B):
    if d is None:
        return x.unsqueeze(0).expand(B, *x.shape)
    return x.movedim(d, 0)


# =============================================================================================== RMSNorm
def _rms_ref(x, w, eps, offset):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + offset)
    return y.to(x.dtype)


class _RMSNormBwd(torch.autograd.Function):
    @staticmethod
    def forward(dy, x, w, rstd, offset):
        from ...ops import kernels as K
        D = x.shape[-1]
        dw = torch.zeros(D, dtype=torch.float32, device=x.device)
        dx = K.rmsnorm_bwd(dy.reshape(-1, D).contiguous(), x.reshape(-1, D).contiguous(), w, rstd.reshape(-1), dw=dw, w_offset=offset)
        return dx.view_as(x), dw.to(w.dtype)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused RMSNorm is not supported")

    @staticmethod
    def vmap(info, in_dims, dy, x, w, rstd, offset):
        from ...ops import kernels as K
        if in_dims[2] is not None:
            raise NotImplementedError("per-example norm weights are not supported")
        B = info.batch_size
        dy, x, rstd = _front(dy, in_dims[0], B), _front(x, in_dims[1], B), _front(rstd, in_dims[3], B)
        D = x.shape[-1]
        dx = K.rmsnorm_bwd(dy.reshape(-1, D).contiguous(), x.reshape(-1, D).contiguous(), w, rstd.reshape(-1).contiguous(),
                           dw=None, w_offset=offset).view_as(x)
        # the weight gradient stays per example: one reduction kernel over each example's rows
        # (packages/opake-patches/src/opake/api/patches/kernels/rms_norm.py:292-373)
        dw = K.rmsnorm_dw_per_example(dy.reshape(-1, D).contiguous(), x.reshape(-1, D).contiguous(),
                                      rstd.reshape(-1).contiguous(), B).to(w.dtype)
        return (dx, dw), (0, 0)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(x, w, eps, offset):
        from ...ops import kernels as K
        D = x.shape[-1]
        y, rstd = K.rmsnorm_fwd(x.reshape(-1, D).contiguous(), w, eps, offset)
        return y.view_as(x), rstd.view(x.shape[:-1])

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, w, _eps, offset = inputs
        ctx.save_for_backward(x, w, output[1])
        ctx.mark_non_differentiable(output[1])
        ctx.offset = offset

    @staticmethod
    def backward(ctx, dy, _drstd):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _RMSNormBwd.apply(dy.contiguous(), x, w, rstd, ctx.offset)
        return dx, dw, None, None

    @staticmethod
    def vmap(info, in_dims, x, w, eps, offset):
        if in_dims[1] is not None:
            raise NotImplementedError("per-example norm weights are not supported")
        x = _front(x, in_dims[0], info.batch_size)
        y, rstd = _RMSNorm.apply(x, w, eps, offset)
        return (y, rstd), (0, 0)


def opake_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * (weight + offset)`` over the last dimension (``offset = 1`` is the Gemma form)."""
    if native_rows(x) and weight.dtype == torch.bfloat16:
        return _RMSNorm.apply(x, weight, float(eps), float(offset))[0]
    return _rms_ref(x, weight, eps, offset)


class _AddRMSNormBwd(torch.autograd.Function):
    """``d(x) = d(residual) = ds + d(rmsnorm)/d(sum)``: the residual gradient is added inside the norm-backward kernel."""

    @staticmethod
    def forward(dy, ds, s, w, rstd, offset):
        from ...ops import kernels as K
        D = s.shape[-1]
        dw = torch.zeros(D, dtype=torch.float32, device=s.device)
        dx = K.rmsnorm_bwd(dy.reshape(-1, D).contiguous(), s.reshape(-1, D).contiguous(), w, rstd.reshape(-1),
                           dres=ds.reshape(-1, D).contiguous(), dw=dw, w_offset=offset)
        return dx.view_as(s), dw.to(w.dtype)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused add + RMSNorm is not supported")

    @staticmethod
    def vmap(info, in_dims, dy, ds, s, w, rstd, offset):
        from ...ops import kernels as K
        if in_dims[3] is not None:
            raise NotImplementedError("per-example norm weights are not supported")
        B = info.batch_size
        dy, ds, s, rstd = (_front(t, d, B) for t, d in zip((dy, ds, s, rstd), (in_dims[0], in_dims[1], in_dims[2], in_dims[4])))
        D = s.shape[-1]
        dy2, s2, r1 = dy.reshape(-1, D).contiguous(), s.reshape(-1, D).contiguous(), rstd.reshape(-1).contiguous()
        dx = K.rmsnorm_bwd(dy2, s2, w, r1, dres=ds.reshape(-1, D).contiguous(), dw=None, w_offset=offset).view_as(s)
        dw = K.rmsnorm_dw_per_example(dy2, s2, r1, B).to(w.dtype)
        return (dx, dw), (0, 0)


class _AddRMSNorm(torch.autograd.Function):
    """``s = x + residual; y = rmsnorm(s)`` in one kernel (packages/opake-patches/src/opake/api/patches/kernels/
    fused_add_rms_norm.py:68-134); returns ``(y, s, rstd)``."""

    @staticmethod
    def forward(x, residual, w, eps, offset):
        from ...ops import kernels as K
        D = x.shape[-1]
        s, y, rstd = K.add_rmsnorm_fwd(x.reshape(-1, D).contiguous(), residual.reshape(-1, D).contiguous(), w, eps, offset)
        return y.view_as(x), s.view_as(x), rstd.view(x.shape[:-1])

    @staticmethod
    def setup_context(ctx, inputs, output):
        _x, _r, w, _eps, offset = inputs
        ctx.save_for_backward(output[1], w, output[2])
        ctx.mark_non_differentiable(output[2])
        ctx.offset = offset

    @staticmethod
    def backward(ctx, dy, ds, _drstd):
        s, w, rstd = ctx.saved_tensors
        if ds is None:
            ds = torch.zeros_like(s)
        if dy is None:
            dy = torch.zeros_like(s)
        dx, dw = _AddRMSNormBwd.apply(dy.contiguous(), ds.contiguous(), s, w, rstd, ctx.offset)
        return dx, dx, dw, None, None

    @staticmethod
    def vmap(info, in_dims, x, residual, w, eps, offset):
        if in_dims[2] is not None:
            raise NotImplementedError("per-example norm weights are not supported")
        B = info.batch_size
        x, residual = _front(x, in_dims[0], B), _front(residual, in_dims[1], B)
        y, s, rstd = _AddRMSNorm.apply(x, residual, w, eps, offset)
        return (y, s, rstd), (0, 0, 0)


def opake_fused_add_rms_norm(x, residual, weight, eps: float = 1e-6, offset: float = 0.0):
    """Returns ``(normed, new_residual)`` with ``new_residual = x + residual``; one kernel forward, and the residual
    gradient is folded into the norm's backward kernel."""
    if native_rows(x) and residual.dtype == x.dtype and residual.shape == x.shape and weight.dtype == torch.bfloat16:
        y, s, _ = _AddRMSNorm.apply(x, residual, weight, float(eps), float(offset))
        return y, s
    s = x + residual
    return opake_rms_norm(s, weight, eps, offset), s


# =============================================================================================== gated activations
def _interleave(gate, up):
    return torch.stack([gate, up], dim=-1).reshape(*gate.shape[:-1], 2 * gate.shape[-1])


class _GluBwd(torch.autograd.Function):
    @staticmethod
    def forward(dact, gu, kind):
        from ...ops import kernels as K
        F2 = gu.shape[-1]
        d2, g2 = dact.reshape(-1, F2 // 2).contiguous(), gu.reshape(-1, F2).contiguous()
        out = K.swiglu_bwd(d2, g2) if kind == 0 else K.geglu_bwd(d2, g2, approximate=(kind == 2))
        return out.view_as(gu)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused gated activation is not supported")

    @staticmethod
    def vmap(info, in_dims, dact, gu, kind):
        B = info.batch_size
        return _GluBwd.apply(_front(dact, in_dims[0], B).contiguous(), _front(gu, in_dims[1], B).contiguous(), kind), 0


class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(gu, kind):
        from ...ops import kernels as K
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2).contiguous()
        out = K.swiglu_fwd(g2) if kind == 0 else K.geglu_fwd(g2, approximate=(kind == 2))
        return out.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(inputs[0])
        ctx.kind = inputs[1]

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        return _GluBwd.apply(dact.contiguous(), gu, ctx.kind), None

    @staticmethod
    def vmap(info, in_dims, gu, kind):
        return _Glu.apply(_front(gu, in_dims[0], info.batch_size).contiguous(), kind), 0


def opake_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up``."""
    if native_rows(gate) and gate.shape == up.shape:
        return _Glu.apply(_interleave(gate, up), 0)
    return F.silu(gate) * up


def opake_geglu(gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    """``gelu(gate) * up`` (exact or tanh approximation)."""
    if native_rows(gate) and gate.shape == up.shape:
        return _Glu.apply(_interleave(gate, up), 2 if approximate == "tanh" else 1)
    return F.gelu(gate, approximate=approximate) * up


# =============================================================================================== cross entropy
class _CEBwd(torch.autograd.Function):
    @staticmethod
    def forward(g, logits, labels, lse, scale, softcap):
        from ...ops import kernels as K
        V = logits.shape[-1]
        coef = (g.reshape(-1).float() * (labels.reshape(-1) >= 0)).contiguous()
        d = K.cross_entropy_bwd(logits.reshape(-1, V), labels.reshape(-1), lse.reshape(-1), coef, scale, softcap)
        return d.view_as(logits)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise NotImplementedError("double backward through the fused cross-entropy is not supported")

    @staticmethod
    def vmap(info, in_dims, g, logits, labels, lse, scale, softcap):
        B = info.batch_size
        args = [_front(t, d, B).contiguous() for t, d in zip((g, logits, labels, lse), in_dims[:4])]
        return _CEBwd.apply(*args, scale, softcap), 0


class _CE(torch.autograd.Function):
    @staticmethod
    def forward(logits, labels, scale, softcap):
        from ...ops import kernels as K
        V = logits.shape[-1]
        lab = labels.reshape(-1).to(torch.int32).contiguous()
        nll, lse = K.cross_entropy_fwd(logits.reshape(-1, V), lab, scale, softcap)
        return nll.view(labels.shape), lse.view(labels.shape), lab.view(labels.shape)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(inputs[0], output[2], output[1])
        ctx.mark_non_differentiable(output[1], output[2])
        ctx.scale, ctx.softcap = inputs[2], inputs[3]

    @staticmethod
    def backward(ctx, g, _g1, _g2):
        logits, lab, lse = ctx.saved_tensors
        return _CEBwd.apply(g.contiguous(), logits, lab, lse, ctx.scale, ctx.softcap), None, None, None

    @staticmethod
    def vmap(info, in_dims, logits, labels, scale, softcap):
        B = info.batch_size
        out = _CE.apply(_front(logits, in_dims[0], B).contiguous(), _front(labels, in_dims[1], B).contiguous(), scale, softcap)
        return out, (0, 0, 0)


def opake_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100, logit_scale: float = 1.0,
                        logit_softcapping: float = 0.0) -> torch.Tensor:
    """Per-position NLL (fp32; zero where ``labels == ignore_index``) of row-wise softmax over the last dimension."""
    lab = torch.where(labels == ignore_index, torch.full_like(labels, -1), labels)
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(-1) == 1 and logits.is_contiguous():
        return _CE.apply(logits, lab, float(logit_scale), float(logit_softcapping))[0]
    z = logits.float() * logit_scale
    if logit_softcapping:
        z = logit_softcapping * torch.tanh(z / logit_softcapping)
    nll = torch.logsumexp(z, -1) - z.gather(-1, lab.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    return torch.where(lab >= 0, nll, torch.zeros_like(nll))


def opake_selective_log_softmax(logits: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., indices]``: minus the cross entropy against ``indices``."""
    return -opake_cross_entropy(logits, indices, ignore_index=-(2**31))


# =============================================================================================== RoPE
class _RopeQK(torch.autograd.Function):
    """Rotates q and k heads of a fused ``[rows, (Hq + Hk) * hd]`` buffer (rotate-half); backward = inverse rotation."""

    @staticmethod
    def forward(qk, table, n_heads, head_dim, sign):
        from ...ops import kernels as K
        out = qk.clone()
        K.rope_(out.view(-1, out.shape[-1]), table, n_heads, head_dim, backward=(sign < 0))
        return out

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(inputs[1])
        ctx.n_heads, ctx.head_dim, ctx.sign = inputs[2], inputs[3], inputs[4]

    @staticmethod
    def backward(ctx, g):
        (table,) = ctx.saved_tensors
        return _RopeQK.apply(g.contiguous(), table, ctx.n_heads, ctx.head_dim, -ctx.sign), None, None, None, None

    @staticmethod
    def vmap(info, in_dims, qk, table, n_heads, head_dim, sign):
        if in_dims[1] is not None:
            raise NotImplementedError("per-example rotary tables are not supported")
        qk = _front(qk, in_dims[0], info.batch_size).contiguous()          # [B, T, C]: the table indexes T
        outs = [_RopeQK.apply(qk[b], table, n_heads, head_dim, sign) for b in range(qk.shape[0])]
        return torch.stack(outs), 0


def opake_rope_qk(qk: torch.Tensor, table: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """``qk`` is ``[T, n_heads * head_dim (+ untouched columns)]``; ``table`` the ``[T, head_dim/2, 2]`` cos/sin table."""
    if native_rows(qk):
        return _RopeQK.apply(qk.contiguous(), table, int(n_heads), int(head_dim), 1.0)
    T = qk.shape[-2]
    x = qk[..., : n_heads * head_dim].reshape(*qk.shape[:-1], n_heads, head_dim)
    cos = torch.cat([table[:T, :, 0], table[:T, :, 0]], -1)[:, None, :].to(x.dtype)
    sin = torch.cat([table[:T, :, 1], table[:T, :, 1]], -1)[:, None, :].to(x.dtype)
    rot = torch.cat([-x[..., head_dim // 2:], x[..., : head_dim // 2]], -1)
    y = (x * cos + rot * sin).reshape(*qk.shape[:-1], n_heads * head_dim)
    return torch.cat([y, qk[..., n_heads * head_dim:]], -1)
