"""Fused linear + cross-entropy: per-token NLL of ``hidden @ weight.T`` without materialising fp32 logits.

Counterpart of ``opake_linear_cross_entropy_loss`` (packages/opake-patches/src/opake/api/patches/kernels/
linear_cross_entropy.py:1223-1276, kernels :101-247 and :292-528). The reference tiles the vocabulary inside a Triton
program and merges partial log-sum-exps under a spin lock; here the vocabulary GEMM runs on the tcgen05 kernel with
two epilogues: the forward epilogue reduces every 128-column tile to (max, sum-exp, target logit) per row, a tiny
finalize kernel merges the tiles, and the backward epilogue recomputes the logits tile and writes
``coef * (softmax - onehot)`` in bf16, from which dH and dW are two more GEMMs.

Both directions are ``torch.autograd.Function`` objects with ``vmap`` rules so that ``vmap(grad(loss))`` works: a
batch of examples sharing one weight is flattened into rows for the forward and dH; the per-example weight gradient
is one batched GEMM (packages/opake-patches/src/opake/api/patches/kernels/linear_cross_entropy.py:772-779 allocates
the same ``(B, V, D)`` result).
"""
from __future__ import annotations

import torch

IGNORE_INDEX = -100


def native_available(hidden: torch.Tensor, weight: torch.Tensor) -> bool:
    return (hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and hidden.shape[-1] % 8 == 0)


# ------------------------------------------------------------------------------------------- plain-torch fallback
def _chunked_nll(hidden, weight, labels, logit_scale, softcap, chunk: int = 4096):
    """Per-token NLL in fp32, differentiable, ``chunk`` rows at a time (portable path, CPU included)."""
    out = []
    for s in range(0, hidden.shape[0], chunk):
        h = hidden[s:s + chunk]
        lab = labels[s:s + chunk]
        logits = (h.to(torch.float32) @ weight.to(torch.float32).t()) * logit_scale
        if softcap:
            logits = softcap * torch.tanh(logits / softcap)
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(-1, lab.clamp(min=0).unsqueeze(-1)).squeeze(-1)
        out.append(torch.where(lab >= 0, lse - tgt, torch.zeros_like(lse)))
    return torch.cat(out) if out else hidden.new_zeros(0, dtype=torch.float32)


# ------------------------------------------------------------------------------------------- native forward
def _native_fwd(hidden, weight, labels, logit_scale, softcap):
    from . import gemm as G, kernels as K
    T = hidden.shape[0]
    tiles = G.lce_tiles(weight.shape[0])
    pmax = torch.empty(T, tiles, dtype=torch.float32, device=hidden.device)
    psum = torch.empty_like(pmax)
    tgt = torch.empty(T, dtype=torch.float32, device=hidden.device)
    lab = labels.to(torch.int32).contiguous()
    G.gemm(hidden, weight, epilogue=G.EPI_LCE_FWD, labels=lab, pmax=pmax, psum=psum, tgt=tgt, alpha=logit_scale,
           softcap=softcap)
    lse, nll = K.lce_finalize(pmax, psum, tgt, lab)
    return nll, lse, lab


def _native_dlogits(hidden, weight, lab, lse, coef, logit_scale, softcap):
    from . import gemm as G
    T, V = hidden.shape[0], weight.shape[0]
    Vp = (V + 7) // 8 * 8
    dlog = torch.empty(T, Vp, dtype=torch.bfloat16, device=hidden.device)[:, :V]
    G.gemm(hidden, weight, out=dlog, epilogue=G.EPI_LCE_BWD, labels=lab, lse=lse, coef=coef.contiguous(),
           alpha=logit_scale, softcap=softcap)
    return dlog


class _LinearCEBackward(torch.autograd.Function):
    """Backward of the fused loss as its own Function so that it can carry a vmap rule (per-example dW)."""

    @staticmethod
    def forward(grad_nll, hidden, weight, lab, lse, logit_scale, softcap):
        from . import gemm as G
        coef = (grad_nll.to(torch.float32) * (lab >= 0)).contiguous()
        dlog = _native_dlogits(hidden, weight, lab, lse, coef, logit_scale, softcap)
        # dlog is the gradient with respect to logit_scale * (hidden @ weight.T)
        d_hidden = G.gemm(dlog, weight, b_mn=True, alpha=logit_scale)
        d_weight = G.linear_wgrad(dlog, hidden)
        if logit_scale != 1.0:
            d_weight = d_weight * logit_scale
        return d_hidden, d_weight

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.set_materialize_grads(False)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("second-order differentiation of the fused linear cross-entropy is not supported")

    @staticmethod
    def vmap(info, in_dims, grad_nll, hidden, weight, lab, lse, logit_scale, softcap):
        from . import gemm as G
        if in_dims[2] is not None:
            raise NotImplementedError("fused linear cross-entropy under vmap needs one shared weight")
        B = info.batch_size

        def front(x, d):
            return x.movedim(d, 0) if d is not None else x.unsqueeze(0).expand(B, *x.shape)

        g, h, lb, ls = (front(x, d) for x, d in zip((grad_nll, hidden, lab, lse), (in_dims[0], in_dims[1], in_dims[3], in_dims[4])))
        T, D = h.shape[1], h.shape[2]
        hf = h.reshape(B * T, D).contiguous()
        labf = lb.reshape(B * T).contiguous()
        coef = (g.to(torch.float32).reshape(B * T) * (labf >= 0)).contiguous()
        dlog = _native_dlogits(hf, weight, labf, ls.reshape(B * T).contiguous(), coef, logit_scale, softcap)
        d_hidden = G.gemm(dlog, weight, b_mn=True, alpha=logit_scale).view(B, T, D)
        V = weight.shape[0]
        d_weight = torch.empty(B, V, D, dtype=torch.bfloat16, device=hidden.device)
        G.gemm(dlog.view(B, T, -1), hf.view(B, T, D), a_mn=True, b_mn=True, out=d_weight)
        if logit_scale != 1.0:
            d_weight = d_weight * logit_scale
        return (d_hidden, d_weight), (0, 0)


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(hidden, weight, labels, logit_scale, softcap):
        nll, lse, lab = _native_fwd(hidden.contiguous(), weight, labels, logit_scale, softcap)
        return nll, lse, lab

    @staticmethod
    def setup_context(ctx, inputs, output):
        hidden, weight, _labels, logit_scale, softcap = inputs
        _nll, lse, lab = output
        ctx.save_for_backward(hidden, weight, lab, lse)
        ctx.mark_non_differentiable(lse, lab)
        ctx.logit_scale, ctx.softcap = logit_scale, softcap

    @staticmethod
    def backward(ctx, g_nll, _g_lse, _g_lab):
        hidden, weight, lab, lse = ctx.saved_tensors
        d_hidden, d_weight = _LinearCEBackward.apply(g_nll, hidden, weight, lab, lse, ctx.logit_scale, ctx.softcap)
        return d_hidden, d_weight, None, None, None

    @staticmethod
    def vmap(info, in_dims, hidden, weight, labels, logit_scale, softcap):
        if in_dims[1] is not None:
            raise NotImplementedError("fused linear cross-entropy under vmap needs one shared weight")
        B = info.batch_size
        h = hidden.movedim(in_dims[0], 0) if in_dims[0] is not None else hidden.unsqueeze(0).expand(B, *hidden.shape)
        lb = labels.movedim(in_dims[2], 0) if in_dims[2] is not None else labels.unsqueeze(0).expand(B, *labels.shape)
        T, D = h.shape[1], h.shape[2]
        nll, lse, lab = _native_fwd(h.reshape(B * T, D).contiguous(), weight, lb.reshape(B * T), logit_scale, softcap)
        return (nll.view(B, T), lse.view(B, T), lab.view(B, T)), (0, 0, 0)


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, *, logit_scale: float = 1.0,
                         logit_softcapping: float = 0.0, use_token_scaling: bool = False,
                         force_portable: bool = False) -> torch.Tensor:
    """Per-token NLL (fp32, zero where ``labels < 0``) of ``softmax(logit_scale * hidden @ weight.T)``.

    ``hidden`` is ``[T, D]``, ``weight`` ``[V, D]``, ``labels`` ``[T]`` already aligned with ``hidden`` (the caller
    shifts). ``use_token_scaling`` multiplies each token's loss by its detached target probability (the DFT
    objective, packages/opake-alignment/src/opake/api/alignment/sft/loss/_dft.py:43-88).
    """
    if hidden.dim() != 2:
        raise ValueError("hidden must be [T, D]; flatten leading dimensions first")
    if not force_portable and native_available(hidden, weight):
        nll, _lse, _lab = _LinearCE.apply(hidden, weight, labels, float(logit_scale), float(logit_softcapping))
    else:
        nll = _chunked_nll(hidden, weight, labels, float(logit_scale), float(logit_softcapping))
    if use_token_scaling:
        nll = nll * torch.exp(-nll).detach()
    return nll


def opake_linear_cross_entropy_loss(hidden_states, weight, labels, ignore_index: int = IGNORE_INDEX,
                                    logit_softcapping: float = 0, label_smoothing: float = 0.0,
                                    use_token_scaling: bool = False, logit_scale: float = 1.0) -> torch.Tensor:
    """Reference-shaped entry (packages/opake-patches/src/opake/api/patches/kernels/linear_cross_entropy.py:1223):
    ``hidden_states [..., L, D]`` and ``labels [..., L]`` in Hugging Face layout (position t predicts t+1); returns
    the per-sequence **sum** of token losses, shape ``[...]``."""
    if label_smoothing:
        raise NotImplementedError("label smoothing is not implemented in the fused linear cross-entropy")
    lead = hidden_states.shape[:-2]
    L, D = hidden_states.shape[-2:]
    h = hidden_states[..., :-1, :].reshape(-1, D)
    lab = labels[..., 1:]
    lab = torch.where(lab == ignore_index, torch.full_like(lab, -1), lab).reshape(-1)
    nll = linear_cross_entropy(h, weight, lab, logit_scale=logit_scale, logit_softcapping=logit_softcapping,
                               use_token_scaling=use_token_scaling)
    return nll.view(*lead, L - 1).sum(-1)
