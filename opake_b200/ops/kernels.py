"""Functional wrappers over the bandwidth-bound sm_100a kernels (csrc/kernels/elementwise.cu, dp_step.cu).

They replace the reference's Triton kernels (packages/opake-patches/src/opake/api/patches/kernels/:
rms_norm.py, fused_add_rms_norm.py, rope_embedding.py, swiglu.py, geglu.py, cross_entropy.py, _clip_sum.py)
and the eager noise/optimizer math (opake-dpsgd noise/_gaussian.py, opake-optimizers _adam.py).
Every function launches on the current CUDA stream and returns without synchronising.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._protos import DpStepArgs

_bf16 = torch.bfloat16


def _L():
    return _lib.lib()


def _s(t: torch.Tensor) -> int:
    return _lib.stream_ptr(t.device)


def _p(t):
    return None if t is None else t.data_ptr()


def _chk(code: int, name: str) -> None:
    _lib.LAUNCHES[0] += 1
    if code != 0:
        raise _lib.KernelLibraryError(f"{name} failed with code {code}: {_L().opk_last_error().decode()}")


# ------------------------------------------------------------------------------------------------ norms
def rmsnorm_fwd(x, w, eps: float = 1e-6, w_offset: float = 0.0, out=None):
    """``x`` and ``out`` may be column slices of wider row-major matrices (row pitch = ``stride(0)``)."""
    T, D = x.shape
    y = torch.empty_like(x) if out is None else out
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _chk(_L().opk_rmsnorm_fwd_ld(_p(x), x.stride(0), _p(w), _p(y), y.stride(0), _p(rstd), T, D, eps, w_offset, _s(x)),
         "rmsnorm_fwd")
    return y, rstd


def add_rmsnorm_fwd(x, r, w, eps: float = 1e-6, w_offset: float = 0.0):
    T, D = x.shape
    s, y = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _chk(_L().opk_add_rmsnorm_fwd(_p(x), _p(r), _p(w), _p(s), _p(y), _p(rstd), T, D, eps, w_offset, _s(x)),
         "add_rmsnorm_fwd")
    return s, y, rstd


_RMS_WS: dict = {}
_RMS_WS_ROWS = 296


def _rms_workspace(device, D: int) -> torch.Tensor:
    """Per-device scratch for the per-CTA partial weight gradients of the norm backward kernel. Calls on one device
    share it, so they must be ordered on one stream (the model runtimes issue every example on a single stream)."""
    key = device.index
    ws = _RMS_WS.get(key)
    if ws is None or ws.numel() < _RMS_WS_ROWS * D:
        ws = torch.empty(_RMS_WS_ROWS * D, dtype=torch.float32, device=device)
        _RMS_WS[key] = ws
    return ws


def rmsnorm_bwd(dy, x, w, rstd, dres=None, dw=None, w_offset: float = 0.0, out=None):
    """Returns ``dx`` (plus ``dres`` when given); accumulates the weight gradient into fp32 ``dw`` when given."""
    T, D = x.shape
    dx = torch.empty_like(x) if out is None else out
    ws = _rms_workspace(x.device, D) if dw is not None else None
    if dres is not None and dres.stride(0) != dx.stride(0):
        raise ValueError("dres must have the row pitch of the output")
    _chk(_L().opk_rmsnorm_bwd_ld(_p(dy), dy.stride(0), _p(x), x.stride(0), _p(w), _p(rstd), _p(dres), _p(dx), dx.stride(0),
                                 _p(dw), _p(ws), _RMS_WS_ROWS, T, D, w_offset, _s(x)), "rmsnorm_bwd")
    return dx


def layernorm_fwd(x, w, b, eps: float = 1e-5, out=None):
    T, D = x.shape
    y = torch.empty_like(x) if out is None else out
    mean = torch.empty(T, dtype=torch.float32, device=x.device)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _chk(_L().opk_layernorm_fwd(_p(x), _p(w), _p(b), _p(y), _p(mean), _p(rstd), T, D, eps, _s(x)), "layernorm_fwd")
    return y, mean, rstd


def layernorm_bwd(dy, x, w, mean, rstd, dres=None, dw=None, db=None, out=None):
    T, D = x.shape
    dx = torch.empty_like(x) if out is None else out
    _chk(_L().opk_layernorm_bwd(_p(dy), _p(x), _p(w), _p(mean), _p(rstd), _p(dres), _p(dx), _p(dw), _p(db), T, D,
                                _s(x)), "layernorm_bwd")
    return dx


# ------------------------------------------------------------------------------------------------ rope
def rope_table(seq_len: int, head_dim: int, theta: float = 10000.0, device=None, scaling: dict | None = None):
    """``[T, head_dim/2, 2]`` fp32 (cos, sin) table; ``scaling`` implements the Llama-3 frequency rescale."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * torch.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    ang = torch.arange(seq_len, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()


def rope_(qk, table, n_heads: int, head_dim: int, pos=None, backward: bool = False):
    """Rotate the first ``n_heads`` heads of every row of ``qk`` in place (rotate-half convention)."""
    T = qk.shape[0]
    _chk(_L().opk_rope(_p(qk), _p(table), _p(pos), T, n_heads, head_dim, qk.stride(0), -1.0 if backward else 1.0,
                       _s(qk)), "rope")
    return qk


# ------------------------------------------------------------------------------------------------ activations
def swiglu_fwd(gu):
    T, F2 = gu.shape
    act = torch.empty(T, F2 // 2, dtype=_bf16, device=gu.device)
    _chk(_L().opk_swiglu_fwd(_p(gu), _p(act), T, F2 // 2, _s(gu)), "swiglu_fwd")
    return act


def swiglu_bwd(dact, gu, out=None):
    T, F = dact.shape
    dgu = torch.empty_like(gu) if out is None else out
    _chk(_L().opk_swiglu_bwd(_p(dact), _p(gu), _p(dgu), T, F, _s(gu)), "swiglu_bwd")
    return dgu


def geglu_fwd(gu, approximate: bool = True, out=None):
    T, F2 = gu.shape
    act = torch.empty(T, F2 // 2, dtype=_bf16, device=gu.device) if out is None else out
    _chk(_L().opk_geglu_fwd(_p(gu), _p(act), T, F2 // 2, int(approximate), _s(gu)), "geglu_fwd")
    return act


def geglu_bwd(dact, gu, approximate: bool = True, out=None):
    T, F = dact.shape
    dgu = torch.empty_like(gu) if out is None else out
    _chk(_L().opk_geglu_bwd(_p(dact), _p(gu), _p(dgu), T, F, int(approximate), _s(gu)), "geglu_bwd")
    return dgu


def gelu_fwd(x, out=None):
    y = torch.empty_like(x) if out is None else out
    _chk(_L().opk_gelu_fwd(_p(x), _p(y), x.numel(), _s(x)), "gelu_fwd")
    return y


def gelu_bwd(dy, x, out=None):
    dx = torch.empty_like(x) if out is None else out
    _chk(_L().opk_gelu_bwd(_p(dy), _p(x), _p(dx), x.numel(), _s(x)), "gelu_bwd")
    return dx


# ------------------------------------------------------------------------------------------------ embedding
def embedding_fwd(tok, table, pos_table=None, out=None):
    T, D = tok.numel(), table.shape[1]
    if out is None:
        out = torch.empty(T, D, dtype=_bf16, device=table.device)
    _chk(_L().opk_embedding_fwd(_p(tok), _p(table), _p(pos_table), _p(out), T, D, table.shape[0], _s(table)), "embedding_fwd")
    return out


class EmbeddingGradWorkspace:
    """Scratch for the per-example compact embedding gradient (first-occurrence table, fp32 rows)."""

    def __init__(self, vocab: int, max_tokens: int, dim: int, device):
        self.first_pos = torch.full((vocab,), 2**31 - 1, dtype=torch.int32, device=device)
        self.rep = torch.empty(max_tokens, dtype=torch.int32, device=device)
        self.gc = torch.empty(max_tokens, dim, dtype=torch.float32, device=device)


def embedding_bwd_compact(tok, dx, ws: EmbeddingGradWorkspace, sumsq):
    T, D = dx.shape
    _chk(_L().opk_embedding_bwd_compact(_p(tok), _p(dx), _p(ws.first_pos), _p(ws.rep), _p(ws.gc), _p(sumsq), T, D,
                                        ws.first_pos.numel(), _s(dx)), "embedding_bwd_compact")


def embedding_accumulate(tok, ws: EmbeddingGradWorkspace, scale, acc, T: int, shared: bool = False):
    """``acc[tok[t]] += bf16(gc[t] * scale)`` for representative rows. ``shared``: other GPUs add to the same rows at the
    same time (sharded sums; ``acc`` may alias the owner's shard on another GPU), so reductions are used."""
    D = acc.shape[1]
    fn = _L().opk_embedding_accumulate_shared if shared else _L().opk_embedding_accumulate
    _chk(fn(_p(tok), _p(ws.rep), _p(ws.gc), _p(scale), _p(acc), T, D, _s(tok)), "embedding_accumulate")


# ------------------------------------------------------------------------------------------------ losses
def lce_finalize(pmax, psum, tgt, labels):
    T, tiles = pmax.shape
    lse = torch.empty(T, dtype=torch.float32, device=pmax.device)
    nll = torch.empty(T, dtype=torch.float32, device=pmax.device)
    _chk(_L().opk_lce_finalize(_p(pmax), _p(psum), _p(tgt), _p(labels), _p(lse), _p(nll), T, tiles, _s(pmax)),
         "lce_finalize")
    return lse, nll


def rmsnorm_dw_per_example(dy, x, rstd, batch: int):
    """``[batch, D]`` fp32 RMSNorm weight gradients, one per example, of a batch folded into rows (``dy``, ``x``:
    ``[batch * rows, D]`` bf16 contiguous; ``rstd``: ``[batch * rows]``)."""
    D = x.shape[-1]
    rows = x.numel() // D // batch
    dw = torch.zeros(batch, D, dtype=torch.float32, device=x.device)
    _chk(_L().opk_rmsnorm_dw_per_example(_p(dy), _p(x), _p(rstd), _p(dw), batch, rows, D, _s(x)), "rmsnorm_dw_per_example")
    return dw


def loss_coef(labels, nll, coef, loss, ntok=None, weight=None):
    """Mean-over-supervised-tokens loss of one example and the per-token coefficients of its gradient:
    ``coef[t] = (labels[t] >= 0) / max(1, n_supervised)`` (times ``weight``), ``loss = sum(nll * coef)``."""
    _chk(_L().opk_loss_coef(_p(labels), _p(nll), _p(weight), _p(coef), _p(loss), _p(ntok), labels.numel(), _s(nll)), "loss_coef")


def cross_entropy_fwd(logits, labels, scale: float = 1.0, softcap: float = 0.0):
    T, V = logits.shape
    nll = torch.empty(T, dtype=torch.float32, device=logits.device)
    lse = torch.empty(T, dtype=torch.float32, device=logits.device)
    _chk(_L().opk_cross_entropy_fwd(_p(logits), int(logits.dtype == torch.float32), _p(labels), _p(nll), _p(lse), T, V,
                                    logits.stride(0), scale, softcap, _s(logits)), "cross_entropy_fwd")
    return nll, lse


def cross_entropy_bwd(logits, labels, lse, coef, scale: float = 1.0, softcap: float = 0.0):
    T, V = logits.shape
    d = torch.empty_like(logits)
    _chk(_L().opk_cross_entropy_bwd(_p(logits), int(logits.dtype == torch.float32), _p(labels), _p(lse), _p(coef), _p(d),
                                    T, V, logits.stride(0), scale, softcap, _s(logits)), "cross_entropy_bwd")
    return d


# ------------------------------------------------------------------------------------------------ DP primitives
def sumsq_(x, out, round_bf16: bool = False):
    """``out (float64 scalar) += sum(x**2)``."""
    _chk(_L().opk_sumsq(_p(x), int(x.dtype == torch.float32), int(round_bf16), x.numel(), _p(out), _s(x)), "sumsq")


def scatter_rows_cast_sumsq(src, dst_base, offsets, sumsq):
    """fp32 rows ``src[r]`` -> bf16 at ``dst_base + offsets[r]``; ``sumsq += sum(stored**2)``."""
    R, D = src.shape
    _chk(_L().opk_scatter_rows_cast_sumsq(_p(src), _p(dst_base), _p(offsets), R, D, _p(sumsq), _s(src)),
         "scatter_rows_cast_sumsq")


def colsum_(dy, out):
    T, N = dy.shape
    _chk(_L().opk_colsum(_p(dy), _p(out), T, N, dy.stride(0), _s(dy)), "colsum")


def embedding_add_rows(tok, ws, dense, T: int):
    _chk(_L().opk_embedding_add_rows(_p(tok), _p(ws.rep), _p(ws.gc), _p(dense), T, dense.shape[1], _s(dense)),
         "embedding_add_rows")


def cast_f32_bf16(src, dst):
    _chk(_L().opk_cast_f32_bf16(_p(src), _p(dst), src.numel(), _s(src)), "cast_f32_bf16")


def clip_scale(sumsq, clip: float, *, scale_out, norm_out=None, counters=None, auto: bool = False, gamma: float = 0.01,
               n_leaves: int = 1, widest_leaf: int = 1, reset: bool = True):
    _chk(_L().opk_clip_scale(_p(sumsq), clip, int(auto), gamma, n_leaves, widest_leaf, _p(scale_out), _p(norm_out),
                             _p(counters), int(reset), _s(sumsq)), "clip_scale")


def clip_accumulate(g, scale, acc, overwrite: bool = False):
    _chk(_L().opk_clip_accumulate2(_p(g), _p(scale), _p(acc), g.numel(), int(overwrite), _s(g)), "clip_accumulate")


def clip_accumulate_group(gs, scales, acc, overwrite: bool = False):
    """``acc (+)= sum_j stored(gs[j] * scales[j])`` for up to 8 examples in one pass over the fp32 sums."""
    import ctypes

    n = len(gs)
    if not 1 <= n <= 8 or len(scales) != n:
        raise ValueError("a group holds 1 to 8 gradient buffers with one scale each")
    gp = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gs])
    sp = (ctypes.c_void_p * n)(*[t.data_ptr() for t in scales])
    _chk(_L().opk_clip_accumulate_group(gp, sp, n, _p(acc), gs[0].numel(), int(overwrite), _s(acc)), "clip_accumulate_group")


def clip_accumulate_group_push(gs, scales, acc_ptrs: list[int], bounds: list[int], rank: int, n: int):
    """Sharded sums: the group's clipped sum ``sum_j stored(gs[j] * scales[j])`` over the first ``n`` elements is added
    to the owners' shards with reductions (``acc_ptrs[o]`` = device address of owner ``o``'s fp32 shard, peer-mapped for
    remote owners; owner ``o`` holds the elements ``[bounds[o], bounds[o+1])``)."""
    import ctypes

    k = len(gs)
    if not 1 <= k <= 8 or len(scales) != k:
        raise ValueError("a group holds 1 to 8 gradient buffers with one scale each")
    gp = (ctypes.c_void_p * k)(*[g.data_ptr() for g in gs])
    sp = (ctypes.c_void_p * k)(*[t.data_ptr() for t in scales])
    ap = (ctypes.c_void_p * len(acc_ptrs))(*acc_ptrs)
    bp = (ctypes.c_int64 * len(bounds))(*bounds)
    _chk(_L().opk_clip_accumulate_group_push(gp, sp, k, ap, bp, len(acc_ptrs), rank, n, _s(gs[0])), "clip_accumulate_group_push")


def copy_bytes(dst_ptr: int, src_ptr: int, nbytes: int, device) -> None:
    """Copy with the library's own kernel; either address may be peer-mapped memory of another GPU."""
    _chk(_L().opk_copy_bytes(dst_ptr, src_ptr, nbytes, _lib.stream_ptr(device)), "copy_bytes")


def philox_normal_(out, seed: int, step: int, *, stream_id: int = 0, offset: int = 0, sigma: float = 1.0,
                   accumulate: bool = False):
    _chk(_L().opk_philox_normal(_p(out), out.numel(), seed & (2**64 - 1), stream_id, step, offset, sigma,
                                int(accumulate), _s(out)), "philox_normal")
    return out


def dp_step(*, grad_src: list[int], shard_begin: int, shard_len: int, inv_batch: float, sigma: float, seed: int,
            step: int, m, v, master, param_dst: list[int], param_src, lr: float, beta1: float, beta2: float, eps: float,
            weight_decay: float, bc1: float, bc2: float, phi_hat: float, stream_id: int = 0, zero_grad: bool = False,
            blt_state=None, blt_decay=None, blt_scale=None, toep_state=None, toep_coef=None, toep_pos: int = 0,
            sgd_mode: bool = False, device=None):
    """Launch the fused reduce-scatter + noise + DP-AdamW(-BC) + all-gather kernel for this rank's shard.

    ``grad_src`` / ``param_dst`` are raw device addresses (this rank first, then its peers).
    """
    a = DpStepArgs()
    gs = (ctypes.c_void_p * len(grad_src))(*grad_src)
    pd = (ctypes.c_void_p * max(1, len(param_dst)))(*param_dst)
    a.grad_src, a.n_src = gs, len(grad_src)
    a.shard_begin, a.shard_len = shard_begin, shard_len
    a.inv_batch, a.sigma = inv_batch, sigma
    a.seed, a.stream_id, a.step = seed & (2**64 - 1), stream_id, step & 0xFFFFFFFF
    a.m, a.v, a.master = _p(m), _p(v), _p(master)
    a.param_dst, a.n_dst, a.param_src = pd, len(param_dst), _p(param_src)
    a.lr, a.beta1, a.beta2, a.eps, a.weight_decay = lr, beta1, beta2, eps, weight_decay
    a.bc1, a.bc2, a.phi_hat, a.zero_grad = bc1, bc2, phi_hat, int(zero_grad)
    if blt_state is not None:
        a.blt_state, a.blt_nbuf = _p(blt_state), blt_state.shape[0]
        a.blt_decay, a.blt_scale = _p(blt_decay), _p(blt_scale)
    if toep_coef is not None:       # banded Toeplitz C^-1: ring of the last len(coef) - 1 outputs (none for one coefficient)
        a.toep_coef = _p(toep_coef)
        a.toep_nlag = 0 if toep_state is None else toep_state.shape[0]
        a.toep_state, a.toep_pos = _p(toep_state), toep_pos
        if toep_coef.numel() != a.toep_nlag + 1:
            raise ValueError("toep_coef holds one coefficient more than the ring has slots")
    a.sgd_mode = int(sgd_mode)
    dev = device if device is not None else (m.device if m is not None else torch.device("cuda"))
    _chk(_L().opk_dp_step(ctypes.byref(a), _lib.stream_ptr(dev)), "dp_step")


# ------------------------------------------------------------------------------------------------ mixture of experts
class MoePlan:
    """Device-side routing state of one MoE layer invocation (buffers are reused across examples)."""

    def __init__(self, T: int, E: int, k: int, device):
        self.T, self.E, self.k = T, E, k
        self.n = T * k
        self.R = _L().opk_moe_rows_capacity(self.n, E)
        i32 = dict(dtype=torch.int32, device=device)
        self.idx = torch.empty(T, k, **i32)
        self.wts = torch.empty(T, k, dtype=torch.float32, device=device)
        self.probs = torch.empty(T, E, dtype=torch.float32, device=device)
        self.dest = torch.empty(T, k, **i32)
        self.src_entry = torch.empty(self.R, **i32)
        self.tile_group = torch.empty(self.R // 128, **i32)
        self.group_k = torch.empty(E, 2, **i32)
        self.counts = torch.empty(E, **i32)

    def build(self, idx: torch.Tensor) -> "MoePlan":
        """Row plan for expert ids chosen by the caller (``[T, k]`` int32). Ids outside ``[0, E)`` are dropped: their
        ``dest`` entry becomes -1 and the combine kernels skip them."""
        self.idx.copy_(idx.reshape(self.T, self.k))
        _chk(_L().opk_moe_plan(_p(self.idx), self.n, self.E, self.R, _p(self.dest), _p(self.src_entry), _p(self.tile_group),
                               _p(self.group_k), _p(self.counts), _s(self.idx)), "moe_plan")
        return self


def moe_route(logits, plan: MoePlan, norm_topk: bool = False):
    T, E = logits.shape
    _chk(_L().opk_moe_route(_p(logits), logits.stride(0), T, E, plan.k, int(norm_topk), _p(plan.idx), _p(plan.wts), _p(plan.probs),
                            _s(logits)), "moe_route")
    _chk(_L().opk_moe_plan(_p(plan.idx), plan.n, E, plan.R, _p(plan.dest), _p(plan.src_entry), _p(plan.tile_group), _p(plan.group_k),
                           _p(plan.counts), _s(logits)), "moe_plan")
    return plan


def moe_route_bwd(plan: MoePlan, dwts, dlogits, norm_topk: bool = False):
    _chk(_L().opk_moe_route_bwd(_p(plan.probs), _p(plan.idx), _p(dwts), plan.T, plan.E, plan.k, int(norm_topk), _p(dlogits),
                                dlogits.stride(0), _s(dlogits)), "moe_route_bwd")
    return dlogits


def moe_gather(x, plan: MoePlan, out, entry_scale=None):
    _chk(_L().opk_moe_gather(_p(x), x.stride(0), _p(plan.src_entry), plan.k, _p(entry_scale), plan.R, x.shape[1], _p(out), _s(x)),
         "moe_gather")
    return out


def moe_combine(y, plan: MoePlan, out, wts=None, residual=None):
    _chk(_L().opk_moe_combine(_p(y), _p(plan.dest), _p(wts), plan.k, _p(residual), plan.T, y.shape[1], _p(out), _s(y)), "moe_combine")
    return out


def moe_combine_bwd(dy, y, plan: MoePlan, dwts):
    _chk(_L().opk_moe_combine_bwd(_p(dy), _p(y), _p(plan.dest), plan.n, plan.k, y.shape[1], _p(dwts), _s(y)), "moe_combine_bwd")
    return dwts
