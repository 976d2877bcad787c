"""bf16 tensor-core matrix products on the tcgen05 GEMM kernel (csrc/kernels/gemm_sm100.cuh).

All functions take 2-D (or batched 3-D) row-major bf16 CUDA tensors whose row pitch is a multiple of 8 elements
and return bf16. They correspond to the cuBLAS/ATen matmuls the reference runs under ``vmap(grad)``
(reference: packages/opake-patches/src/opake/api/patches/kernels — "everything else on GPU" path).
"""
from __future__ import annotations

import torch

from . import _lib

EPI_STORE, EPI_SUMSQ, EPI_SWIGLU, EPI_LCE_FWD, EPI_LCE_BWD, EPI_SWIGLU_BWD = range(6)


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise TypeError(f"{name}: expected a CUDA bf16 tensor, got {t.dtype} on {t.device}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: last dimension must be contiguous")
    if t.stride(-2) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: row pitch must be a multiple of 8 elements and the base 16-byte aligned")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    alpha: float = 1.0,
    epilogue: int = EPI_STORE,
    sumsq: torch.Tensor | None = None,
    act: torch.Tensor | None = None,
    labels: torch.Tensor | None = None,
    pmax: torch.Tensor | None = None,
    psum: torch.Tensor | None = None,
    tgt: torch.Tensor | None = None,
    lse: torch.Tensor | None = None,
    coef: torch.Tensor | None = None,
    softcap: float = 0.0,
    b_batch_div: int = 1,
    max_ctas: int = 0,
    tile_group: torch.Tensor | None = None,
    group_k: torch.Tensor | None = None,
    sumsq_shared: bool = False,
    norm_only: bool = False,
    stage: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> torch.Tensor | None:
    """General entry: ``out[b] = alpha * op(a[b]) @ op(b[b // b_batch_div])^T`` with an epilogue.

    ``a_mn=False``: ``a`` is ``[M, K]``; ``a_mn=True``: ``a`` is ``[K, M]`` (used as its transpose).
    ``b_mn=False``: ``b`` is ``[N, K]``; ``b_mn=True``: ``b`` is ``[K, N]``.
    """
    _check2d(a, "a")
    _check2d(b, "b")
    batched = a.dim() == 3
    batch = a.shape[0] if batched else 1
    if a_mn:
        K, M = a.shape[-2], a.shape[-1]
    else:
        M, K = a.shape[-2], a.shape[-1]
    if b_mn:
        Kb, N = b.shape[-2], b.shape[-1]
    else:
        N, Kb = b.shape[-2], b.shape[-1]
    if K != Kb:
        raise ValueError(f"reduction sizes differ: {K} vs {Kb}")
    if group_k is not None:
        batch = group_k.shape[0]          # one output per group; operands stay un-batched
    if norm_only and (epilogue != EPI_SUMSQ or out is not None or residual is not None):
        raise ValueError("norm_only: EPI_SUMSQ without an output or residual (only sum(C^2) is produced)")
    need_out = epilogue != EPI_LCE_FWD and not norm_only
    if epilogue == EPI_SWIGLU_BWD and (out is None or act is None or out.shape != act.shape or act.shape[-1] != 2 * N):
        raise ValueError("swiglu backward epilogue: act (saved gate/up pairs) and out must both be [M, 2N]")
    if out is None and need_out:
        shape = (batch, M, N) if (batched or group_k is not None) else (M, N)
        out = torch.empty(shape, dtype=torch.bfloat16, device=a.device)
    args = _lib.GemmArgs()
    args.A, args.B = a.data_ptr(), b.data_ptr()
    args.C = out.data_ptr() if out is not None else None
    if out is not None:
        _check2d(out, "out")
        args.ldc = out.stride(-2)
        args.strideC = out.stride(0) if (batched or group_k is not None) else 0
    if residual is not None:
        if residual.shape != out.shape or residual.stride() != out.stride():
            raise ValueError("residual must have the layout of out")
        args.R = residual.data_ptr()
    args.bias = _lib.ptr(bias)
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.a_mn, args.b_mn, args.epilogue, args.b_batch_div = int(a_mn), int(b_mn), epilogue, b_batch_div
    args.lda, args.ldb = a.stride(-2), b.stride(-2)
    args.strideA = a.stride(0) if batched else 0
    args.strideB = b.stride(0) if b.dim() == 3 else 0
    args.alpha, args.softcap = alpha, softcap
    args.sumsq = _lib.ptr(sumsq)
    if act is not None:
        args.act, args.ld_act = act.data_ptr(), act.stride(-2)
    args.labels, args.pmax, args.psum, args.tgt = map(_lib.ptr, (labels, pmax, psum, tgt))
    args.lse, args.coef = _lib.ptr(lse), _lib.ptr(coef)
    args.err = _lib.err_word(a.device).data_ptr()
    args.max_ctas = max_ctas
    if tile_group is not None:      # row-grouped A / C, B batched per group (mixture of experts forward / dgrad)
        args.tile_group, args.n_groups = tile_group.data_ptr(), b.shape[0]
        args.strideB = b.stride(0)
    if group_k is not None:         # per-batch reduction ranges over un-batched operands (mixture of experts wgrad)
        args.group_k = group_k.data_ptr()
    args.sumsq_shared = int(sumsq_shared)
    if stage is not None:           # b lives on another GPU: (local scratch [N, K] bf16, int32 band counters)
        scratch, ready = stage
        if scratch.numel() < N * K or scratch.dtype != torch.bfloat16 or ready.dtype != torch.int32 or ready.numel() * 2048 < N:
            raise ValueError("stage: scratch must hold N * K bf16 values and the counters one int32 per 2048 rows of b")
        args.stage_dst, args.stage_ready = scratch.data_ptr(), ready.data_ptr()
    _lib.check(_lib.lib().opk_gemm(args, _lib.stream_ptr(a.device)), "opk_gemm")
    return out


def linear_fwd(x: torch.Tensor, w: torch.Tensor, *, bias=None, residual=None, out=None) -> torch.Tensor:
    """``y = x @ w.T (+bias) (+residual)`` with ``x [T, K]``, ``w [N, K]``."""
    return gemm(x, w, out=out, bias=bias, residual=residual)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, *, out=None, residual=None) -> torch.Tensor:
    """``dx = dy @ w`` with ``dy [T, N]``, ``w [N, K]`` (weight consumed in place, no transposed copy)."""
    return gemm(dy, w, b_mn=True, out=out, residual=residual)


def swiglu_dgrad(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor, *, out: torch.Tensor, tile_group=None) -> torch.Tensor:
    """Backward through ``act = silu(gate) * up`` fused into the down projection's data gradient: the accumulator
    ``d_act = dy @ w_down`` (``dy [T, d]``, ``w_down [d, F]``) never reaches memory; the epilogue reads the saved
    interleaved pre-activations ``gu [T, 2F]`` and writes ``out [T, 2F]`` = interleaved ``(d_gate, d_up)``."""
    return gemm(dy, w_down, b_mn=True, out=out, epilogue=EPI_SWIGLU_BWD, act=gu, tile_group=tile_group)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, *, out=None, sumsq: torch.Tensor | None = None) -> torch.Tensor:
    """``dw = dy.T @ x`` with ``dy [T, N]``, ``x [T, K]`` -> ``[N, K]``.

    With ``sumsq`` (a float64 scalar tensor) the kernel also adds ``sum(dw**2)`` of the stored bf16 values to it,
    which is the per-example squared gradient norm contribution of this weight.
    """
    epi = EPI_SUMSQ if sumsq is not None else EPI_STORE
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, epilogue=epi, sumsq=sumsq)


def lce_tiles(n_vocab: int) -> int:
    return _lib.lib().opk_gemm_tiles_n(n_vocab, EPI_LCE_FWD)


def set_pair_mode(on: bool) -> None:
    """Route eligible products (256-wide column tiles, at least 256 rows, no grouped tables) to the two-CTA
    (``cta_group::2``) kernel, or keep everything on the single-CTA kernel. Process-wide; the default is on
    (environment variable ``OPK_GEMM_PAIR=0`` turns it off)."""
    _lib.lib().opk_gemm_set_pair_mode(1 if on else 0)


def pair_mode() -> bool:
    return bool(_lib.lib().opk_gemm_get_pair_mode())
