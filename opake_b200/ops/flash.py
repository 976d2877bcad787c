"""Python entry points of the tcgen05 flash-attention kernels (csrc/kernels/attention_sm100.cuh)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float


def _fn(name, argtypes):
    f = getattr(_lib.lib(), name)
    f.restype = _I
    f.argtypes = argtypes
    return f


def flash_fwd(qkv: torch.Tensor, H: int, KV: int, hd: int, out: torch.Tensor | None = None):
    """Causal GQA attention over the fused projection buffer. Returns ``(out [T, H*hd], lse [H, T])``."""
    T = qkv.shape[0]
    if out is None:
        out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(H, T, dtype=torch.float32, device=qkv.device)
    f = _fn("opk_attn_fwd", [_P, _P, _P, _I, _I, _I, _I, _L, _L, _F, _P, _P])
    rc = f(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), T, H, KV, hd, qkv.stride(0), out.stride(0), hd**-0.5,
           _lib.err_word(qkv.device).data_ptr(), _lib.stream_ptr(qkv.device))
    _lib.check(rc, "opk_attn_fwd")
    return out, lse


def flash_bwd(dout, qkv, out, lse, H: int, KV: int, hd: int, dqkv: torch.Tensor, split_heads: bool = True):
    """Gradient with respect to the fused projection buffer (dQ, dK, dV written into ``dqkv``)."""
    T = qkv.shape[0]
    t64 = (T + 63) // 64 * 64
    dsum = torch.empty(2, H, t64, dtype=torch.float32, device=qkv.device)   # rowsum(dO*O), then -lse*log2(e)
    part = None
    if H > KV and split_heads:
        part = torch.empty(2 * (H // KV) * T * KV * hd, dtype=torch.float32, device=qkv.device)
    f = _fn("opk_attn_bwd", [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _F, _P, _P])
    rc = f(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), dsum.data_ptr(), dqkv.data_ptr(),
           None if part is None else part.data_ptr(), T, H, KV, hd,
           qkv.stride(0), out.stride(0), hd**-0.5, _lib.err_word(qkv.device).data_ptr(), _lib.stream_ptr(qkv.device))
    _lib.check(rc, "opk_attn_bwd")
    return dqkv
