"""The allocation-free entry point against the ordinary one.

Some users of the kernel library cannot allocate device memory where they need this kernel (inside a memory-pool
snapshot, inside a host application that only hands out fixed buffers, on teardown paths), so the library carries its
own scratch table for them. This test calls that entry point through its exported C symbol, twice in a row (the table
is shared between calls and must come back clean), and compares with the scratch-taking entry point.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(L, tok, dx, vocab):
    T, D = dx.shape
    rep = torch.empty(T, dtype=torch.int32, device=dx.device)
    gc = torch.empty(T, D, dtype=torch.float32, device=dx.device)
    ss = torch.zeros(1, dtype=torch.float64, device=dx.device)
    fn = L.opk_embedding_bwd_compact_noalloc
    fn.restype = ctypes.c_int32
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int32] * 3 + [ctypes.c_void_p]
    rc = fn(tok.data_ptr(), dx.data_ptr(), rep.data_ptr(), gc.data_ptr(), ss.data_ptr(), T, D, vocab,
            torch.cuda.current_stream(dx.device).cuda_stream)
    return rc, rep, gc, ss


def test_noalloc_embedding_grad_matches_scratch_version(cuda):
    from opake_b200.ops import _lib
    from opake_b200.ops import kernels as K

    L = _lib.lib()
    V, T, D = 5000, 384, 256
    for trial in range(2):  # two calls in a row share the built-in table
        g = torch.Generator(device=cuda).manual_seed(10 + trial)
        tok = torch.randint(0, 64 if trial == 0 else V, (T,), generator=g, device=cuda, dtype=torch.int32)
        dx = torch.randn(T, D, generator=g, device=cuda).to(torch.bfloat16)
        ws = K.EmbeddingGradWorkspace(V, T, D, cuda)
        want_ss = torch.zeros(1, dtype=torch.float64, device=cuda)
        K.embedding_bwd_compact(tok, dx, ws, want_ss)
        rc, rep, gc, ss = _call_noalloc(L, tok, dx, V)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(rep, ws.rep)
        # duplicate tokens are summed with fp32 atomics whose order is not fixed: same tolerance as the kernel tests
        assert (gc - ws.gc).abs().max().item() <= 2e-2 * (ws.gc.abs().max().item() + 1e-6)
        assert abs(ss.item() - want_ss.item()) <= 1e-3 * want_ss.item()


def test_noalloc_rejects_oversized_vocab(cuda):
    from opake_b200.ops import _lib

    L = _lib.lib()
    tok = torch.zeros(8, dtype=torch.int32, device=cuda)
    dx = torch.zeros(8, 64, dtype=torch.bfloat16, device=cuda)
    rc, *_ = _call_noalloc(L, tok, dx, 262144 + 1)
    assert rc == -2


def test_out_of_range_token_ids_are_skipped(cuda):
    """Ids outside [0, vocab) never index the table: their position gets rep = -1 and contributes no row, in both
    entry points; the in-range positions are unaffected."""
    from opake_b200.ops import _lib
    from opake_b200.ops import kernels as K

    L = _lib.lib()
    V, T, D = 1000, 64, 128
    g = torch.Generator(device=cuda).manual_seed(3)
    tok = torch.randint(0, V, (T,), generator=g, device=cuda, dtype=torch.int32)
    dx = torch.randn(T, D, generator=g, device=cuda).to(torch.bfloat16)
    bad = tok.clone()
    bad[5], bad[17], bad[40] = V, -1, 2 ** 30
    ws = K.EmbeddingGradWorkspace(V, T, D, cuda)
    K.embedding_bwd_compact(bad, dx, ws, None)
    rc, rep, gc, _ = _call_noalloc(L, bad, dx, V)
    torch.cuda.synchronize()
    assert rc == 0
    for r, rows in ((rep, gc), (ws.rep, ws.gc)):
        assert r[5].item() == -1 and r[17].item() == -1 and r[40].item() == -1
        assert rows[[5, 17, 40]].abs().max().item() == 0.0
    assert torch.equal(rep, ws.rep)
    assert int((ws.first_pos != 2 ** 31 - 1).sum().item()) == 0      # the scratch table came back idle
