"""CUDA-graph replay of the per-micro-batch kernel of the generic clipping path.

Counterpart of packages/opake-engine/src/opake/api/engine/clipping/_cuda_graph.py:110-219: graphs are cached by the
structure, shapes, strides, dtypes and devices of the inputs; inputs are copied into static buffers, the graph is
replayed and outputs are cloned. Capture happens on a side stream after ``warmup_runs`` eager runs. At most
``max_graphs`` graphs are kept (least recently used is dropped).
"""
from __future__ import annotations

from collections import OrderedDict
from contextlib import contextmanager
from contextvars import ContextVar

import torch

from ..pytree import tree_flatten, tree_unflatten

_CAPTURING: ContextVar[bool] = ContextVar("opk_capture_safe", default=False)


@contextmanager
def capture_safe_kernels():
    """Within this context kernels must avoid host synchronisation and data-dependent launches."""
    tok = _CAPTURING.set(True)
    try:
        yield
    finally:
        _CAPTURING.reset(tok)


def capture_safe_active() -> bool:
    return _CAPTURING.get()


class CudaGraphChunkCompiler:
    def __init__(self, *, warmup_runs: int = 2, max_graphs: int = 4):
        self.warmup_runs, self.max_graphs = warmup_runs, max_graphs
        self._cache: OrderedDict = OrderedDict()
        self._pool = None

    @staticmethod
    def _key(leaves, td):
        sig = []
        for l in leaves:
            if isinstance(l, torch.Tensor):
                sig.append((tuple(l.shape), tuple(l.stride()), l.dtype, str(l.device), l.requires_grad))
            else:
                sig.append(("py", repr(l)))
        return (td, tuple(sig))

    def wrap(self, fn):
        def run(args, kwargs):
            leaves, td = tree_flatten((args, kwargs))
            tens = [l for l in leaves if isinstance(l, torch.Tensor)]
            if not tens or not all(t.is_cuda for t in tens):
                return fn(args, kwargs)
            key = self._key(leaves, td)
            entry = self._cache.get(key)
            if entry is None:
                entry = self._capture(fn, leaves, td)
                self._cache[key] = entry
                while len(self._cache) > self.max_graphs:
                    self._cache.popitem(last=False)
            else:
                self._cache.move_to_end(key)
            graph, static_in, static_out, out_td = entry
            src = [l for l in leaves if isinstance(l, torch.Tensor)]
            torch._foreach_copy_(static_in, src)
            graph.replay()
            return tree_unflatten(out_td, [o.clone() if isinstance(o, torch.Tensor) else o for o in static_out])

        return run

    def _capture(self, fn, leaves, td):
        static = [l.clone() if isinstance(l, torch.Tensor) else l for l in leaves]
        s_args, s_kwargs = tree_unflatten(td, static)
        dev = next(l.device for l in leaves if isinstance(l, torch.Tensor))
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), capture_safe_kernels():
            for _ in range(self.warmup_runs):
                fn(s_args, s_kwargs)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self._pool, stream=side), capture_safe_kernels():
            out = fn(s_args, s_kwargs)
        out_leaves, out_td = tree_flatten(out)
        return graph, [l for l in static if isinstance(l, torch.Tensor)], out_leaves, out_td


__all__ = ["CudaGraphChunkCompiler", "capture_safe_kernels", "capture_safe_active"]
