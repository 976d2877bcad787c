"""Activation checkpointing under ``vmap(grad)`` (packages/opake-patches/src/opake/api/patches/torch/checkpoint/
__init__.py:38-64: saved_tensor_hooks_guard, save_on_cpu, noop_save_inputs, create_graph, reparametrize_recompute,
huggingface, native_support).

Non-reentrant ``torch.utils.checkpoint`` stores tensors through saved-tensor hooks; inside functorch transforms the
stored objects are wrapped (batched / grad-tracking) tensors, and recomputation has to happen at the same transform
level. ``checkpoint_under_vmap`` is a functional checkpoint that sidesteps the hooks: it is an ``autograd.Function``
-free formulation where the segment is simply re-run inside the backward of a ``torch.func.vjp``, which composes
with ``vmap`` and ``grad``. ``offload_activations`` moves what a segment saves to pinned host memory and brings it back
for the backward pass (the ``save_on_cpu`` behaviour) for the eager per-example path."""
from __future__ import annotations

import contextlib
from typing import Callable

import torch

__all__ = ["checkpoint_under_vmap", "native_support", "offload_activations", "apply_gradient_checkpointing"]


def native_support() -> bool:
    """Whether this PyTorch runs non-reentrant checkpoint inside functorch transforms without help."""
    try:
        from torch.utils.checkpoint import checkpoint

        def f(w, x):
            return checkpoint(lambda a: torch.tanh(a * w).sum(), x, use_reentrant=False)

        torch.func.vmap(torch.func.grad(f), in_dims=(None, 0))(torch.ones(3), torch.ones(2, 3))
        return True
    except Exception:
        return False


def checkpoint_under_vmap(fn: Callable, *args):
    """Runs ``fn(*args)`` keeping only its inputs; the backward pass recomputes the segment. Implemented with a
    custom ``autograd.Function`` whose backward calls ``torch.func.vjp`` on ``fn`` (``generate_vmap_rule`` lets the
    whole thing sit under vmap)."""
    tensors = [a for a in args if isinstance(a, torch.Tensor)]
    if not tensors or not any(t.requires_grad or torch._C._functorch.is_gradtrackingtensor(t) for t in tensors):
        return fn(*args)

    class _Segment(torch.autograd.Function):
        generate_vmap_rule = True

        @staticmethod
        def forward(*xs):
            with torch.no_grad():
                return fn(*xs)

        @staticmethod
        def setup_context(ctx, inputs, output):
            ctx.save_for_backward(*inputs)

        @staticmethod
        def backward(ctx, *gs):
            xs = ctx.saved_tensors
            with torch.enable_grad():
                _, pull = torch.func.vjp(fn, *xs)
            return pull(gs[0] if len(gs) == 1 else gs)

    return _Segment.apply(*args)


@contextlib.contextmanager
def offload_activations(pin_memory: bool = True):
    """Saved activations live in (pinned) host memory between forward and backward."""
    with torch.autograd.graph.save_on_cpu(pin_memory=pin_memory and torch.cuda.is_available()):
        yield


def apply_gradient_checkpointing(model, enable: bool = True, **kwargs) -> bool:
    """Turns on the model's own checkpointing in the non-reentrant form when PyTorch supports it under transforms;
    returns whether it is active."""
    if not enable:
        return False
    if hasattr(model, "gradient_checkpointing_enable") and native_support():
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False, **kwargs})
        return True
    return False
