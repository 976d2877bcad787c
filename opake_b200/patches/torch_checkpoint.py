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

__all__ = ["checkpoint_under_vmap", "hf_checkpoint_under_transforms", "native_support", "offload_activations",
           "apply_gradient_checkpointing"]


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


def checkpoint_under_vmap(fn: Callable, *args, offload: bool = False):
    """Runs ``fn(*args)`` keeping only its inputs; the backward pass recomputes the segment. Implemented with a
    custom ``autograd.Function`` whose backward calls ``torch.func.vjp`` on ``fn`` (``generate_vmap_rule`` lets the
    whole thing sit under vmap). Everything ``fn`` needs a gradient for must be among ``args``: tensors it merely
    closes over are constants of the segment. ``offload``: the kept inputs wait in host memory between forward and
    backward (the functional counterpart of ``save_on_cpu``, which relies on saved-tensor hooks and is therefore not
    available inside ``torch.func`` transforms)."""
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
            ctx.devices = [x.device for x in inputs]
            ctx.save_for_backward(*[(x.to("cpu") if offload and x.is_cuda else x) for x in inputs])

        @staticmethod
        def backward(ctx, *gs):
            xs = [x.to(d) for x, d in zip(ctx.saved_tensors, ctx.devices)]
            with torch.enable_grad():
                _, pull = torch.func.vjp(fn, *xs)
            return pull(gs[0] if len(gs) == 1 else gs)

    return _Segment.apply(*args)


def hf_checkpoint_under_transforms(fn, *args, offload: bool = False, **_kw):
    """Drop-in for the ``_gradient_checkpointing_func`` of Hugging Face ``GradientCheckpointingLayer`` modules that works
    inside ``vmap(grad(...))``. ``fn`` is the ``partial(layer.__call__, **kwargs)`` the library builds. The layer's
    current parameters (under ``functional_call`` these are the transform-level tensors) and every floating-point
    tensor among the arguments become explicit inputs of a ``checkpoint_under_vmap`` segment, which re-runs the layer
    through ``torch.func.functional_call`` in the backward pass; integer tensors, masks and flags are constants."""
    from torch.func import functional_call

    from ..engine.pytree import tree_flatten, tree_unflatten

    layer = getattr(getattr(fn, "func", None), "__self__", None)
    if layer is None or not isinstance(layer, torch.nn.Module):
        return fn(*args)
    kwargs = dict(getattr(fn, "keywords", None) or {})
    named = list(layer.named_parameters())
    names = [n for n, _ in named]
    leaves, spec = tree_flatten((list(args), kwargs))
    idx = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor) and l.is_floating_point()]

    def segment(*flat):
        ps, rest = flat[: len(names)], flat[len(names):]
        cur = list(leaves)
        for i, t in zip(idx, rest):
            cur[i] = t
        a, kw = tree_unflatten(spec, cur)
        was = getattr(layer, "gradient_checkpointing", False)
        layer.gradient_checkpointing = False          # the recomputation runs the layer itself, not another checkpoint
        try:
            return functional_call(layer, dict(zip(names, ps)), tuple(a), kw)
        finally:
            layer.gradient_checkpointing = was

    return checkpoint_under_vmap(segment, *[p for _, p in named], *[leaves[i] for i in idx], offload=offload)


@contextlib.contextmanager
def offload_activations(pin_memory: bool = True):
    """Saved activations live in (pinned) host memory between forward and backward."""
    with torch.autograd.graph.save_on_cpu(pin_memory=pin_memory and torch.cuda.is_available()):
        yield


def apply_gradient_checkpointing(model, enable: bool = True, offload: bool = False, **kwargs) -> bool:
    """Turns on the model's own layer checkpointing for use under ``vmap(grad)``; returns whether it is active.
    Where PyTorch runs non-reentrant checkpoints inside functorch transforms by itself, the library's function is kept;
    otherwise every checkpointing layer is pointed at ``hf_checkpoint_under_transforms``. ``offload`` keeps the layer
    inputs in host memory between the passes (activation offloading)."""
    if not enable or not hasattr(model, "gradient_checkpointing_enable"):
        return False
    model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False, **kwargs})
    # the library also hooks the embedding output with ``requires_grad_()`` (needed by its reentrant checkpoint for
    # frozen-embedding PEFT runs); in-place autograd flags are illegal inside functorch transforms, and the functional
    # path tracks gradients through the transform itself
    for owner in {model, getattr(model, "base_model", model)}:
        if hasattr(owner, "disable_input_require_grads"):
            try:
                owner.disable_input_require_grads()
            except Exception:
                pass
        hook = getattr(owner, "_require_grads_hook", None)
        if hook is not None:
            hook.remove()
    if native_support() and not offload:
        return True
    import functools

    n = 0
    for m in model.modules():
        if hasattr(m, "_gradient_checkpointing_func") and getattr(m, "gradient_checkpointing", False):
            m._gradient_checkpointing_func = functools.partial(hf_checkpoint_under_transforms, offload=offload)
            n += 1
    return n > 0
