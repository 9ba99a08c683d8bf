"""Activation checkpointing for whole modules.

``checkpoint_module(module, *args)`` runs the module without recording a graph, keeps only its
inputs, and recomputes the forward inside the backward. It is the per-layer recomputation of the
``checkpoint`` optimisation (reference: atorch/auto/opt_lib/checkpoint_optimization.py:15-271, which
wraps modules with torch's ``checkpoint_wrapper``). RNG state is saved and restored so that dropout
replays identically.
"""
from __future__ import annotations

import contextlib
import itertools
import threading
from typing import Any, Callable, Optional, Tuple

import torch
from torch.utils._pytree import tree_flatten, tree_unflatten

# ---------------------------------------------------------------------------------------------
# Pass tokens. The no-grad first pass of a checkpointed block and the recomputation of the SAME
# block in the backward pass run under one shared token, so an operator inside the block can keep a
# result of the first pass for the recomputation (ops/flash.py keeps attention output + lse) and be
# certain that the two belong together. A forward that is not the first pass of a checkpointed block
# (validation without .eval(), reference log-probs, a dry run) has no token and caches nothing.
# ---------------------------------------------------------------------------------------------
_tokens = itertools.count(1)
_tls = threading.local()


def new_pass_token() -> int:
    return next(_tokens)


@contextlib.contextmanager
def checkpoint_pass(token: int, recompute: bool):
    prev = getattr(_tls, "cur", None)
    _tls.cur = (token, recompute)
    try:
        yield
    finally:
        _tls.cur = prev


def current_pass() -> Optional[Tuple[int, bool]]:
    """``(token, is_recompute)`` while a checkpointed block runs its first pass or its recomputation."""
    return getattr(_tls, "cur", None)


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run: Callable, spec, preserve_rng: bool, n_tensors: int, *flat):
        ctx.run, ctx.spec, ctx.preserve_rng = run, spec, preserve_rng
        tensors = flat[:n_tensors]
        ctx.others = flat[n_tensors:]
        ctx.tensor_idx = [i for i, t in enumerate(tensors) if isinstance(t, torch.Tensor)]
        ctx.save_for_backward(*[tensors[i] for i in ctx.tensor_idx])
        ctx.flat_proto = list(tensors)
        if preserve_rng:
            ctx.cpu_rng = torch.get_rng_state()
            ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        ctx.token = new_pass_token()
        # the recomputation must run under the same autocast state as this pass
        dev_type = next((t.device.type for t in tensors if isinstance(t, torch.Tensor)), "cpu")
        ctx.autocast = (dev_type, torch.is_autocast_enabled(dev_type), torch.get_autocast_dtype(dev_type))
        with torch.no_grad(), checkpoint_pass(ctx.token, False):
            args, kwargs = tree_unflatten(list(tensors), spec)
            out = run(*args, **kwargs)
        return out

    @staticmethod
    def backward(ctx, *grad_out):
        saved = ctx.saved_tensors
        flat = list(ctx.flat_proto)
        detached = []
        for i, t in zip(ctx.tensor_idx, saved):
            d = t.detach()
            d.requires_grad_(t.requires_grad)
            flat[i] = d
            detached.append(d)
        if ctx.preserve_rng:
            cpu_now = torch.get_rng_state()
            torch.set_rng_state(ctx.cpu_rng)
            if ctx.cuda_rng is not None:
                cuda_now = torch.cuda.get_rng_state()
                torch.cuda.set_rng_state(ctx.cuda_rng)
        dev_type, ac_on, ac_dtype = ctx.autocast
        with torch.enable_grad(), torch.autocast(dev_type, dtype=ac_dtype, enabled=ac_on), \
                checkpoint_pass(ctx.token, True):
            args, kwargs = tree_unflatten(flat, ctx.spec)
            out = ctx.run(*args, **kwargs)
        if ctx.preserve_rng:
            torch.set_rng_state(cpu_now)
            if ctx.cuda_rng is not None:
                torch.cuda.set_rng_state(cuda_now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grad_out) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        grads = [None] * len(ctx.flat_proto)
        for i, d in zip(ctx.tensor_idx, detached):
            grads[i] = d.grad
        return (None, None, None, None, *grads, *([None] * len(ctx.others)))


def checkpoint_function(run: Callable, *args: Any, preserve_rng_state: bool = False, **kwargs: Any):
    """Checkpointed call of ``run(*args, **kwargs)``; tensors anywhere in the arguments are tracked."""
    flat, spec = tree_flatten((args, kwargs))
    extra = []
    if not any(isinstance(t, torch.Tensor) and t.requires_grad for t in flat):
        # parameters inside `run` may still need gradients: an extra scalar that requires grad makes
        # the node differentiable (it rides after the real arguments and is ignored by `run`)
        dev = next((t.device for t in flat if isinstance(t, torch.Tensor)), None)
        extra = [torch.zeros((), device=dev, requires_grad=True)]
    return _Checkpoint.apply(run, spec, preserve_rng_state, len(flat), *flat, *extra)


def checkpoint_module(module: torch.nn.Module, *args: Any, preserve_rng_state: bool = False, **kwargs: Any):
    return checkpoint_function(module.__call__ if not hasattr(module, "_atb_orig_call") else module._atb_orig_call,
                               *args, preserve_rng_state=preserve_rng_state, **kwargs)
