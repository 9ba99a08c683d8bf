"""Activation checkpointing for tensor-parallel blocks: recomputation with every random stream replayed, and the
saved input kept as one ``1 / tp`` slice per rank instead of a full replica.

Inside a tensor-parallel group the input of a transformer block is identical on all ranks, so holding it for the
backward pass on every rank wastes ``(tp - 1) / tp`` of that memory. ``checkpoint(fn, True, x, ...)`` keeps only
this rank's flat chunk of ``x`` and all-gathers the chunks right before the recomputation.

Random streams: ``CudaRNGStatesTracker`` holds named generator states of the compute device (CUDA when present,
else the CPU generator, which keeps the logic testable without a GPU). ``model_parallel_cuda_manual_seed(seed)``
seeds the default stream with ``seed`` (same inside a tensor group) and adds the ``"model-parallel-rng"`` stream with
a seed that depends on the tensor-parallel size; ``with get_cuda_rng_tracker().fork():`` draws from it. The
checkpoint restores the default CPU and device generators, every tracked stream and the randomizers of
``parallel.randomizer`` before it recomputes, and puts the current states back afterwards.
(Reference: atorch/modules/distributed_modules/activation_checkpointing.py:43-361, mappings.py:115-158.)
"""
from __future__ import annotations

import contextlib
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ...distributed import distributed as D

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"
_TENSOR_SLOT = object()          # marks the positions of tensor arguments (``None`` is a legal argument)


def _on_cuda() -> bool:
    return torch.cuda.is_available()


def _device_rng_state() -> torch.Tensor:
    return torch.cuda.get_rng_state() if _on_cuda() else torch.get_rng_state()


def _set_device_rng_state(state: torch.Tensor) -> None:
    if _on_cuda():
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


def _device_manual_seed(seed: int) -> None:
    if _on_cuda():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


class CudaRNGStatesTracker:
    """Named generator states; ``fork(name)`` runs a block on one of them and stores where it ended."""

    def __init__(self):
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def reset(self) -> None:
        self.states_, self.seeds_ = {}, set()

    def get_states(self) -> Dict[str, torch.Tensor]:
        return dict(self.states_)

    def set_states(self, states: Dict[str, torch.Tensor]) -> None:
        self.states_ = states

    def add(self, name: str, seed: int) -> None:
        if seed in self.seeds_:
            raise Exception("seed {} already exists".format(seed))
        if name in self.states_:
            raise Exception("cuda rng state {} already exists".format(name))
        self.seeds_.add(seed)
        here = _device_rng_state()
        _device_manual_seed(seed)
        self.states_[name] = _device_rng_state()
        _set_device_rng_state(here)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise Exception("cuda rng state {} is not added".format(name))
        here = _device_rng_state()
        _set_device_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = _device_rng_state()
            _set_device_rng_state(here)


_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker() -> CudaRNGStatesTracker:
    return _TRACKER


def model_parallel_cuda_manual_seed(seed: int, group: str = "tensor") -> None:
    """Replaces ``torch.cuda.manual_seed`` once the parallel groups exist: default stream ``seed``, model-parallel
    stream ``seed + 2718 + size(group)``."""
    _TRACKER.reset()
    _device_manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, seed + 2718 + (D.parallel_group_size(group) or 1))


# ---------------------------------------------------------------------------------- the 1 / tp slice of a replica
def split_tensor_into_1d_equal_chunks(tensor: torch.Tensor, group: str = "tensor", new_buffer: bool = False):
    """This rank's ``numel / size`` elements of the flattened tensor (a view, or a copy with ``new_buffer``)."""
    size, rank = D.parallel_group_size(group) or 1, D.parallel_rank(group) or 0
    assert tensor.numel() % size == 0, (tensor.numel(), size)
    n = tensor.numel() // size
    chunk = tensor.reshape(-1)[rank * n: (rank + 1) * n]
    return chunk.clone() if new_buffer else chunk


def gather_split_1d_tensor(tensor: torch.Tensor, group: str = "tensor") -> torch.Tensor:
    """The flat concatenation of all ranks' chunks."""
    size = D.parallel_group_size(group) or 1
    if size == 1:
        return tensor.reshape(-1).clone()
    out = torch.empty(tensor.numel() * size, dtype=tensor.dtype, device=tensor.device)
    dist.all_gather_into_tensor(out, tensor.contiguous().reshape(-1), group=D.parallel_group(group))
    return out


def _all_rng_states():
    from ...parallel import randomizer as R

    streams = list(R._RANDOMIZERS.values())
    return (torch.get_rng_state(), torch.cuda.get_rng_state() if _on_cuda() else None, _TRACKER.get_states(),
            [(r, r.cpu_state, r.cuda_state) for r in streams])


def _restore_rng_states(saved) -> None:
    cpu, cuda, tracked, streams = saved
    torch.set_rng_state(cpu)
    if cuda is not None:
        torch.cuda.set_rng_state(cuda)
    _TRACKER.set_states(tracked)
    for r, c, g in streams:
        r.cpu_state, r.cuda_state = c, g


class CheckpointFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, distribute_saved_activations, *args):
        ctx.run_function = run_function
        ctx.rng = _all_rng_states()
        ctx.autocast = (torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")) if _on_cuda() \
            else (False, None)
        with torch.no_grad():
            outputs = run_function(*args)
        tp = (D.parallel_group_size("tensor") or 1) if distribute_saved_activations else 1
        ctx.first_shape = None
        tensors: List[torch.Tensor] = []
        ctx.proto = []
        for i, a in enumerate(args):
            if not torch.is_tensor(a):
                ctx.proto.append(a)
                continue
            ctx.proto.append(_TENSOR_SLOT)
            if i == 0 and tp > 1 and a.dim() > 1 and a.shape[0] % tp == 0:
                ctx.first_shape = a.shape
                ctx.first_requires_grad = a.requires_grad
                a = split_tensor_into_1d_equal_chunks(a.detach(), new_buffer=True)
            tensors.append(a)
        ctx.save_for_backward(*tensors)
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        if not torch.autograd._is_checkpoint_valid():
            raise RuntimeError("Checkpointing is not compatible with .grad(), please use .backward() if possible")
        it = iter(ctx.saved_tensors)
        inputs = [next(it) if p is _TENSOR_SLOT else p for p in ctx.proto]
        if ctx.first_shape is not None:
            inputs[0] = gather_split_1d_tensor(inputs[0]).view(ctx.first_shape).requires_grad_(ctx.first_requires_grad)
        detached = [a.detach().requires_grad_(a.requires_grad) if torch.is_tensor(a) else a for a in inputs]
        now = _all_rng_states()
        _restore_rng_states(ctx.rng)
        try:
            with torch.enable_grad(), (torch.autocast("cuda", dtype=ctx.autocast[1]) if ctx.autocast[0]
                                       else contextlib.nullcontext()):
                outputs = ctx.run_function(*detached)
        finally:
            _restore_rng_states(now)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        pairs: List[Tuple[torch.Tensor, torch.Tensor]] = [
            (o, g) for o, g in zip(outputs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if not pairs:
            raise RuntimeError("none of output has requires_grad=True, this checkpoint() is not necessary")
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if torch.is_tensor(a) else None for a in detached)


def checkpoint(function: Callable, distribute_saved_activations: bool, *args):
    """``function(*args)`` now, recomputed in the backward pass. Positional arguments only; with
    ``distribute_saved_activations`` the first argument (replicated over the tensor group, first dimension divisible by
    its size) is kept as this rank's slice."""
    return CheckpointFunction.apply(function, distribute_saved_activations, *args)


class TPCheckpointWrapper(nn.Module):
    """Module wrapper: keyword arguments are flattened into positional ones for ``checkpoint_fn`` and restored for the
    wrapped module, which stays reachable as ``_checkpoint_wrapped_module`` (same attribute as torch's wrapper, so
    state-dict prefixes can be handled alike)."""

    def __init__(self, mod: nn.Module, checkpoint_fn: Callable = checkpoint):
        super().__init__()
        self._checkpoint_wrapped_module = mod
        self.checkpoint_fn = checkpoint_fn

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._checkpoint_wrapped_module, name)

    def forward(self, *args, **kwargs):
        keys = list(kwargs)
        flat = tuple(args) + tuple(kwargs[k] for k in keys)
        n_pos = len(args)

        def run(*inputs):
            return self._checkpoint_wrapped_module(*inputs[:n_pos], **dict(zip(keys, inputs[n_pos:])))

        return self.checkpoint_fn(run, True, *flat)


def tp_wrap_fn(module: nn.Module, amp_config: Optional[dict] = None) -> TPCheckpointWrapper:
    """The wrap function the checkpoint optimisation uses for tensor-parallel blocks; ``amp_config`` (arguments of
    ``torch.autocast``) makes the block run, and rerun, under that autocast."""
    if amp_config is not None:
        cfg = dict(amp_config)
        cfg.setdefault("device_type", "cuda" if _on_cuda() else "cpu")
        inner = module.forward

        def forward(*a, **k):
            with torch.autocast(**cfg):
                return inner(*a, **k)

        module.forward = forward
    return TPCheckpointWrapper(module, checkpoint)
