"""Trainer-side helpers that do not depend on the training engine: process roles, dict <-> byte-tensor transport (to
broadcast small Python objects with tensor collectives), distributed standard deviations of parameters, nested metric
dicts to tensorboard / wandb, the argument banner, and the interval enum of the training arguments.
(Reference: atorch/trainer/utils.py:54-94, 134-148, 267-277, 821-838; the Megatron-specific gradient and logging
helpers of that file have their counterparts in ``trainer/engine.py`` and ``trainer/atorch_trainer_v2.py``.)
"""
from __future__ import annotations

import logging
import pickle
from enum import Enum
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..distributed import distributed as D

logger = logging.getLogger("atorch.logger")


class DistributedType(str, Enum):
    NO_DISTRIBUTE = "NO_DISTRIBUTE"
    DEEPSPEED = "DEEPSPEED"
    FSDP = "FSDP"
    MEGATRON = "MEGATRON"
    MINDSPEED = "MINDSPEED"
    MULTI_CPU = "MULTI_CPU"
    MULTI_GPU = "MULTI_GPU"
    MULTI_NPU = "MULTI_NPU"
    MULTI_MLU = "MULTI_MLU"
    MULTI_MUSA = "MULTI_MUSA"
    MULTI_XPU = "MULTI_XPU"


class IntervalStrategy(str, Enum):
    NO = "no"
    STEPS = "steps"
    EPOCH = "epoch"
    SAMPLES = "samples"


def is_main_process() -> bool:
    r = D.rank()
    return r is None or r == 0


def is_local_main_process() -> bool:
    return (D.local_rank() or 0) == 0


def is_last_rank_on_current_stage() -> bool:
    """Last data-parallel (and sequence-parallel) rank and last tensor-parallel rank of this pipeline stage: the rank
    that logs per-stage quantities."""
    for name in ("data", "sequence", "tensor"):
        size = D.parallel_group_size(name)
        if size and (D.parallel_rank(name) or 0) != size - 1:
            return False
    return True


def dict_to_tensor(input_dict, device=None) -> torch.Tensor:
    """A picklable object as a uint8 tensor (on the current CUDA device when there is one)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
    return torch.frombuffer(bytearray(pickle.dumps(input_dict)), dtype=torch.uint8).to(device)


def tensor_to_dict(tensor: torch.Tensor):
    return pickle.loads(bytes(tensor.cpu().tolist()))


def distributed_std(name: str, param: torch.Tensor, data_group=None, tensor_group=None) -> torch.Tensor:
    """Unbiased standard deviation of a parameter whose pieces are spread over the data group (sharded engine) and,
    when it is marked ``tensor_model_parallel``, over the tensor group as well. Groups default to the named parallel
    groups."""
    data_group = data_group if data_group is not None else D.parallel_group("data")
    tensor_group = tensor_group if tensor_group is not None else D.parallel_group("tensor")
    count = torch.tensor(param.numel(), dtype=torch.int64, device=param.device)
    total = param.detach().float().sum()
    groups = [data_group]
    if getattr(param, "tensor_model_parallel", False) and tensor_group is not None:
        groups.insert(0, tensor_group)
    live = [g for g in groups if g is not None and dist.get_world_size(g) > 1]
    for g in live:
        dist.all_reduce(count, group=g)
        dist.all_reduce(total, group=g)
    mean = total / count
    sq = torch.sum(torch.square(param.detach().float() - mean))
    for g in live:
        dist.all_reduce(sq, group=g)
    return (sq / (count - 1)) ** 0.5


def calc_params_std(model: torch.nn.Module, gather_to_last_rank: bool = False) -> Dict[str, float]:
    """``{parameter name: std}`` over whole (unsharded) parameters; parameters of a sharded engine are given by the
    piece this rank holds, reduced over the data group."""
    return {n: float(distributed_std(n, p)) for n, p in model.named_parameters() if p.numel() > 1}


def write_dict_to_tensorboard(writer, wandb_writer, index: int, metrics: dict, prefix: str = "") -> None:
    """Nested dicts become ``a/b/c`` scalar names."""
    for key, value in metrics.items():
        name = prefix + key
        if isinstance(value, dict):
            write_dict_to_tensorboard(writer, wandb_writer, index, value, prefix=name + "/")
        else:
            writer.add_scalar(name, value, index)
            if wandb_writer is not None:
                wandb_writer.log({name: value}, index)


def print_all_args_before_training(all_args: Dict[str, Dict], log: Optional[logging.Logger] = None) -> None:
    log = log or logger
    log.info("\n=============== Print all args before training ===============")
    for title, args in all_args.items():
        log.info("************************ %s ************************", title)
        for line in sorted(("  {} {} {}".format(k, "*" * (48 - len(k)), v) for k, v in args.items()), key=str.lower):
            log.info(line)
        log.info("******************** end of %s *********************\n", title)
