"""``ModelContext``: everything a training job is made of (model, optimizer factory, dataset, loss,
input preparation) plus the registry of *wrappers* that optimisation methods add to it.

Optimisation methods only *register* wrappers (``add_wrapper``); ``adjust_wrappers`` resolves the
interactions between them and ``apply_wrappers`` executes them in a fixed order, first the
pre-wrappers (before the optimizer exists), then, after ``update_optim``, the post-wrappers:

    pre : half -> module_replace -> sequence_parallel -> tp -> fp8 -> checkpoint -> fsdp -> dynamo
    post: amp_native -> zero1 -> ddp

Interactions resolved here:
* ``amp_native`` together with ``fsdp``/``zero2`` becomes the mixed-precision setting of the
  sharded engine (bf16 compute copy, fp32 master shards) instead of a separate autocast wrapper;
* ``checkpoint`` on the same classes as the sharding units becomes per-unit recomputation inside
  the engine (parameters are gathered once per recompute+backward);
* sharded engines take over data parallelism, so the ``ddp`` wrapper is dropped next to them;
  when both a ``zero`` and a ``data`` group exist the engine runs hybrid shard;
* ``half=bf16`` without a sharded engine wraps the optimizer in ``BF16Optimizer``.

Dataloader creation follows strong scaling: ``batch_size`` in ``dataloader_args`` is the global
batch and is divided by the data-parallel size (atorch/auto/model_context.py:309-321 of the
reference; the whole class mirrors the behaviour of :101-868 there).
"""
from __future__ import annotations

import collections
import logging
import types
from typing import Any, Callable, Dict, Optional

import torch
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from ..distributed import distributed as D

logger = logging.getLogger("atorch.logger")

PRE_ORDER = ["half", "module_replace", "sequence_parallel", "tp", "fp8", "checkpoint", "fsdp", "fsdp2",
             "native_dynamo"]
POST_ORDER = ["amp_native", "zero1", "zero2", "ddp", "pipe"]


def get_mc_default_args() -> dict:
    return {"use_optim_backward": False, "requires_set_gradient_accumulation_boundary": False}


class ModelContext:
    def __init__(self, model=None, optim_func=None, dataset=None, loss_func=None, prepare_input=None,
                 model_input_format=None, optim_args=None, optim_param_func=None, dataloader_args=None,
                 distributed_sampler_cls=None, lr_scheduler_cls=None, lr_scheduler_args=None, extra_args=None):
        if model_input_format not in (None, "unpack_sequence", "unpack_dict"):
            raise ValueError(f"model_input_format {model_input_format!r} not in None|unpack_sequence|unpack_dict")
        self.model = model
        self.optim_func = optim_func
        self.optim = None
        self.dataset = dataset
        self.loss_func = loss_func
        self.prepare_input = prepare_input
        self.model_input_format = model_input_format
        self.optim_args = dict(optim_args) if optim_args is not None else {}
        self.optim_param_func = optim_param_func
        self.dataloader_args = dict(dataloader_args) if dataloader_args is not None else None
        self.dataloader = None
        self.pre_wrappers: "collections.OrderedDict[str, tuple]" = collections.OrderedDict()
        self.post_wrappers: "collections.OrderedDict[str, tuple]" = collections.OrderedDict()
        self.parallel_mode_config = None
        self.pre_wrapper_applied = False
        self.post_wrapper_applied = False
        self.distributed_sampler_cls = distributed_sampler_cls or DistributedSampler
        self.lr_scheduler_cls = lr_scheduler_cls
        self.lr_scheduler_args = lr_scheduler_args
        self.lr_scheduler = None
        self.extra_args = dict(extra_args) if extra_args is not None else {}
        self.sample_batch = self.extra_args.get("sample_batch")
        self.sample_batch_size = self.extra_args.get("batch_size")
        self.expand_sample_batch = self.extra_args.get("expand_sample_batch", True)
        self.sampler_seed = self.extra_args.get("sampler_seed", 0)
        self.tp_status = False
        self.args = get_mc_default_args()

    # ------------------------------------------------------------------------------ wrappers
    def add_wrapper(self, wrapper_name: str, wrapper_func: Callable, wrapper_config: Any = None,
                    is_pre_wrapper: bool = True, ignore_duplicated: bool = True) -> None:
        reg = self.pre_wrappers if is_pre_wrapper else self.post_wrappers
        if wrapper_name in reg:
            if ignore_duplicated:
                return
            raise ValueError(f"wrapper {wrapper_name} registered twice")
        reg[wrapper_name] = (wrapper_func, wrapper_config)

    def update_tp_status(self, status: bool) -> None:
        self.tp_status = status

    def adjust_wrappers(self) -> None:
        pre, post = self.pre_wrappers, self.post_wrappers
        sharded = "fsdp" in pre or "fsdp2" in pre
        shard_name = "fsdp" if "fsdp" in pre else ("fsdp2" if "fsdp2" in pre else None)
        if sharded:
            fn, cfg = pre[shard_name]
            cfg = dict(cfg or {})
            if "amp_native" in post:
                _, amp_cfg = post.pop("amp_native")
                dtype = (amp_cfg or {}).get("dtype", torch.float16)
                cfg.setdefault("param_dtype", dtype)
                if dtype == torch.float16:
                    post["amp_native"] = (self._amp_scaler_only_wrapper, amp_cfg)
            if "half" in pre:
                _, half_cfg = pre["half"]
                cfg.setdefault("param_dtype", half_cfg)
            if "checkpoint" in pre:
                _, ck = pre["checkpoint"]
                ck_classes = set(_class_names((ck or {}).get("wrap_class", ())))
                unit_classes = set(_class_names(cfg.get("atorch_wrap_cls", ())))
                if ck_classes and ck_classes <= unit_classes and not (ck or {}).get("selective_offload"):
                    cfg["checkpoint_units"] = True
                    pre.pop("checkpoint")
            if "ddp" in post:
                post.pop("ddp")
            if D.parallel_group("zero") is not None and D.parallel_group("data") is not None:
                cfg.setdefault("process_group", D.parallel_group("zero"))
                cfg.setdefault("replica_group", D.parallel_group("data"))
            pre[shard_name] = (fn, cfg)
        if "zero2" in post and "ddp" in post:
            post.pop("ddp")
        self.pre_wrappers = collections.OrderedDict(
            sorted(pre.items(), key=lambda kv: PRE_ORDER.index(kv[0]) if kv[0] in PRE_ORDER else len(PRE_ORDER)))
        self.post_wrappers = collections.OrderedDict(
            sorted(post.items(), key=lambda kv: POST_ORDER.index(kv[0]) if kv[0] in POST_ORDER else len(POST_ORDER)))

    @staticmethod
    def _amp_scaler_only_wrapper(model_context, wrapper_name, wrapper_config):
        from .opt_lib.amp import apply_grad_scaler

        return apply_grad_scaler(model_context, wrapper_config, sharded=True)

    def apply_wrappers(self, is_pre_wrapper: bool = True) -> None:
        reg = self.pre_wrappers if is_pre_wrapper else self.post_wrappers
        for name, (fn, cfg) in list(reg.items()):
            fn(self, name, cfg)
        if is_pre_wrapper:
            self.pre_wrapper_applied = True
        else:
            self.post_wrapper_applied = True

    # ------------------------------------------------------------------------------ dataloader
    def create_dataloader(self, extra_args: Optional[dict] = None):
        if self.dataset is None:
            return None
        args = dict(self.dataloader_args or {})
        if extra_args:
            args.update(extra_args)
        args.setdefault("num_workers", 0)
        rank, ddp_size = D.get_data_partition_rank_and_size()
        sampler = None
        if ddp_size > 1:
            shuffle = bool(args.pop("shuffle", True))
            sampler = self.distributed_sampler_cls(self.dataset, shuffle=shuffle, num_replicas=ddp_size, rank=rank,
                                                   seed=self.sampler_seed)
            if "batch_size" in args:  # strong scaling: the given batch size is the global one
                ori = args["batch_size"]
                args["batch_size"] = max(ori // ddp_size, 1)
                if args["batch_size"] * ddp_size != ori:
                    logger.warning("batch_size=%d is not a multiple of data parallel size %d, adjusted to %d",
                                   ori, ddp_size, args["batch_size"] * ddp_size)
        from ..data.shm_dataloader import maybe_shm_dataloader

        loader = maybe_shm_dataloader(self.dataset, sampler, args)
        if loader is None:
            loader = DataLoader(self.dataset, sampler=sampler, **args)

        def set_epoch(self_, epoch):
            if hasattr(self_.sampler, "set_epoch"):
                self_.sampler.set_epoch(epoch)

        loader.set_epoch = types.MethodType(set_epoch, loader)
        return loader

    def update_dataloader(self, extra_args: Optional[dict] = None) -> None:
        self.dataloader = self.create_dataloader(extra_args)

    # ------------------------------------------------------------------------------- optimizer
    def create_optim(self):
        if self.optim_func is None:
            return None
        from ..parallel.fsdp import FSDP, FusedShardedOptimizer, ShardedOptimizer
        from ..optimizers import AGD, BF16Optimizer

        model = self.model
        if isinstance(model, FSDP):
            eng = model.engine
            fused_kind = None
            if self.optim_param_func is None and not self.extra_args.get("disable_fused_optimizer", False):
                if self.optim_func in (torch.optim.AdamW,):
                    fused_kind = "adamw"
                elif self.optim_func in (torch.optim.Adam,):
                    fused_kind = "adam"
                elif self.optim_func is AGD:
                    fused_kind = "agd"
            a = self.optim_args
            if fused_kind is not None and not a.get("amsgrad", False) and not a.get("win", False):
                kw = dict(lr=a.get("lr", 1e-3), betas=a.get("betas", (0.9, 0.999)),
                          weight_decay=a.get("weight_decay", 0.01 if fused_kind == "adamw" else 0.0))
                if fused_kind == "agd":
                    kw.update(delta=a.get("delta", 1e-5), clip=a.get("clip"),
                              weight_decouple=a.get("weight_decouple", True), fixed_decay=a.get("fixed_decay", False))
                else:
                    kw.update(eps=a.get("eps", 1e-8))
                return FusedShardedOptimizer(eng, fused_kind, **kw)
            params = self.optim_param_func(model, **self.extra_args.get("optim_param_func_args", {})) \
                if self.optim_param_func is not None else model.parameters()
            return ShardedOptimizer(self.optim_func(params, **self.optim_args), eng)
        params = self.optim_param_func(model) if self.optim_param_func is not None else model.parameters()
        optim = self.optim_func(params, **self.optim_args)
        half = self.pre_wrappers.get("half")
        if half is not None and half[1] in ("bf16", torch.bfloat16) and "zero1" not in self.post_wrappers \
                and "zero2" not in self.post_wrappers:
            optim = BF16Optimizer(optim)
        return optim

    def update_optim(self) -> None:
        self.optim = self.create_optim()
        if self.optim is not None and self.lr_scheduler_cls is not None:
            target = getattr(self.optim, "optimizer", self.optim)
            sched_target = target if isinstance(target, torch.optim.Optimizer) else _SchedulerShim(self.optim)
            self.lr_scheduler = self.lr_scheduler_cls(sched_target, **(self.lr_scheduler_args or {}))

    # ----------------------------------------------------------------------------------- misc
    def gpu_used(self) -> bool:
        return torch.cuda.is_available()

    def find_unused_parameters(self) -> bool:
        return bool(self.extra_args.get("find_unused_parameters", False))

    def get_one_input_batch(self):
        if self.sample_batch is not None:
            return self.sample_batch
        if self.dataloader is None:
            self.update_dataloader()
        if self.dataloader is None:
            return None
        return next(iter(self.dataloader))

    @staticmethod
    def get_loss_from_loss_func_output(output):
        if isinstance(output, (tuple, list)):
            return output[0]
        return output

    def run_one_step(self, batch=None, backward: bool = True):
        """Forward (+ backward + optimizer step) on one batch: used by the dry run."""
        batch = batch if batch is not None else self.get_one_input_batch()
        device = next(iter(self.model.parameters())).device if any(True for _ in self.model.parameters()) else "cpu"
        if self.prepare_input is not None:
            batch = self.prepare_input(batch, device)
        if self.model_input_format == "unpack_dict":
            out = self.model(**batch)
        elif self.model_input_format == "unpack_sequence":
            out = self.model(*batch)
        else:
            out = self.model(batch)
        loss = self.get_loss_from_loss_func_output(self.loss_func(batch, out)) if self.loss_func else out
        if backward:
            if self.optim is not None:
                self.optim.zero_grad()
            loss.backward()
            if self.optim is not None:
                self.optim.step()
        return loss


class _SchedulerShim(torch.optim.Optimizer):
    """Lets torch LR schedulers drive an optimizer-like object that only has ``param_groups``."""

    def __init__(self, optim_like):
        self._inner = optim_like
        self.param_groups = optim_like.param_groups
        self.defaults = dict(getattr(optim_like, "defaults", {}))
        self.state = collections.defaultdict(dict)
        self._optimizer_step_pre_hooks = collections.OrderedDict()
        self._optimizer_step_post_hooks = collections.OrderedDict()

    def step(self, closure=None):
        return self._inner.step(closure)


def _class_names(classes) -> list:
    if classes is None:
        return []
    if not isinstance(classes, (tuple, list, set)):
        classes = (classes,)
    return [c if isinstance(c, str) else c.__name__ for c in classes]
