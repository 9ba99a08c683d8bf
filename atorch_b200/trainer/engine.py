"""Train engines of ``AtorchTrainerV2``.

``AtorchTrainEngine`` is the contract (``train_step / eval_step / optimizer_step / save_checkpoint /
load_checkpoint / training_log``); ``NativeTrainEngine`` implements it on this framework's own
runtimes: sharded data parallel or DDP, optional tensor parallel (automatic plan), micro-batch
accumulation up to the global batch, gradient clipping, LR schedule, spike-loss gradient scaling,
sharded async checkpoints. (The reference implements the contract only for Megatron:
atorch/trainer/base/atorch_train_engine.py:14, atorch/trainer/megatron/megatron_wrapper.py:399-1205.)
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterator, Optional

import torch
import torch.distributed as dist

from ..auto.accelerate import auto_accelerate
from ..auto.clip_grad_norm import clip_grad_norm
from ..common.util_func import data_to_device
from ..distributed import distributed as D
from .args import AtorchTrainingArgs
from .atorch_trainer import get_scheduler
from .fsdp import ExtraState, FsdpShardCkptAsyncSaver, FsdpShardDcpCkptLoader


class AtorchTrainEngine(torch.nn.Module):
    def train_step(self, data_iterator) -> Dict: raise NotImplementedError
    def eval_step(self, data_iterator) -> Dict: raise NotImplementedError
    def optimizer_step(self): raise NotImplementedError
    def save_checkpoint(self, iteration: int, output_dir: str, **kw): raise NotImplementedError
    def load_checkpoint(self, path: str, **kw): raise NotImplementedError
    def training_log(self, **kw): pass
    def forward(self, data_iterator):
        return self.train_step(data_iterator) if self.training else self.eval_step(data_iterator)


class NativeTrainEngine(AtorchTrainEngine):
    def __init__(self, args: AtorchTrainingArgs, model: torch.nn.Module, loss_func: Optional[Callable] = None,
                 wrap_cls=None, optim_func=None, total_steps: Optional[int] = None):
        super().__init__()
        self.args = args
        world = D.world_size() or 1
        self.world = world
        dims = []
        if args.tensor_model_parallel_size > 1:
            dims.append(("tensor", args.tensor_model_parallel_size))
        if args.pipeline_model_parallel_size > 1:
            dims.append(("pipe", args.pipeline_model_parallel_size))
        dims.append(("data", args.data_parallel_size(world)))
        strategy = [("parallel_mode", (dims, None))]
        if args.tensor_model_parallel_size > 1:
            strategy.append(("tensor_parallel", {"sequence_parallel": args.sequence_parallel}))
        if args.distributed_type in ("fsdp", "hybrid", "megatron") and args.use_distributed_optimizer:
            strategy.append(("fsdp", {"atorch_wrap_cls": tuple(wrap_cls)} if wrap_cls else {}))
        if args.bf16 or args.fp16:
            strategy.append(("amp_native", {"dtype": torch.bfloat16 if args.bf16 else torch.float16}))
        if args.recompute_granularity == "full" and wrap_cls:
            strategy.append(("checkpoint", {"wrap_class": tuple(wrap_cls)}))
        from ..optimizers import AGD

        optim_func = optim_func or {"adamw": torch.optim.AdamW, "agd": AGD, "sgd": torch.optim.SGD}[args.optimizer]
        oa = {"lr": args.learning_rate, "weight_decay": args.weight_decay}
        if args.optimizer in ("adamw", "agd"):
            oa["betas"] = (args.adam_beta1, args.adam_beta2)
        ok, res, self.strategy = auto_accelerate(model, optim_func, loss_func=loss_func or self._default_loss,
                                                 prepare_input=data_to_device, model_input_format="unpack_dict",
                                                 optim_args=oa, load_strategy=strategy)
        if not ok:
            raise RuntimeError("could not apply the strategy derived from the training arguments")
        self.module, self.optimizer, self.loss_func, self.prepare_input = res.model, res.optim, res.loss_func, res.prepare_input
        steps = total_steps or args.train_iters or (args.max_steps if args.max_steps > 0 else 1000)
        warm = args.lr_warmup_iters or int((args.lr_warmup_fraction or 0.0) * steps)
        self.lr_scheduler = get_scheduler("cosine" if args.lr_decay_style == "cosine" else
                                          ("constant" if args.lr_decay_style == "constant" else "linear"),
                                          self.optimizer, warm, steps)
        self.num_micro = args.num_micro_batches(world)
        self.device = torch.device("cuda", torch.cuda.current_device()) if (torch.cuda.is_available() and "nccl" in
                                                                            (D.backend() or "nccl")) else torch.device("cpu")
        self.loss_ema = None
        self.saver, self.loader = FsdpShardCkptAsyncSaver(), FsdpShardDcpCkptLoader()
        self.last_grad_norm = None

    @staticmethod
    def _default_loss(batch, out):
        if isinstance(out, dict):
            return out["loss"]
        return out.loss if hasattr(out, "loss") else (out[0] if isinstance(out, (tuple, list)) else out)

    def _forward_loss(self, batch):
        batch = self.prepare_input(batch, self.device)
        out = self.module(**batch) if isinstance(batch, dict) else self.module(batch)
        return self.loss_func(batch, out)

    def train_step(self, data_iterator: Iterator) -> Dict:
        self.module.train()
        self.optimizer.zero_grad()
        total = torch.zeros((), device=self.device)
        for _ in range(self.num_micro):
            loss = self._forward_loss(next(data_iterator))
            (loss / self.num_micro).backward()
            total += loss.detach().float() / self.num_micro
        if self.world > 1:
            dist.all_reduce(total)
            total /= self.world
        ratio = self._spike_ratio(float(total))
        skipped = self.optimizer_step(ratio)
        return {"loss": float(total), "grad_norm": self.last_grad_norm, "skipped": skipped, "spike_ratio": ratio,
                "lr": self.optimizer.param_groups[0]["lr"]}

    def _spike_ratio(self, loss: float) -> float:
        a = self.args
        ratio = 1.0
        if a.spike_loss_ratio is not None and self.loss_ema is not None and loss > a.spike_loss_threshold * self.loss_ema:
            ratio = a.spike_loss_ratio
        self.loss_ema = loss if self.loss_ema is None else 0.9 * self.loss_ema + 0.1 * loss
        return ratio

    def optimizer_step(self, grad_ratio: float = 1.0) -> bool:
        if grad_ratio == 0.0:
            return True
        if grad_ratio != 1.0:
            if hasattr(self.module, "engine"):
                self.module.engine.finalize_grads().mul_(grad_ratio)
            else:
                for p in self.module.parameters():
                    if p.grad is not None:
                        p.grad.mul_(grad_ratio)
        if self.args.clip_grad and self.args.clip_grad > 0:
            self.last_grad_norm = float(clip_grad_norm(self.module, self.args.clip_grad, optimizer=self.optimizer))
        self.optimizer.step()
        self.lr_scheduler.step()
        return False

    @torch.no_grad()
    def eval_step(self, data_iterator: Iterator) -> Dict:
        self.module.eval()
        loss = self._forward_loss(next(data_iterator)).detach().float()
        if self.world > 1:
            dist.all_reduce(loss)
            loss /= self.world
        return {"loss": float(loss)}

    def save_checkpoint(self, iteration: int, output_dir: str, **kw):
        if hasattr(self.module, "engine"):
            self.saver.save(iteration, output_dir, module=self.module, optimizer=self.optimizer,
                            extra_state=ExtraState(iteration=iteration, lr_scheduler=self.lr_scheduler.state_dict(),
                                                   others=kw))
            if not self.args.async_save:
                self.saver.finish()
        elif (D.rank() or 0) == 0:
            import os

            os.makedirs(output_dir, exist_ok=True)
            torch.save({"model": self.module.state_dict(), "optim": self.optimizer.state_dict(),
                        "lr_scheduler": self.lr_scheduler.state_dict(), "iteration": iteration},
                       os.path.join(output_dir, f"iter_{iteration:07d}.pt"))

    def load_checkpoint(self, path: str, **kw) -> Optional[int]:
        if hasattr(self.module, "engine"):
            st = self.loader.load(path, model=self.module, optimizer=self.optimizer)
            if st is None:
                return None
            if st.get("lr_scheduler"):
                self.lr_scheduler.load_state_dict(st["lr_scheduler"])
            return st.get("iteration")
        return None
