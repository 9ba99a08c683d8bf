"""``AtorchTrainer``: Hugging-Face-style training loop on top of ``auto_accelerate``.

    trainer = AtorchTrainer(model, args, train_dataset=..., eval_dataset=..., data_collator=...,
                            compute_metrics=..., callbacks=[...], optimizers=(None, None))
    trainer.train(resume_from_checkpoint=None);  trainer.evaluate();  trainer.save_model()

The acceleration strategy is derived from the arguments (``AtorchArguments.build_strategy``):
parallel groups, module replacement, sharded data parallel (``atorch_opt="fsdp"``) or DDP, bf16/fp16
autocast, activation checkpointing. The loop does gradient accumulation, strategy-aware clipping,
LR scheduling, logging (loss reduced over ranks), evaluation, and checkpointing into
``checkpoint-{step}/`` (weights as a full state dict or as flat sharded files when
``save_by_streaming``; optimizer, scheduler, ``trainer_state.json``, ``rng_state_{rank}.pth``) with
rotation (``save_total_limit``), best-model tracking, resume, and optional asynchronous writing.
(Reference: atorch/trainer/atorch_trainer.py:142-2693.)
"""
from __future__ import annotations

import math
import os
import random
import re
import shutil
import threading
import time
from typing import Callable, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from ..auto.accelerate import auto_accelerate
from ..auto.clip_grad_norm import clip_grad_norm
from ..common.log_utils import default_logger as logger
from ..common.util_func import data_to_device
from ..distributed import distributed as D
from .atorch_args import AtorchArguments
from .callbacks import CallbackHandler, DefaultFlowCallback, TrainerControl, TrainerState

PREFIX_CHECKPOINT_DIR = "checkpoint"


def get_scheduler(name: str, optimizer, num_warmup_steps: int, num_training_steps: int):
    from ..parallel.fsdp import FusedShardedOptimizer
    from ..auto.model_context import _SchedulerShim
    from ..utils.trainer_utils import log_warmup_linear_decay_factor

    target = getattr(optimizer, "optimizer", optimizer)
    if not isinstance(target, torch.optim.Optimizer):
        target = _SchedulerShim(optimizer)

    def lam(step: int) -> float:
        if name == "constant":
            return 1.0
        if name == "log_warmup_linear_decay":
            return log_warmup_linear_decay_factor(step, num_warmup_steps, num_training_steps)
        if step < num_warmup_steps:
            return step / max(1, num_warmup_steps)
        if name == "constant_with_warmup":
            return 1.0
        prog = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
        if name == "cosine":
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * min(prog, 1.0))))
        return max(0.0, 1.0 - prog)          # linear, log_warmup_linear_decay
    return torch.optim.lr_scheduler.LambdaLR(target, lam)


class _AsyncWriter:
    """Background thread that writes host copies of checkpoint payloads; ``wait()`` before the next save."""

    def __init__(self, timeout: float):
        self.timeout, self.thread, self.error = timeout, None, None

    def submit(self, fn: Callable[[], None]) -> None:
        self.wait()

        def run():
            try:
                fn()
            except Exception as e:  # reported at the next wait()
                self.error = e
        self.thread = threading.Thread(target=run, daemon=True)
        self.thread.start()

    def wait(self) -> None:
        if self.thread is not None:
            self.thread.join(self.timeout)
            self.thread = None
        if self.error is not None:
            e, self.error = self.error, None
            raise e


class AtorchTrainer:
    def __init__(self, model, args: Optional[AtorchArguments] = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, tokenizer=None, compute_metrics: Optional[Callable] = None, callbacks=None,
                 optimizers=(None, None), loss_func: Optional[Callable] = None, prepare_input=None,
                 optim_func=None, optim_args=None, **kwargs):
        self.args = args or AtorchArguments()
        self.data_collator, self.train_dataset, self.eval_dataset = data_collator, train_dataset, eval_dataset
        self.tokenizer, self.compute_metrics = tokenizer, compute_metrics
        self.state, self.control = TrainerState(), TrainerControl()
        self._set_seed(self.args.seed)
        self.world = D.world_size() or 1
        self.rank = D.rank() or 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
            (D.backend() is None or "nccl" in (D.backend() or "")) else torch.device("cpu")
        self.loss_func = loss_func or self._default_loss
        self._atorch_init(model, optimizers, optim_func, optim_args, prepare_input)
        self.callback_handler = CallbackHandler([DefaultFlowCallback] + list(callbacks or []), self.model,
                                                self.optimizer, self.lr_scheduler)
        self._writer = _AsyncWriter(self.args.async_timeout) if self.args.async_save else None
        os.makedirs(self.args.output_dir, exist_ok=True)

    # ------------------------------------------------------------------------------- set-up
    @staticmethod
    def _set_seed(seed: int) -> None:
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)

    @staticmethod
    def _default_loss(batch, outputs):
        if isinstance(outputs, dict):
            return outputs["loss"]
        if hasattr(outputs, "loss") and outputs.loss is not None:
            return outputs.loss
        return outputs[0] if isinstance(outputs, (tuple, list)) else outputs

    def _atorch_init(self, model, optimizers, optim_func, optim_args, prepare_input) -> None:
        a = self.args
        if optim_func is None:
            from ..optimizers import AGD

            optim_func = {"adamw": torch.optim.AdamW, "agd": AGD, "sgd": torch.optim.SGD}[a.optim]
        if optim_args is None:
            optim_args = {"lr": a.learning_rate, "weight_decay": a.weight_decay}
            if a.optim in ("adamw", "agd"):
                optim_args["betas"] = (a.adam_beta1, a.adam_beta2)
            if a.optim == "adamw":
                optim_args["eps"] = a.adam_epsilon
        ok, res, self.strategy = auto_accelerate(
            model, optim_func if optimizers[0] is None else None, loss_func=self.loss_func,
            prepare_input=prepare_input or data_to_device, model_input_format="unpack_dict", optim_args=optim_args,
            load_strategy=a.build_strategy(self.world), ignore_dryrun_on_load_strategy=True)
        if not ok:
            raise RuntimeError("auto_accelerate failed to apply the strategy built from the arguments")
        self.model, self.loss_func, self.prepare_input = res.model, res.loss_func, res.prepare_input
        self.optimizer = optimizers[0] if optimizers[0] is not None else res.optim
        self.lr_scheduler = optimizers[1]

    def get_train_dataloader(self) -> DataLoader:
        rank, size = D.get_data_partition_rank_and_size()
        # the order of an epoch depends only on (seed, epoch), so a resumed run replays it exactly
        sampler = torch.utils.data.distributed.DistributedSampler(self.train_dataset, num_replicas=size, rank=rank,
                                                                  seed=self.args.seed)
        return DataLoader(self.train_dataset, batch_size=self.args.per_device_train_batch_size, sampler=sampler,
                          collate_fn=self.data_collator, num_workers=self.args.dataloader_num_workers,
                          drop_last=self.args.dataloader_drop_last)

    def get_eval_dataloader(self, eval_dataset=None) -> DataLoader:
        ds = eval_dataset if eval_dataset is not None else self.eval_dataset
        rank, size = D.get_data_partition_rank_and_size()
        sampler = torch.utils.data.distributed.DistributedSampler(ds, num_replicas=size, rank=rank, shuffle=False) \
            if size > 1 else None
        return DataLoader(ds, batch_size=self.args.per_device_eval_batch_size, sampler=sampler, shuffle=False,
                          collate_fn=self.data_collator, num_workers=self.args.dataloader_num_workers)

    # -------------------------------------------------------------------------------- train
    def compute_loss(self, batch):
        batch = self.prepare_input(batch, self.device) if self.prepare_input else batch
        outputs = self.model(**batch) if isinstance(batch, dict) else self.model(batch)
        return self.loss_func(batch, outputs)

    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        loader = self.get_train_dataloader()
        steps_per_epoch = max(len(loader) // a.gradient_accumulation_steps, 1)
        max_steps = a.max_steps if a.max_steps > 0 else int(math.ceil(a.num_train_epochs * steps_per_epoch))
        epochs = int(math.ceil(max_steps / steps_per_epoch))
        self.state.max_steps, self.state.num_train_epochs = max_steps, epochs
        if self.lr_scheduler is None:
            warm = a.warmup_steps if a.warmup_steps > 0 else int(a.warmup_ratio * max_steps)
            self.lr_scheduler = get_scheduler(a.lr_scheduler_type, self.optimizer, warm, max_steps)
            self.callback_handler.lr_scheduler = self.lr_scheduler
        resume = resume_from_checkpoint or a.resume_from_checkpoint
        if resume is True or resume == "latest":
            resume = self.get_last_checkpoint(a.output_dir)
        start_epoch, skip_batches = 0, 0
        if resume:
            self._load_checkpoint(resume)
            start_epoch = self.state.global_step // steps_per_epoch
            skip_batches = (self.state.global_step % steps_per_epoch) * a.gradient_accumulation_steps
        self.control = self.callback_handler.call("on_train_begin", a, self.state, self.control)
        self.model.train()
        tr_loss = torch.zeros((), device=self.device)
        logged_steps, t_start = self.state.global_step, time.time()
        for epoch in range(start_epoch, epochs):
            if hasattr(loader, "sampler") and hasattr(loader.sampler, "set_epoch"):
                loader.sampler.set_epoch(epoch)
            self.control = self.callback_handler.call("on_epoch_begin", a, self.state, self.control)
            for i, batch in enumerate(loader):
                if skip_batches > 0:
                    skip_batches -= 1
                    continue
                boundary = (i + 1) % a.gradient_accumulation_steps == 0 or (i + 1) == len(loader)
                if i % a.gradient_accumulation_steps == 0:
                    self.control = self.callback_handler.call("on_step_begin", a, self.state, self.control)
                loss = self.compute_loss(batch)
                (loss / a.gradient_accumulation_steps).backward()
                tr_loss += loss.detach().float() / a.gradient_accumulation_steps
                if not boundary:
                    continue
                grad_norm = None
                if a.max_grad_norm and a.max_grad_norm > 0:
                    grad_norm = clip_grad_norm(self.model, a.max_grad_norm, optimizer=self.optimizer)
                self.optimizer.step()
                if not getattr(self.optimizer, "step_was_skipped", False):
                    self.lr_scheduler.step()
                self.optimizer.zero_grad()
                self.state.global_step += 1
                self.state.epoch = epoch + (i + 1) / len(loader)
                self.state.consumed_train_samples += a.per_device_train_batch_size * \
                    a.gradient_accumulation_steps * self.world
                self.control = self.callback_handler.call("on_step_end", a, self.state, self.control)
                tr_loss, logged_steps = self._maybe_log_save_evaluate(tr_loss, logged_steps, grad_norm, t_start)
                if self.control.should_training_stop:
                    break
            self.control = self.callback_handler.call("on_epoch_end", a, self.state, self.control)
            tr_loss, logged_steps = self._maybe_log_save_evaluate(tr_loss, logged_steps, None, t_start)
            if self.control.should_training_stop:
                break
        if self._writer is not None:
            self._writer.wait()
        self.control = self.callback_handler.call("on_train_end", a, self.state, self.control)
        if a.load_best_model_at_end and self.state.best_model_checkpoint:
            self._load_checkpoint(self.state.best_model_checkpoint, model_only=True)
        return self.state

    def _maybe_log_save_evaluate(self, tr_loss, logged_steps, grad_norm, t_start):
        a = self.args
        if self.control.should_log and self.state.global_step > logged_steps:
            t = tr_loss.clone()
            if self.world > 1:
                dist.all_reduce(t)
                t /= self.world
            n = self.state.global_step - logged_steps
            logs = {"loss": round(t.item() / n, 6), "learning_rate": self.optimizer.param_groups[0]["lr"],
                    "epoch": round(self.state.epoch, 4), "step": self.state.global_step,
                    "samples_per_second": round(self.state.consumed_train_samples / max(time.time() - t_start, 1e-9), 3)}
            if grad_norm is not None:
                logs["grad_norm"] = float(grad_norm)
            self.log(logs)
            tr_loss = torch.zeros_like(tr_loss)
            logged_steps = self.state.global_step
        self.control.should_log = False
        metrics = None
        if self.control.should_evaluate and self.eval_dataset is not None:
            metrics = self.evaluate()
        self.control.should_evaluate = False
        if self.control.should_save:
            self._save_checkpoint(metrics)
            self.control = self.callback_handler.call("on_save", a, self.state, self.control)
        self.control.should_save = False
        return tr_loss, logged_steps

    def log(self, logs: Dict) -> None:
        self.state.log_history.append(dict(logs))
        self.control = self.callback_handler.call("on_log", self.args, self.state, self.control, logs=logs)
        if self.rank == 0:
            logger.info(str(logs))

    # ------------------------------------------------------------------------------ evaluate
    @torch.no_grad()
    def evaluate(self, eval_dataset=None, metric_key_prefix: str = "eval") -> Dict[str, float]:
        was_training = self.model.training
        self.model.eval()
        total, count, preds, labels = torch.zeros((), device=self.device), 0, [], []
        for batch in self.get_eval_dataloader(eval_dataset):
            b = self.prepare_input(batch, self.device) if self.prepare_input else batch
            out = self.model(**b) if isinstance(b, dict) else self.model(b)
            total += self.loss_func(b, out).detach().float()
            count += 1
            if self.compute_metrics is not None:
                logits = out["logits"] if isinstance(out, dict) else (out.logits if hasattr(out, "logits") else
                                                                      (out[1] if isinstance(out, (tuple, list)) else out))
                preds.append(logits.detach().float().cpu())
                if isinstance(b, dict) and "labels" in b:
                    labels.append(b["labels"].detach().cpu())
        stats = torch.stack([total, torch.tensor(float(count), device=self.device)])
        if self.world > 1:
            dist.all_reduce(stats)
        metrics = {f"{metric_key_prefix}_loss": (stats[0] / stats[1].clamp(min=1)).item()}
        if self.compute_metrics is not None and preds:
            from types import SimpleNamespace

            extra = self.compute_metrics(SimpleNamespace(predictions=torch.cat(preds).numpy(),
                                                         label_ids=torch.cat(labels).numpy() if labels else None))
            metrics.update({f"{metric_key_prefix}_{k}": v for k, v in extra.items()})
        self.log(metrics)
        self.control = self.callback_handler.call("on_evaluate", self.args, self.state, self.control, metrics=metrics)
        self.model.train(was_training)
        return metrics

    # ---------------------------------------------------------------------------- checkpoints
    @staticmethod
    def get_last_checkpoint(folder: str) -> Optional[str]:
        pat = re.compile(rf"^{PREFIX_CHECKPOINT_DIR}-(\d+)$")
        found = [(int(m.group(1)), d) for d in os.listdir(folder) if (m := pat.match(d))] if os.path.isdir(folder) else []
        return os.path.join(folder, max(found)[1]) if found else None

    def _is_sharded(self) -> bool:
        return hasattr(self.model, "engine")

    def save_model(self, output_dir: Optional[str] = None) -> None:
        out = output_dir or self.args.output_dir
        os.makedirs(out, exist_ok=True)
        if self._is_sharded() and self.args.save_by_streaming:
            from ..utils.fsdp_save_util import save_fsdp_flat_param

            save_fsdp_flat_param(self.model, os.path.join(out, self.args.save_load_by_streaming_dir))
            return
        sd = self.model.state_dict()
        if self.rank == 0:
            self._write(lambda: torch.save(sd, os.path.join(out, "pytorch_model.bin")))

    def _write(self, fn: Callable[[], None]) -> None:
        def safe():
            try:
                fn()
            except OSError as e:
                if not self.args.ignore_write_errors:
                    raise
                logger.warning("checkpoint write failed and was ignored: %s", e)
        if self._writer is not None:
            self._writer.submit(safe)
        else:
            safe()

    def save_optimizer(self, out: str) -> None:
        if self._is_sharded():
            from ..utils.fsdp_save_util import save_fsdp_optim_param

            save_fsdp_optim_param(self.model, self.optimizer, os.path.join(out, self.args.save_load_by_streaming_dir))
        elif self.rank == 0:
            sd = self.optimizer.state_dict()
            self._write(lambda: torch.save(sd, os.path.join(out, "optimizer.pt")))

    def _save_checkpoint(self, metrics=None) -> None:
        a = self.args
        out = os.path.join(a.output_dir, f"{PREFIX_CHECKPOINT_DIR}-{self.state.global_step}")
        os.makedirs(out, exist_ok=True)
        if self._writer is not None:
            self._writer.wait()
        self.save_model(out)
        self.save_optimizer(out)
        rng = {"python": random.getstate(), "numpy": np.random.get_state(), "cpu": torch.get_rng_state()}
        if torch.cuda.is_available():
            rng["cuda"] = torch.cuda.get_rng_state()
        torch.save(rng, os.path.join(out, f"rng_state_{self.rank}.pth" if self.world > 1 else "rng_state.pth"))
        if metrics is not None and a.metric_for_best_model:
            key = a.metric_for_best_model if a.metric_for_best_model.startswith("eval_") else \
                f"eval_{a.metric_for_best_model}"
            if key in metrics:
                greater = a.greater_is_better if a.greater_is_better is not None else not key.endswith("loss")
                v = metrics[key]
                if self.state.best_metric is None or (v > self.state.best_metric if greater else v < self.state.best_metric):
                    self.state.best_metric, self.state.best_model_checkpoint = v, out
        if self.rank == 0:
            torch.save(self.lr_scheduler.state_dict(), os.path.join(out, "scheduler.pt"))
            self.state.save_to_json(os.path.join(out, "trainer_state.json"))
            with open(os.path.join(out, "training_args.json"), "w") as f:
                f.write(a.to_json_string())
        if self.world > 1:
            dist.barrier()
        if self.rank == 0:
            self._rotate_checkpoints()

    def _rotate_checkpoints(self) -> None:
        limit = self.args.save_total_limit
        if not limit or limit <= 0:
            return
        pat = re.compile(rf"^{PREFIX_CHECKPOINT_DIR}-(\d+)$")
        found = sorted((int(m.group(1)), d) for d in os.listdir(self.args.output_dir) if (m := pat.match(d)))
        keep_best = self.state.best_model_checkpoint
        removable = [os.path.join(self.args.output_dir, d) for _, d in found]
        removable = [p for p in removable if p != keep_best]
        extra = len(found) - limit
        for p in removable[:max(extra, 0)]:
            shutil.rmtree(p, ignore_errors=True)

    def _load_checkpoint(self, path: str, model_only: bool = False) -> None:
        a = self.args
        stream_dir = os.path.join(path, a.save_load_by_streaming_dir)
        if self._is_sharded() and os.path.isdir(stream_dir) and os.path.exists(os.path.join(stream_dir, "ckpt_meta")):
            from ..utils.fsdp_save_util import ShardOptim, load_fsdp_flat_param

            load_fsdp_flat_param(self.model, stream_dir)
            if not model_only and os.path.exists(os.path.join(stream_dir, "optim_meta")):
                ShardOptim(stream_dir).load_into(self.model, self.optimizer)
        else:
            f = os.path.join(path, "pytorch_model.bin")
            if os.path.exists(f):
                self.model.load_state_dict(torch.load(f, map_location="cpu"))
            o = os.path.join(path, "optimizer.pt")
            if not model_only and os.path.exists(o) and not self._is_sharded():
                self.optimizer.load_state_dict(torch.load(o, map_location="cpu"))
        if model_only:
            return
        s = os.path.join(path, "scheduler.pt")
        if os.path.exists(s):
            self.lr_scheduler.load_state_dict(torch.load(s))
        st = os.path.join(path, "trainer_state.json")
        if os.path.exists(st):
            self.state = TrainerState.load_from_json(st)
        r = os.path.join(path, f"rng_state_{self.rank}.pth" if self.world > 1 else "rng_state.pth")
        if os.path.exists(r):
            rng = torch.load(r, weights_only=False)
            random.setstate(rng["python"])
            np.random.set_state(rng["numpy"])
            torch.set_rng_state(rng["cpu"])
            if "cuda" in rng and torch.cuda.is_available():
                torch.cuda.set_rng_state(rng["cuda"])
