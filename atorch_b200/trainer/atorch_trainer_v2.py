"""``AtorchTrainerV2``: engine-based trainer. The loop pulls ``num_micro_batches`` batches per step from an
endless iterator, calls the engine, tracks consumed samples / tokens, logs, evaluates, saves (sharded,
asynchronous), resumes, and optionally runs manual garbage collection and a torch profiler window.
(Reference: atorch/trainer/atorch_trainer_v2.py:111-942.)"""
from __future__ import annotations

import gc
import os
import time
from typing import Callable, Dict, Iterator, List, Optional

import torch
from torch.utils.data import DataLoader

from ..common.log_utils import default_logger as logger
from ..distributed import distributed as D
from .args import AtorchTrainingArgs
from .trainer_callback import (AtorchCallbackHandler, AtorchTrainerControl, AtorchTrainerState, FlowCallbackV2,
                               PredictCallback, ProfilerCallback)
from .engine import AtorchTrainEngine, NativeTrainEngine


def _endless(loader):
    epoch = 0
    while True:
        if hasattr(getattr(loader, "sampler", None), "set_epoch"):
            loader.sampler.set_epoch(epoch)
        for b in loader:
            yield b
        epoch += 1


class AtorchTrainerV2:
    def __init__(self, args: AtorchTrainingArgs, model: Optional[torch.nn.Module] = None, train_dataset=None,
                 eval_dataset=None, data_collator=None, loss_func: Optional[Callable] = None, wrap_cls=None,
                 callbacks: Optional[List] = None, train_engine: Optional[AtorchTrainEngine] = None, optim_func=None,
                 test_dataset=None):
        self.args = args
        self.world, self.rank = D.world_size() or 1, D.rank() or 0
        self.train_dataset, self.eval_dataset, self.data_collator = train_dataset, eval_dataset, data_collator
        self.test_dataset = test_dataset
        torch.manual_seed(args.seed)
        self.max_steps = args.max_steps if args.max_steps > 0 else (args.train_iters or self._steps_from_epochs())
        self.train_engine = train_engine or NativeTrainEngine(args, model, loss_func, wrap_cls, optim_func,
                                                              total_steps=self.max_steps)
        self.state, self.control = AtorchTrainerState(max_steps=self.max_steps), AtorchTrainerControl()
        # stock callbacks first (flow control, progress bar, profiler when one is selected), then the user's
        stock = [FlowCallbackV2(), PredictCallback()] + ([ProfilerCallback()] if args.profiler_type else [])
        self.callback_handler = AtorchCallbackHandler(stock + list(callbacks or []),
                                                      getattr(self.train_engine, "module", None),
                                                      getattr(self.train_engine, "optimizer", None),
                                                      getattr(self.train_engine, "lr_scheduler", None))
        self.consumed_train_tokens = 0
        os.makedirs(args.output_dir, exist_ok=True)

    def _steps_from_epochs(self) -> int:
        a = self.args
        dp = a.data_parallel_size(self.world)
        per_step = a.micro_batch_size * dp * a.num_micro_batches(self.world)
        n = len(self.train_dataset) if self.train_dataset is not None else per_step
        return max(int(a.num_train_epochs * n // per_step), 1)

    def _loader(self, ds, shuffle: bool) -> DataLoader:
        rank, size = D.get_data_partition_rank_and_size()
        sampler = torch.utils.data.distributed.DistributedSampler(ds, num_replicas=size, rank=rank, shuffle=shuffle,
                                                                  seed=self.args.seed)
        return DataLoader(ds, batch_size=self.args.micro_batch_size, sampler=sampler, collate_fn=self.data_collator,
                          drop_last=True)

    def train(self, resume_from_checkpoint: Optional[str] = None) -> AtorchTrainerState:
        a, eng = self.args, self.train_engine
        resume = resume_from_checkpoint or a.resume_from_checkpoint
        if resume:
            it = eng.load_checkpoint(resume)
            if it is not None:
                self.state.global_step = it
        loader = self._loader(self.train_dataset, True)
        data = _endless(loader)
        nmb = a.num_micro_batches(self.world)
        per_step = a.micro_batch_size * a.data_parallel_size(self.world) * nmb
        self.state.steps_in_epoch = max(len(loader) // nmb, 1)
        for _ in range(self.state.global_step * nmb):
            next(data)                                           # skip what a resumed run already consumed
        cb = self.callback_handler
        self.control = cb.call("on_train_begin", a, self.state, self.control)
        eng.train()
        t0, window = time.time(), []
        while self.state.global_step < self.max_steps:
            self.control._new_step()
            in_epoch = self.state.global_step % self.state.steps_in_epoch
            if in_epoch == 0:
                self.control._new_epoch()
                self.control = cb.call("on_epoch_begin", a, self.state, self.control)
            self.control = cb.call("on_step_begin", a, self.state, self.control)
            out = eng(data)
            self.state.global_step += 1
            self.state.current_step_in_epoch = in_epoch + 1
            self.state.epoch = self.state.global_step / self.state.steps_in_epoch
            self.state.consumed_train_samples += per_step
            self.state.consumed_train_tokens += per_step * a.seq_length
            self.consumed_train_tokens = self.state.consumed_train_tokens
            window.append(out["loss"])
            self.control = cb.call("on_step_end", a, self.state, self.control)
            if self.state.current_step_in_epoch == self.state.steps_in_epoch:
                self.control = cb.call("on_epoch_end", a, self.state, self.control)
            s = self.state.global_step
            if self.control.should_log and window:
                logs = {"loss": sum(window) / len(window), "lr": out.get("lr"), "grad_norm": out.get("grad_norm"),
                        "step": s, "consumed_train_samples": self.state.consumed_train_samples,
                        "consumed_train_tokens": self.consumed_train_tokens,
                        "tokens_per_sec": self.consumed_train_tokens / max(time.time() - t0, 1e-9)}
                window = []
                self.state.log_history.append(logs)
                self.control = cb.call("on_log", a, self.state, self.control, logs=logs)
                if self.rank == 0:
                    logger.info(str(logs))
            if self.control.should_evaluate and self.eval_dataset is not None:
                self.evaluate()
                eng.train()
            if self.control.should_test and (self.test_dataset or self.eval_dataset) is not None:
                self.evaluate(eval_type="test")
                eng.train()
            if self.control.should_save:
                self.control = cb.on_save_begin(a, self.state, self.control)
                eng.save_checkpoint(s, a.output_dir, consumed_train_samples=self.state.consumed_train_samples)
                if self.rank == 0:
                    self.state.save_to_json(os.path.join(a.output_dir, "trainer_state.json"))
                self.control = cb.call("on_save", a, self.state, self.control)
            if a.manual_gc and a.manual_gc_interval and s % a.manual_gc_interval == 0:
                gc.collect()
            if self.control.should_training_stop:
                break
        if hasattr(eng, "saver"):
            eng.saver.finish()
        self.control = cb.call("on_train_end", a, self.state, self.control)
        return self.state

    def evaluate(self, eval_type: str = "eval") -> Dict[str, float]:
        ds = self.test_dataset if (eval_type == "test" and self.test_dataset is not None) else self.eval_dataset
        cb = self.callback_handler
        self.control = cb.on_evaluate_begin(self.args, self.state, self.control, eval_type=eval_type)
        data = iter(self._loader(ds, False))
        self.train_engine.eval()
        losses = []
        for _ in range(self.args.eval_iters):
            try:
                losses.append(self.train_engine(data)["loss"])
            except StopIteration:
                break
            self.control = cb.on_prediction_step(self.args, self.state, self.control, eval_iters=self.args.eval_iters)
        m = {f"{eval_type}_loss": sum(losses) / max(len(losses), 1)}
        self.state.log_history.append(m)
        self.control = cb.call("on_evaluate", self.args, self.state, self.control, metrics=m)
        return m
