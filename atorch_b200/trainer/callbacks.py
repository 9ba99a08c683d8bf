"""Trainer state, control flags and callbacks (the subset of the Hugging Face callback protocol the
trainer drives: on_train_begin/end, on_epoch_begin/end, on_step_begin/end, on_log, on_evaluate, on_save).
(Reference: atorch/trainer/trainer_callback.py:35-468 and transformers.TrainerCallback.)
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional


@dataclass
class TrainerState:
    epoch: float = 0.0
    global_step: int = 0
    max_steps: int = 0
    num_train_epochs: int = 0
    total_flos: float = 0.0
    log_history: List[Dict] = field(default_factory=list)
    best_metric: Optional[float] = None
    best_model_checkpoint: Optional[str] = None
    consumed_train_samples: int = 0

    def save_to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=2, sort_keys=True)

    @classmethod
    def load_from_json(cls, path: str) -> "TrainerState":
        with open(path) as f:
            return cls(**json.load(f))


@dataclass
class TrainerControl:
    should_training_stop: bool = False
    should_epoch_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False


class TrainerCallback:
    def on_train_begin(self, args, state, control, **kw): pass
    def on_train_end(self, args, state, control, **kw): pass
    def on_epoch_begin(self, args, state, control, **kw): pass
    def on_epoch_end(self, args, state, control, **kw): pass
    def on_step_begin(self, args, state, control, **kw): pass
    def on_step_end(self, args, state, control, **kw): pass
    def on_log(self, args, state, control, logs=None, **kw): pass
    def on_evaluate(self, args, state, control, metrics=None, **kw): pass
    def on_save(self, args, state, control, **kw): pass


class CallbackHandler:
    def __init__(self, callbacks, model=None, optimizer=None, lr_scheduler=None):
        self.callbacks = [c() if isinstance(c, type) else c for c in (callbacks or [])]
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler

    def add_callback(self, cb):
        self.callbacks.append(cb() if isinstance(cb, type) else cb)

    def call(self, event: str, args, state, control, **kw):
        for cb in self.callbacks:
            r = getattr(cb, event)(args, state, control, model=self.model, optimizer=self.optimizer,
                                   lr_scheduler=self.lr_scheduler, **kw)
            if r is not None:
                control = r
        return control


class DefaultFlowCallback(TrainerCallback):
    """Turns the logging / evaluation / save intervals of the arguments into control flags."""

    def on_step_end(self, args, state, control, **kw):
        s = state.global_step
        if (s == 1 and args.logging_first_step) or (args.logging_steps > 0 and s % args.logging_steps == 0):
            control.should_log = True
        if args.eval_strategy == "steps" and args.eval_steps and s % args.eval_steps == 0:
            control.should_evaluate = True
        if args.save_strategy == "steps" and args.save_steps > 0 and s % args.save_steps == 0:
            control.should_save = True
        if s >= state.max_steps:
            control.should_training_stop = True
        return control

    def on_epoch_end(self, args, state, control, **kw):
        if args.eval_strategy == "epoch":
            control.should_evaluate = True
        if args.save_strategy == "epoch":
            control.should_save = True
        return control
