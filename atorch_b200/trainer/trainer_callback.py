"""Callbacks of the engine-based trainer: state and control with the extra fields of the reference
(``steps_in_epoch``, ``current_step_in_epoch``, consumed samples / tokens, ``should_test``), the extra events
``on_evaluate_begin`` / ``on_save_begin`` / ``on_predict_begin`` / ``on_prediction_step``, a handler that
skips callbacks which do not define an event, and the stock callbacks:

* ``FlowCallbackV2``: turns the logging / evaluation / test / save intervals into control flags. Saving can
  be keyed on steps, on consumed samples (within half a global batch of a multiple of ``save_samples``), on
  listed steps inside an epoch, or on a list of global steps read from a JSON file that is re-read whenever
  its modification time changes (``{"save_at_dynamic_steps": [..]}``).
* ``PredictCallback``: progress bar over evaluation / prediction iterations on the printing rank.
* ``ProfilerCallback``: drives the profiler selected by ``profiler_type`` (``trainer/atorch_profiler.py``).

(Reference: atorch/trainer/trainer_callback.py:35-468.)
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import List, Optional

from ..common.log_utils import default_logger as logger
from .callbacks import CallbackHandler, TrainerCallback, TrainerControl, TrainerState


@dataclass
class AtorchTrainerState(TrainerState):
    steps_in_epoch: int = 0
    current_step_in_epoch: int = 0
    consumed_train_tokens: int = 0

    @classmethod
    def load_from_json(cls, json_path: str, origin_train_state_to_fill: Optional["AtorchTrainerState"] = None):
        """Keys of the file that this version does not know are dropped (files of newer versions stay
        loadable); with ``origin_train_state_to_fill`` the loaded values are copied into that object."""
        with open(json_path, encoding="utf-8") as f:
            sd = json.load(f)
        names = {f.name for f in fields(cls)}
        extra = set(sd) - names
        if extra:
            logger.info(f"keys {sorted(extra)} of {json_path} are not used by this version")
        new = cls(**{k: v for k, v in sd.items() if k in names})
        if origin_train_state_to_fill is not None:
            origin_train_state_to_fill.replace(new)
            return origin_train_state_to_fill
        return new

    def replace(self, new_state) -> None:
        for f in fields(new_state):
            setattr(self, f.name, getattr(new_state, f.name))


@dataclass
class AtorchTrainerControl(TrainerControl):
    should_test: bool = False

    def _new_step(self) -> None:
        self.should_test = False
        self.should_save = self.should_evaluate = self.should_log = False

    def _new_epoch(self) -> None:
        self.should_epoch_stop = False


class AtorchTrainerCallback(TrainerCallback):
    def on_evaluate_begin(self, args, state, control, **kw): pass
    def on_save_begin(self, args, state, control, **kw): pass
    def on_predict_begin(self, args, state, control, **kw): pass
    def on_prediction_step(self, args, state, control, **kw): pass
    def on_predict(self, args, state, control, **kw): pass


class AtorchCallbackHandler(CallbackHandler):
    """Every event goes through ``call_event_safely``: a callback that lacks the method is skipped, a
    callback that returns nothing leaves the control object unchanged."""

    def __init__(self, callbacks, model=None, optimizer=None, lr_scheduler=None, train_dataloader=None,
                 eval_dataloader=None):
        super().__init__(callbacks, model, optimizer, lr_scheduler)
        self.train_dataloader, self.eval_dataloader = train_dataloader, eval_dataloader

    def call_event_safely(self, event, args, state, control, **kw):
        for cb in self.callbacks:
            fn = getattr(cb, event, None)
            if fn is None:
                continue
            r = fn(args, state, control, model=self.model, optimizer=self.optimizer, lr_scheduler=self.lr_scheduler,
                   train_dataloader=self.train_dataloader, eval_dataloader=self.eval_dataloader, **kw)
            if r is not None:
                control = r
        return control

    call = call_event_safely

    def on_evaluate_begin(self, args, state, control, **kw):
        return self.call_event_safely("on_evaluate_begin", args, state, control, **kw)

    def on_save_begin(self, args, state, control, **kw):
        return self.call_event_safely("on_save_begin", args, state, control, **kw)

    def on_predict_begin(self, args, state, control, **kw):
        return self.call_event_safely("on_predict_begin", args, state, control, **kw)

    def on_prediction_step(self, args, state, control, **kw):
        return self.call_event_safely("on_prediction_step", args, state, control, **kw)


class _FileWatcher:
    """Returns the content of a file when its modification time has changed since the last read."""

    def __init__(self, path: str):
        self.path, self.mtime = path, None

    def read_if_modified(self) -> Optional[str]:
        try:
            m = os.path.getmtime(self.path)
        except OSError:
            return None
        if m == self.mtime:
            return None
        self.mtime = m
        with open(self.path) as f:
            return f.read()


class FlowCallbackV2(AtorchTrainerCallback):
    def __init__(self):
        self.watcher: Optional[_FileWatcher] = None
        self.save_at_dynamic_steps: List[int] = []

    def _read_dynamic(self, args) -> None:
        text = self.watcher.read_if_modified() if self.watcher is not None else None
        if text is None:
            return
        try:
            cfg = json.loads(text)
        except ValueError:
            logger.warning(f"{args.dynamic_save_config_path} is not valid JSON; ignored")
            return
        steps = cfg.get("save_at_dynamic_steps") if isinstance(cfg, dict) else None
        if isinstance(steps, list):
            self.save_at_dynamic_steps = [int(s) for s in steps]
            logger.info(f"[dynamic saving] checkpoints will be saved at global steps {self.save_at_dynamic_steps}")
        else:
            logger.warning(f"'save_at_dynamic_steps' in {args.dynamic_save_config_path} must be a list")

    def on_train_begin(self, args, state, control, **kw):
        if getattr(args, "dynamic_save_config_path", None):
            self.watcher = _FileWatcher(args.dynamic_save_config_path)
            self._read_dynamic(args)

    def on_step_begin(self, args, state, control, **kw):
        control.should_test = False

    def on_step_end(self, args, state, control, **kw):
        s = state.global_step
        if s == 1 and getattr(args, "logging_first_step", False):
            control.should_log = True
        if args.logging_strategy == "steps" and args.logging_steps and s % args.logging_steps == 0:
            control.should_log = True
        if (args.evaluation_strategy == "steps" and args.eval_steps and s % args.eval_steps == 0
                and args.eval_delay <= s):
            control.should_evaluate = True
        if args.test_strategy == "steps" and args.test_steps and s % args.test_steps == 0 and args.test_delay <= s:
            control.should_test = True
        gbs = args.global_train_batch_size
        by_samples = False
        if args.save_strategy == "samples" and args.save_samples > 0:
            rem = state.consumed_train_samples % args.save_samples
            by_samples = rem == 0 or rem <= gbs / 2 or (args.save_samples - rem) < gbs / 2
        self._read_dynamic(args)
        in_epoch = args.extra_save_frequency_in_epoch
        if ((args.save_strategy == "steps" and args.save_steps and args.save_steps > 0 and s % args.save_steps == 0)
                or by_samples or (in_epoch is not None and state.current_step_in_epoch in in_epoch)
                or s in self.save_at_dynamic_steps):
            control.should_save = True
            if args.test_on_save:
                control.should_test = True
        if s >= state.max_steps:
            control.should_training_stop = True
        return control

    def on_epoch_end(self, args, state, control, **kw):
        if args.logging_strategy == "epoch":
            control.should_log = True
        if args.evaluation_strategy == "epoch" and args.eval_delay <= state.epoch:
            control.should_evaluate = True
        if args.test_strategy == "epoch" and args.test_delay <= state.epoch:
            control.should_test = True
        if args.save_strategy == "epoch":
            control.should_save = True
        return control

    def on_evaluate_begin(self, args, state, control, eval_type=None, **kw):
        if eval_type is not None:
            args.eval_type = eval_type

    def on_evaluate(self, args, state, control, **kw):
        if getattr(args, "eval_type", None) == "test":
            control.should_test = False
        args.eval_type = None


class PredictCallback(AtorchTrainerCallback):
    def __init__(self):
        self.bar = None

    @staticmethod
    def should_print(args) -> bool:
        return bool(getattr(args, "is_main_process", True))

    def on_prediction_step(self, args, state, control, eval_iters=0, **kw):
        if self.should_print(args) and eval_iters > 0:
            if self.bar is None:
                from tqdm import tqdm

                self.bar = tqdm(total=eval_iters, dynamic_ncols=True)
            self.bar.update(1)

    def _close(self, args):
        if self.bar is not None:
            self.bar.close()
        self.bar = None

    def on_evaluate(self, args, state, control, **kw):
        self._close(args)

    def on_predict(self, args, state, control, **kw):
        self._close(args)


class ProfilerCallback(AtorchTrainerCallback):
    """``nv``: a scheduled torch profiler stepped once per training step; ``nsys``: brackets the steps
    ``[profile_step_start, profile_step_end]`` of the chosen ranks with cudaProfilerStart/Stop and NVTX
    ranges for an external tracer; ``nv_dp``: the file-driven dynamic profiler."""

    def __init__(self):
        self.prof = None
        self._nvtx = None

    def on_train_begin(self, args, state, control, **kw):
        from .atorch_profiler import get_profiler

        self.prof = get_profiler(args)
        if hasattr(self.prof, "start"):
            self.prof.start()

    def on_train_end(self, args, state, control, **kw):
        if hasattr(self.prof, "stop"):
            self.prof.stop()

    def _mine(self, args) -> bool:
        ranks = getattr(args, "profile_ranks", [-1])
        return ranks == [-1] or getattr(args, "process_index", 0) in ranks

    def on_step_begin(self, args, state, control, **kw):
        if args.profiler_type == "nsys" and state.global_step == args.profile_step_start and self._mine(args):
            import torch

            if torch.cuda.is_available():
                torch.cuda.cudart().cudaProfilerStart()
                self._nvtx = torch.autograd.profiler.emit_nvtx(record_shapes=True)
                self._nvtx.__enter__()

    def on_step_end(self, args, state, control, **kw):
        if args.profiler_type == "nsys":
            if state.global_step == args.profile_step_end and self._mine(args) and self._nvtx is not None:
                import torch

                self._nvtx.__exit__(None, None, None)
                self._nvtx = None
                torch.cuda.cudart().cudaProfilerStop()
        elif args.profiler_type == "nv_dp":
            from ..utils import dynamic_profiler

            if hasattr(dynamic_profiler, "step"):
                dynamic_profiler.step()
        elif self.prof is not None and hasattr(self.prof, "step"):
            self.prof.step()
