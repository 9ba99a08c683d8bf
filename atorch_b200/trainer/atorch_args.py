"""``AtorchArguments``: training arguments of ``AtorchTrainer`` (Hugging Face ``TrainingArguments``
field names where they overlap, plus the atorch_* fields that pick the acceleration strategy).
(Reference: atorch/trainer/atorch_args.py:20-399.)
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class AtorchArguments:
    output_dir: str = "./output"
    overwrite_output_dir: bool = False
    do_train: bool = True
    do_eval: bool = False
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 3.0
    max_steps: int = -1
    lr_scheduler_type: str = "linear"      # linear | cosine | constant | constant_with_warmup | log_warmup_linear_decay
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    logging_steps: int = 10
    logging_first_step: bool = False
    save_strategy: str = "steps"           # no | steps | epoch
    save_steps: int = 500
    save_total_limit: Optional[int] = None
    eval_strategy: str = "no"              # no | steps | epoch
    eval_steps: Optional[int] = None
    seed: int = 42
    bf16: bool = False
    fp16: bool = False
    gradient_checkpointing: bool = False
    dataloader_num_workers: int = 0
    dataloader_drop_last: bool = False
    resume_from_checkpoint: Optional[str] = None
    load_best_model_at_end: bool = False
    metric_for_best_model: Optional[str] = None
    greater_is_better: Optional[bool] = None
    ignore_write_errors: bool = False
    optim: str = "adamw"                   # adamw | agd | sgd
    # --- acceleration strategy -------------------------------------------------------------
    atorch_opt: str = "fsdp"               # fsdp | ddp
    atorch_parallel_mode: Optional[Tuple] = None
    atorch_load_strategy: Optional[List] = None
    atorch_module_replace: bool = True
    atorch_wrap_cls: Optional[Tuple] = None
    atorch_checkpoint_cls: Optional[Tuple] = None
    atorch_fsdp_config: Dict[str, Any] = field(default_factory=dict)
    save_by_streaming: bool = False        # flat-param sharded checkpoints (every rank writes its shards)
    load_by_streaming: bool = False
    async_save: bool = False
    async_timeout: int = 300
    max_num_writing_processes: int = 1
    save_load_by_streaming_dir: str = "streaming_ckpt"

    def to_dict(self) -> dict:
        d = asdict(self)
        for k in ("atorch_wrap_cls", "atorch_checkpoint_cls"):
            if d[k] is not None:
                d[k] = [c if isinstance(c, str) else getattr(c, "__name__", str(c)) for c in getattr(self, k)]
        return d

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, default=str)

    def build_strategy(self, world_size: int) -> list:
        if self.atorch_load_strategy is not None:
            return list(self.atorch_load_strategy)
        st: list = [("parallel_mode", self.atorch_parallel_mode or ([("data", world_size)], None))]
        if self.atorch_module_replace:
            st.append("module_replace")
        if self.atorch_opt == "fsdp":
            cfg = dict(self.atorch_fsdp_config)
            if self.atorch_wrap_cls:
                cfg.setdefault("atorch_wrap_cls", tuple(self.atorch_wrap_cls))
            st.append(("fsdp", cfg))
        if self.bf16 or self.fp16:
            import torch

            st.append(("amp_native", {"dtype": torch.bfloat16 if self.bf16 else torch.float16}))
        if self.gradient_checkpointing and (self.atorch_checkpoint_cls or self.atorch_wrap_cls):
            st.append(("checkpoint", {"wrap_class": tuple(self.atorch_checkpoint_cls or self.atorch_wrap_cls),
                                      "no_reentrant": True}))
        return st
