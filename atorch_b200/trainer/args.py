"""``AtorchTrainingArgs``: arguments of the engine-based trainer (``AtorchTrainerV2``). Field names follow
atorch/trainer/args.py:41-900; parallel layout fields (tensor / pipeline / context / expert sizes,
sequence parallel, micro and global batch sizes) configure the native engine of this framework instead
of Megatron. ``extra_configs`` is carried through to the engine unchanged."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class AtorchTrainingArgs:
    output_dir: str = "./output"
    distributed_type: str = "fsdp"            # fsdp | ddp | hybrid (tp/pp/dp) | megatron (alias of hybrid)
    do_train: bool = True
    do_eval: bool = False
    seed: int = 1234
    bf16: bool = True
    fp16: bool = False
    # batch sizes
    micro_batch_size: int = 1
    global_batch_size: Optional[int] = None
    seq_length: int = 4096
    # parallel layout
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    sequence_parallel: bool = False
    use_distributed_optimizer: bool = True
    # optimisation
    optimizer: str = "adamw"
    learning_rate: float = 3e-4
    min_lr: float = 0.0
    weight_decay: float = 0.01
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    lr_decay_style: str = "cosine"
    lr_warmup_iters: int = 0
    lr_warmup_fraction: Optional[float] = None
    train_iters: Optional[int] = None
    max_steps: int = -1
    num_train_epochs: float = 1.0
    recompute_granularity: Optional[str] = "full"     # None | selective | full
    # logging / eval / test / save (strategies: "no" | "steps" | "epoch", save also "samples")
    logging_strategy: str = "steps"
    logging_first_step: bool = False
    logging_steps: int = 10
    log_params_std: bool = False
    log_grad_diff_for_debug: bool = False
    tensorboard_dir: Optional[str] = None
    evaluation_strategy: str = "no"
    eval_steps: Optional[int] = None
    eval_iters: int = 10
    eval_delay: float = 0
    test_strategy: str = "no"
    test_steps: Optional[int] = None
    test_delay: float = 0
    test_on_save: bool = False
    save_strategy: str = "steps"
    save_steps: int = 500
    save_samples: int = 0                              # save_strategy="samples": every this many consumed samples
    extra_save_frequency_in_epoch: Optional[List[int]] = None   # extra saves at these steps inside every epoch
    dynamic_save_config_path: Optional[str] = None     # JSON {"save_at_dynamic_steps": [..]}, re-read when it changes
    save_total_limit: Optional[int] = None
    async_save: bool = True
    resume_from_checkpoint: Optional[str] = None
    # robustness
    spike_loss_ratio: Optional[float] = None          # scale gradients by this when the loss spikes
    spike_loss_threshold: float = 2.0                  # spike = loss > threshold * running mean
    manual_gc: bool = False
    manual_gc_interval: int = 0
    profiler_type: Optional[str] = None               # nv | nv_dp | nsys
    profiler_schedule_wait: int = 1
    profiler_schedule_warmup: int = 1
    profiler_schedule_active: int = 1
    profiler_schedule_repeat: int = 1
    profiler_schedule_skip_first: int = 0
    profiler_file_path: Optional[str] = None
    profiler_config: Dict[str, Any] = field(default_factory=dict)   # overrides of torch.profiler.profile keywords
    profile_ranks: List[int] = field(default_factory=lambda: [-1])  # [-1] = every rank
    profile_use_gzip: bool = False
    profile_step_start: int = 0                        # nsys: first / last profiled global step
    profile_step_end: int = 0
    dynamic_profiler_config_path: Optional[str] = None
    memory_snapshot_path: Optional[str] = None
    use_local_sgd: bool = False
    local_sgd_sync_interval: int = 1
    local_sgd_warmup_steps: int = 0
    extra_configs: Dict[str, Any] = field(default_factory=dict)

    eval_type: Optional[str] = None                    # set by the trainer around an evaluation ("eval" | "test")

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def process_index(self) -> int:
        import os

        return int(os.environ.get("RANK", "0"))

    @property
    def is_main_process(self) -> bool:
        return self.process_index == 0

    @property
    def global_train_batch_size(self) -> int:
        import os

        if self.global_batch_size:
            return self.global_batch_size
        return self.micro_batch_size * self.data_parallel_size(int(os.environ.get("WORLD_SIZE", "1")))

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, default=str)

    def data_parallel_size(self, world_size: int) -> int:
        mp = self.tensor_model_parallel_size * self.pipeline_model_parallel_size * self.context_parallel_size
        assert world_size % mp == 0, f"world size {world_size} not divisible by model-parallel size {mp}"
        return world_size // mp

    def num_micro_batches(self, world_size: int) -> int:
        dp = self.data_parallel_size(world_size)
        gbs = self.global_batch_size or self.micro_batch_size * dp
        assert gbs % (self.micro_batch_size * dp) == 0
        return gbs // (self.micro_batch_size * dp)
