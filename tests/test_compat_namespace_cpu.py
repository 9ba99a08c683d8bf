"""The ``atorch`` import paths users of the original package rely on resolve to this framework."""
import importlib

import pytest

PATHS = [
    ("atorch", ["init_distributed", "reset_distributed", "rank", "local_rank", "world_size", "coworker_size"]),
    ("atorch.auto", ["auto_accelerate"]),
    ("atorch.auto.accelerate", ["auto_accelerate", "get_strategy", "save_strategy"]),
    ("atorch.auto.strategy", ["Strategy"]),
    ("atorch.auto.model_context", ["ModelContext"]),
    ("atorch.auto.clip_grad_norm", ["clip_grad_norm"]),
    ("atorch.auto.opt_lib.module_replace_optimization", ["register_replace_pair"]),
    ("atorch.distributed.distributed", ["create_parallel_group", "destroy_parallel_group", "parallel_group",
                                        "parallel_group_size", "parallel_rank", "parallel_group_and_ranks",
                                        "get_data_partition_rank_and_size", "get_device_mesh",
                                        "ParallelGroupContextManager"]),
    ("atorch.distributed", ["seq_all_to_all", "create_sequence_parallel_group", "get_sequence_parallel_group",
                            "get_sequence_parallel_rank", "get_sequence_parallel_size"]),
    ("atorch.distributed.run", ["main"]),
    ("atorch.local_sgd", ["LocalSGDConfig", "OuterOptimizerConfig", "GTAConfig", "OuterOptimPeriodicModelAverager",
                          "StatefulPostLocalSGDOptimizer", "patch_local_sgd_to_fsdp"]),
    ("atorch.optimizers", ["AGD", "WeightedSAM", "BF16Optimizer", "AdamL"]),
    ("atorch.optimizers.low_bit.optim", ["Q_AdamW", "Q_AGD", "Q_CAME", "Q_Adafactor"]),
    ("atorch.modules.transformer.layers", ["FlashAttnModule"]),
    ("atorch.modules.transformer.rmsnorm", ["AtorchRmsNorm"]),
    ("atorch.modules.transformer.losses", ["CrossEntropyLoss"]),
    ("atorch.modules.normalization", ["AtorchLayerNorm"]),
    ("atorch.modules.moe", ["MOELayer", "Experts", "TopkGate", "SwitchGate", "set_experts_process_group"]),
    ("atorch.modules.moe.grouped_gemm_moe", ["Grouped_GEMM_MoE"]),
    ("atorch.modules.fp8", ["ScaledLinear", "PrecisionSwitchableLinear", "set_linear_modules_precision",
                            "get_fp8_module_count"]),
    ("atorch.modules.fp8.quantized_grouped_linear", ["ATorchGroupedLinear"]),
    ("atorch.modules.distributed_modules.layers", ["RowParallelLinear", "ColumnParallelLinear",
                                                   "VocabParallelEmbedding"]),
    ("atorch.modules.distributed_modules.cross_entropy", ["vocab_parallel_cross_entropy"]),
    ("atorch.tensor_parallel.manual_tp", ["TPInfo", "tp_manual_shard_custom_fn"]),
    ("atorch.pipeline_parallel.pipe_module", ["PipeModuleConfig", "make_pipe_module"]),
    ("atorch.pipeline_parallel.pipe_schedule", ["make_pipe_schedule", "make_pipe_schedule_from_pipe_module"]),
    ("atorch.pipeline_parallel.pipe_partition", ["get_rank_stage_info"]),
    ("atorch.utils.fsdp_save_util", ["save_fsdp_flat_param", "save_fsdp_optim_param", "ShardTensorUtil", "ShardOptim",
                                     "ConvertFlatParam"]),
    ("atorch.utils.fsdp_async_ckpt_util", ["save_checkpoint"]),
    ("atorch.utils.meta_model_utils", ["init_empty_weights_with_disk_offload", "reload_meta_module",
                                       "record_module_init"]),
    ("atorch.utils.fsdp_init_util", ["FSDPCkptConfig", "FSDPInitFn"]),
    ("atorch.trainer.atorch_trainer", ["AtorchTrainer"]),
    ("atorch.trainer.atorch_args", ["AtorchArguments"]),
    ("atorch.trainer", ["AtorchTrainerV2", "AtorchTrainingArgs"]),
    ("atorch.trainer.fsdp.fsdp_shard_async_saver", ["FsdpShardCkptAsyncSaver"]),
    ("atorch.trainer.fsdp.fsdp_shard_dcp_loader", ["FsdpShardDcpCkptLoader"]),
    ("atorch.trainer.fsdp.fsdp_ckpt_saver", ["ExtraState"]),
    ("atorch.checkpoint.torch_checkpoint", ["TorchDCPCheckpointManager"]),
    ("atorch.fault_tolerance.hanging_detector", ["HangingDetector"]),
    ("atorch.data", ["ShmDataloader", "GpuPreLoader"]),
    ("atorch.utils.prof", ["AProfiler"]),
    ("atorch.utils.timer", ["ThroughputTimer"]),
    ("atorch.utils.loss_spike_utils", ["TokenLossSpike"]),
    ("atorch.common.util_func", ["data_to_device"]),
    ("atorch.local_sgd.configs.configs", ["LocalSGDConfig", "GTAConfig", "OuterOptimizerConfig"]),
    ("atorch.local_sgd.DDP.outer_optim_model_averager", ["OuterOptimPeriodicModelAverager"]),
    ("atorch.local_sgd.DDP.stateful_post_localSGD_optimizer", ["StatefulPostLocalSGDOptimizer"]),
    ("atorch.local_sgd.utils.anomaly_detection", ["OnlineDynamicEWMA"]),
    ("atorch.local_sgd.utils.reduce_methods", ["GTAReducer", "LinearReducer", "TensorReducer"]),
    ("atorch.local_sgd.utils.reduce_methods.sparsify", ["SparsificationMethod", "magnitude", "bernoulli", "sparsify"]),
    ("atorch.local_sgd.utils.reduce_methods.generalized_task_arithmetic", ["GTAReducer",
                                                                           "get_consensus_mask_distributed"]),
    ("atorch.auto.engine.acceleration_engine", ["AccelerationEngine"]),
    ("atorch.auto.task", ["Task"]),
    ("atorch.auto.opt_lib.half_optimization", ["HalfOptimization"]),
    ("atorch.auto.opt_lib.shard_planners.mip_tp_planner", ["MIPTensorParallelPlanner"]),
    ("atorch.optimizers.low_bit.optim.q_agd", ["Q_AGD"]),
    ("atorch.rl.replay_buffer.replay_buffer", ["ReplayBuffer"]),
    ("atorch.rl.trainer.ppo_trainer", ["PPOTrainer"]),
    ("atorch.trainer.base.atorch_train_engine", ["AtorchTrainEngine"]),
    ("atorch.mup.shape", ["set_base_shapes", "make_base_shapes", "save_base_shapes", "load_base_shapes"]),
    ("atorch.mup.optim", ["MuAdam", "MuSGD", "MuAdamParamGroupsAdjust"]),
    ("atorch.mup.init", ["normal_", "xavier_uniform_", "kaiming_normal_", "trunc_normal_"]),
    ("atorch.utils.path_utils", ["path_is_empty"]),
    ("atorch.common.singleton", ["SingletonMeta"]),
    ("atorch.utils.hooks", ["ATorchHooks"]),
    ("atorch.utils.metric_util", ["calc_mlm_acc", "MaskedLM"]),
    ("atorch.utils.graph_transform_utils", ["topo_sort", "map_aggregate", "combine_map_aggregate"]),
    ("atorch.utils.dev_utils", ["raise_not_impl"]),
    ("atorch.modules.distributed_modules.activation_checkpointing", [
        "CudaRNGStatesTracker", "get_cuda_rng_tracker", "model_parallel_cuda_manual_seed", "CheckpointFunction",
        "checkpoint", "TPCheckpointWrapper", "tp_wrap_fn"]),
    ("atorch.utils.trainer_utils", ["AtorchSchedulerType", "get_linear_schedule_with_log_warmup", "get_scheduler",
                                    "AsyncCheckpointSignal", "PipeMessageEntity"]),
    ("atorch.rl.ppo_utils.ppo_util", ["dist_fn", "get_kl_penalty", "get_rewards", "loss", "get_advantages_and_returns"]),
    ("atorch.rl.model_utils.model_util", ["RunningMoments", "FixedKLController", "get_tensor_stats", "whiten",
                                          "logprobs_of_labels", "flatten_dict", "hf_get_decoder_blocks", "make_head",
                                          "freeze_bottom_causal_layers", "get_global_statistics", "set_seed"]),
]


@pytest.mark.parametrize("mod,names", PATHS)
def test_import_path(mod, names):
    m = importlib.import_module(mod)
    for n in names:
        assert hasattr(m, n), f"{mod}.{n}"


def test_same_objects():
    import atorch_b200.auto
    from atorch.auto import auto_accelerate

    assert auto_accelerate is atorch_b200.auto.auto_accelerate
