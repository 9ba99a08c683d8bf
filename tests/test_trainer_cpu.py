"""AtorchTrainer on CPU: training, logging, evaluation with metrics, checkpoint rotation, resume."""
import os

import pytest
import torch
import torch.nn as nn

from atorch_b200.trainer import AtorchArguments, AtorchTrainer, TrainerCallback


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.body = nn.Sequential(nn.Linear(8, 32), nn.ReLU(), nn.Linear(32, 3))

    def forward(self, x, labels=None):
        logits = self.body(x)
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = nn.functional.cross_entropy(logits, labels)
        return out


def dataset(n=96):
    g = torch.Generator().manual_seed(1)
    w = torch.randn(8, 3, generator=g)
    xs = torch.randn(n, 8, generator=g)
    return [{"x": x, "labels": (x @ w).argmax()} for x in xs]


def args(tmp_path, **kw):
    d = dict(output_dir=str(tmp_path), per_device_train_batch_size=8, learning_rate=5e-2, num_train_epochs=2,
             logging_steps=4, save_steps=6, save_total_limit=2, atorch_opt="ddp", atorch_module_replace=False,
             max_grad_norm=1.0, lr_scheduler_type="cosine", warmup_steps=2, eval_strategy="epoch",
             metric_for_best_model="accuracy")
    d.update(kw)
    return AtorchArguments(**d)


def accuracy(p):
    return {"accuracy": float((p.predictions.argmax(-1) == p.label_ids).mean())}


def test_train_eval_rotate_resume(tmp_path):
    seen = []

    class CB(TrainerCallback):
        def on_log(self, args, state, control, logs=None, **kw):
            seen.append(logs)
    tr = AtorchTrainer(Net(), args(tmp_path), train_dataset=dataset(), eval_dataset=dataset(32),
                       compute_metrics=accuracy, callbacks=[CB()])
    state = tr.train()
    assert state.global_step == 24
    losses = [l["loss"] for l in state.log_history if "loss" in l]
    assert losses[-1] < losses[0]
    evals = [l for l in state.log_history if "eval_accuracy" in l]
    assert len(evals) == 2 and evals[-1]["eval_accuracy"] > 0.5 and seen
    ckpts = sorted(d for d in os.listdir(tmp_path) if d.startswith("checkpoint-"))
    assert len(ckpts) <= 3 and "checkpoint-24" in ckpts
    for f in ("pytorch_model.bin", "optimizer.pt", "scheduler.pt", "trainer_state.json", "rng_state.pth"):
        assert os.path.exists(tmp_path / "checkpoint-24" / f), f
    # resume from step 18 and reach the same final weights
    ref = {k: v.clone() for k, v in tr.model.state_dict().items()}
    tr2 = AtorchTrainer(Net(), args(tmp_path, save_steps=1000, eval_strategy="no"), train_dataset=dataset())
    tr2.train(resume_from_checkpoint=str(tmp_path / "checkpoint-18"))
    assert tr2.state.global_step == 24
    for k, v in tr2.model.state_dict().items():
        assert torch.allclose(v, ref[k], atol=1e-5), k


def test_sharded_streaming_checkpoint_and_async(tmp_path):
    a = args(tmp_path, atorch_opt="fsdp", atorch_wrap_cls=(nn.Linear,), save_by_streaming=True, async_save=True,
             num_train_epochs=1, eval_strategy="no", metric_for_best_model=None)
    tr = AtorchTrainer(Net(), a, train_dataset=dataset())
    tr.train()
    last = AtorchTrainer.get_last_checkpoint(str(tmp_path))
    assert last.endswith("checkpoint-12") and os.path.exists(os.path.join(last, "streaming_ckpt", "ckpt_meta"))
    tr2 = AtorchTrainer(Net(), a, train_dataset=dataset())
    tr2.lr_scheduler = torch.optim.lr_scheduler.LambdaLR(
        __import__("atorch_b200.auto.model_context", fromlist=["_SchedulerShim"])._SchedulerShim(tr2.optimizer),
        lambda s: 1.0)
    tr2._load_checkpoint(last)
    for (k, v), (_, v2) in zip(tr.model.state_dict().items(), tr2.model.state_dict().items()):
        assert torch.equal(v, v2), k


def test_trainer_v2_engine_loop_and_resume(tmp_path):
    from atorch_b200.trainer import AtorchTrainerV2, AtorchTrainingArgs

    a = AtorchTrainingArgs(output_dir=str(tmp_path), bf16=False, micro_batch_size=4, global_batch_size=8,
                           learning_rate=5e-2, max_steps=12, logging_steps=4, save_steps=6, seq_length=1,
                           lr_warmup_iters=2, recompute_granularity=None, async_save=True, spike_loss_ratio=0.5)
    tr = AtorchTrainerV2(a, Net(), train_dataset=dataset(), eval_dataset=dataset(32), wrap_cls=(nn.Linear,))
    assert tr.train_engine.num_micro == 2
    st = tr.train()
    assert st.global_step == 12 and st.consumed_train_samples == 96
    losses = [l["loss"] for l in st.log_history if "loss" in l]
    assert losses[-1] < losses[0]
    assert tr.evaluate()["eval_loss"] < 2.0
    assert os.path.exists(tmp_path / "iter_0000012" / ".metadata")
    tr2 = AtorchTrainerV2(a, Net(), train_dataset=dataset(), wrap_cls=(nn.Linear,))
    tr2.train(resume_from_checkpoint=str(tmp_path))
    assert tr2.state.global_step == 12
    for (k, v), (_, v2) in zip(tr.train_engine.module.state_dict().items(),
                               tr2.train_engine.module.state_dict().items()):
        assert torch.equal(v, v2), k


def test_trainer_v2_flow_callback_samples_dynamic_steps_test_and_profiler(tmp_path):
    import json

    from atorch_b200.trainer import AtorchTrainerV2, AtorchTrainingArgs
    from atorch_b200.trainer.trainer_callback import AtorchTrainerCallback, AtorchTrainerState

    dyn = tmp_path / "dyn.json"
    dyn.write_text(json.dumps({"save_at_dynamic_steps": [5]}))
    prof_dir = tmp_path / "prof"
    a = AtorchTrainingArgs(output_dir=str(tmp_path / "out"), bf16=False, micro_batch_size=4, global_batch_size=8,
                           learning_rate=1e-2, max_steps=8, logging_steps=2, logging_first_step=True,
                           save_strategy="samples", save_samples=24, seq_length=1, recompute_granularity=None,
                           async_save=False, dynamic_save_config_path=str(dyn), test_strategy="steps", test_steps=4,
                           profiler_type="nv", profiler_file_path=str(prof_dir), profiler_schedule_wait=1,
                           profiler_schedule_warmup=1, profiler_schedule_active=1)

    class Spy(AtorchTrainerCallback):
        def __init__(self):
            self.saves, self.evals, self.begun = [], [], 0

        def on_save(self, args, state, control, **kw):
            self.saves.append(state.global_step)

        def on_save_begin(self, args, state, control, **kw):
            self.begun += 1

        def on_evaluate(self, args, state, control, metrics=None, **kw):
            self.evals.append((state.global_step, sorted(metrics)))

    spy = Spy()
    tr = AtorchTrainerV2(a, Net(), train_dataset=dataset(), eval_dataset=dataset(32), wrap_cls=(nn.Linear,),
                         callbacks=[spy])
    st = tr.train()
    # 8 samples per step: multiples of 24 consumed samples fall on steps 3 and 6; step 5 comes from the file
    assert spy.saves == [3, 5, 6] and spy.begun == 3
    assert spy.evals == [(4, ["test_loss"]), (8, ["test_loss"])]
    assert [l["step"] for l in st.log_history if "step" in l] == [1, 2, 4, 6, 8]
    assert st.consumed_train_tokens == 64 and st.current_step_in_epoch >= 1
    assert any(f.endswith(".pt.trace.json") for f in os.listdir(prof_dir))
    loaded = AtorchTrainerState.load_from_json(str(tmp_path / "out" / "trainer_state.json"))
    assert loaded.global_step == 6
    js = json.load(open(tmp_path / "out" / "trainer_state.json"))
    js["future_field"] = 1
    json.dump(js, open(tmp_path / "out" / "trainer_state.json", "w"))
    filled = AtorchTrainerState.load_from_json(str(tmp_path / "out" / "trainer_state.json"), AtorchTrainerState())
    assert filled.global_step == 6 and not hasattr(filled, "future_field")


def test_log_warmup_linear_decay_schedule_values():
    """Zero at steps 0 and 1, one at the end of the logarithmic warm-up, linear decay to zero afterwards; the trainer's
    scheduler factory and the standalone one agree; Hugging Face names are passed through."""
    import math

    from atorch_b200.trainer.atorch_trainer import get_scheduler as trainer_sched
    from atorch_b200.utils.trainer_utils import (AtorchSchedulerType, get_linear_schedule_with_log_warmup, get_scheduler,
                                                 log_warmup_linear_decay_factor)

    W, T = 10, 50
    f = [log_warmup_linear_decay_factor(s, W, T) for s in range(T + 5)]
    assert f[0] == 0.0 and abs(f[1]) < 1e-5 and abs(f[5] - math.log(5) / math.log(10)) < 1e-5
    assert f[W] == 1.0 and abs(f[30] - 0.5) < 1e-12 and f[T] == 0.0 and f[T + 3] == 0.0
    p = torch.nn.Parameter(torch.zeros(1))
    lrs = []
    for make in (lambda o: get_linear_schedule_with_log_warmup(o, W, T),
                 lambda o: get_scheduler(AtorchSchedulerType.LOG_WARMUP_LINEAR_DECAY, o, W, T),
                 lambda o: trainer_sched("log_warmup_linear_decay", o, W, T)):
        opt = torch.optim.SGD([p], lr=2.0)
        sch = make(opt)
        seq = []
        for _ in range(T):
            seq.append(opt.param_groups[0]["lr"])
            opt.step()
            sch.step()
        lrs.append(seq)
    assert lrs[0] == lrs[1] == lrs[2] and lrs[0][:W + 1] == [2.0 * x for x in f[:W + 1]]
    opt = torch.optim.SGD([p], lr=1.0)
    cos = get_scheduler("cosine", opt, W, T)
    assert type(cos).__name__ == "LambdaLR"
    with pytest.raises(ValueError):
        get_scheduler("no_such_schedule", opt, W, T)


def _trainer_utils(rank, world):
    from atorch_b200.distributed.distributed import create_parallel_group
    from atorch_b200.trainer.utils import (dict_to_tensor, distributed_std, is_last_rank_on_current_stage,
                                           is_main_process, tensor_to_dict)

    create_parallel_group(([("data", world)], None))
    assert is_main_process() == (rank == 0) and is_last_rank_on_current_stage() == (rank == world - 1)
    payload = {"a": [1, 2, {"b": "x"}], "r": 0}
    t = dict_to_tensor(payload if rank == 0 else {"pad": "y" * 40}, device="cpu")
    n = torch.tensor([t.numel()])
    torch.distributed.broadcast(n, 0)
    buf = t if rank == 0 else torch.empty(int(n), dtype=torch.uint8)
    torch.distributed.broadcast(buf, 0)
    assert tensor_to_dict(buf) == payload
    torch.manual_seed(3)
    full = torch.randn(world * 6, 5)
    piece = full.chunk(world)[rank].clone()                 # this rank's shard of a sharded parameter
    assert torch.allclose(distributed_std("w", piece), full.std(), rtol=1e-5)


def test_trainer_utils_roles_object_transport_and_sharded_std_gloo():
    from tests.dist_utils import run_distributed

    run_distributed(_trainer_utils, world=2)


def test_trainer_utils_tensorboard_writer_and_banner(caplog):
    import logging

    from atorch_b200.trainer.utils import (DistributedType, IntervalStrategy, print_all_args_before_training,
                                           write_dict_to_tensorboard)

    class W:
        def __init__(self):
            self.rows = []

        def add_scalar(self, k, v, i):
            self.rows.append((k, v, i))

        def log(self, d, i):
            self.rows.append((d, i))

    tb, wb = W(), W()
    write_dict_to_tensorboard(tb, wb, 7, {"loss": 1.5, "grad": {"norm": 2.0, "layers": {"l0": 0.1}}}, prefix="train/")
    assert tb.rows == [("train/loss", 1.5, 7), ("train/grad/norm", 2.0, 7), ("train/grad/layers/l0", 0.1, 7)]
    assert wb.rows[1] == ({"train/grad/norm": 2.0}, 7)
    assert IntervalStrategy("steps") is IntervalStrategy.STEPS and DistributedType.FSDP.value == "FSDP"
    with caplog.at_level(logging.INFO, logger="atorch.logger"):
        print_all_args_before_training({"Train": {"lr": 0.1, "Batch": 4}})
    lines = [r.getMessage() for r in caplog.records]
    assert any(l.startswith("  Batch ****") and l.endswith(" 4") for l in lines)
    assert lines.index(next(l for l in lines if l.startswith("  Batch"))) < lines.index(next(l for l in lines if l.startswith("  lr")))
