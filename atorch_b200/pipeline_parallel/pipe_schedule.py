"""Pipeline schedules executed over NCCL p2p: GPipe, 1F1B and interleaved 1F1B.

A schedule is first written down as an explicit per-rank list of actions
``(kind, stage_index, micro_batch)`` with kind in {F, B} (pure function, unit-tested without any
process group), then executed: before every F the stage receives its activations (first stage:
takes the micro-batch from the input), after it sends its outputs; B mirrors that with gradients.
Sends are asynchronous (their handles are drained at the end of the step), so a stage goes on computing
while its output is on the wire; a receive is posted when its action starts and waited for at once —
receives are not posted ahead, because NCCL runs the point-to-point operations of one communicator in
stream order and two neighbours that both queue a receive before their send would wait on each other.

``schedule.step(*inputs, target=..., losses=[...], **batch_kwargs)``: inputs/kwargs are split into
``n_microbatches`` along dim 0 on the first stage; ``target`` is consumed by the last stage as
``loss_fn(output, target_mb)``. Returns the mean loss on the last stage, else None.
(Reference: atorch/pipeline_parallel/pipe_schedule.py:19-55 selects torch.distributed.pipelining
schedules; scheduler stubs at atorch/pipeline_parallel/scheduler.py:203-331.)
"""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .pipe_stage import PipeStage, _as_tuple


class PipeSchedulerType(Enum):
    ScheduleGPipe = "ScheduleGPipe"
    Schedule1F1B = "Schedule1F1B"
    ScheduleInterleaved1F1B = "ScheduleInterleaved1F1B"
    ScheduleZeroBubble = "ScheduleZeroBubble"


def gpipe_actions(pp_rank: int, pp_size: int, n_mb: int) -> List[Tuple[str, int, int]]:
    return [("F", 0, m) for m in range(n_mb)] + [("B", 0, m) for m in range(n_mb)]


def one_f_one_b_actions(pp_rank: int, pp_size: int, n_mb: int) -> List[Tuple[str, int, int]]:
    """Warm-up of ``pp_size - rank - 1`` forwards, steady one-forward-one-backward, cool-down."""
    warm = min(pp_size - pp_rank - 1, n_mb)
    acts = [("F", 0, m) for m in range(warm)]
    f, b = warm, 0
    while f < n_mb:
        acts.append(("F", 0, f))
        f += 1
        acts.append(("B", 0, b))
        b += 1
    while b < n_mb:
        acts.append(("B", 0, b))
        b += 1
    return acts


def interleaved_actions(pp_rank: int, pp_size: int, n_mb: int, n_local: int) -> List[Tuple[str, int, int]]:
    """Interleaved 1F1B (Megatron order): micro-batches advance in groups of ``pp_size`` through
    the local stages; requires ``n_mb % pp_size == 0``."""
    assert n_mb % pp_size == 0, "interleaved schedule needs n_microbatches divisible by the pipeline size"
    total = n_mb * n_local

    def fwd_item(k):
        group, within = divmod(k, pp_size * n_local)
        chunk, pos = divmod(within, pp_size)
        return chunk, group * pp_size + pos

    def bwd_item(k):
        chunk, mb = fwd_item(k)
        return n_local - 1 - chunk, mb
    warm = min((pp_size - pp_rank - 1) * 2 + (n_local - 1) * pp_size, total)
    acts = [("F",) + fwd_item(k) for k in range(warm)]
    f, b = warm, 0
    while f < total:
        acts.append(("F",) + fwd_item(f))
        f += 1
        acts.append(("B",) + bwd_item(b))
        b += 1
    while b < total:
        acts.append(("B",) + bwd_item(b))
        b += 1
    return acts


class PipelineSchedule:
    def __init__(self, stages: Sequence[PipeStage], n_microbatches: int, loss_fn: Optional[Callable], kind: str,
                 pp_rank: int, pp_size: int):
        self.stages = list(stages)
        self.n_mb, self.loss_fn, self.kind = n_microbatches, loss_fn, kind
        self.pp_rank, self.pp_size = pp_rank, pp_size
        if kind == "ScheduleGPipe":
            self.actions = gpipe_actions(pp_rank, pp_size, n_microbatches)
        elif kind == "Schedule1F1B":
            assert len(self.stages) == 1
            self.actions = one_f_one_b_actions(pp_rank, pp_size, n_microbatches)
        else:
            self.actions = interleaved_actions(pp_rank, pp_size, n_microbatches, len(self.stages))

    @staticmethod
    def _split(x, n):
        if isinstance(x, torch.Tensor):
            return list(x.chunk(n, dim=0))
        return [x] * n

    def step(self, *inputs, target=None, losses: Optional[list] = None, **batch_kwargs):
        n = self.n_mb
        in_mbs = [tuple(self._split(a, n)[m] for a in inputs) for m in range(n)] if inputs else [()] * n
        kw_mbs = [{k: self._split(v, n)[m] for k, v in batch_kwargs.items()} for m in range(n)]
        tgt_mbs = self._split(target, n) if target is not None else [None] * n
        pending, loss_vals = [], []
        mb_loss: Dict[Tuple[int, int], torch.Tensor] = {}
        b_counts = {i: 0 for i in range(len(self.stages))}
        for kind, si, mb in self.actions:
            st = self.stages[si]
            if kind == "F":
                if st.is_first:
                    acts = in_mbs[mb]
                elif st.prev_rank == st.my_rank:      # previous stage lives on this rank (single-rank pipelines)
                    acts = self._local_handoff.pop((st.stage_id, mb))
                else:
                    acts = st.comm.recv_wait(st.prev_rank, meta_id=("f", st.stage_id), slot=mb % 2)
                    acts = [a.clone() for a in acts]
                batch = kw_mbs[mb] if kw_mbs[mb] else None
                out = st.forward_one_chunk(mb, acts, batch)
                if st.is_last:
                    if self.loss_fn is not None:
                        o = out[0] if isinstance(out, (tuple, list)) and len(out) == 1 else out
                        loss = self.loss_fn(o, tgt_mbs[mb]) if tgt_mbs[mb] is not None else self.loss_fn(o)
                        mb_loss[(si, mb)] = loss / n
                        loss_vals.append(loss.detach())
                else:
                    outs = [o.detach() for o in _as_tuple(out)]
                    if st.next_rank == st.my_rank:
                        if not hasattr(self, "_local_handoff"):
                            self._local_handoff = {}
                        self._local_handoff[(st.stage_id + 1, mb)] = outs
                    else:
                        pending += st.comm.send(outs, st.next_rank, meta_id=("f", st.stage_id + 1))
            else:
                b_counts[si] += 1
                last_mb = b_counts[si] == n
                if st.is_last:
                    grads = st.backward_one_chunk(mb, mb_loss.pop((si, mb), None), None, last_mb)
                else:
                    if st.next_rank == st.my_rank:
                        og = self._local_grad.pop((st.stage_id, mb))
                    else:
                        og = st.comm.recv_wait(st.next_rank, meta_id=("b", st.stage_id), slot=mb % 2)
                        og = [g.clone() for g in og]
                    grads = st.backward_one_chunk(mb, None, og, last_mb)
                if not st.is_first and grads:
                    if st.prev_rank == st.my_rank:
                        if not hasattr(self, "_local_grad"):
                            self._local_grad = {}
                        self._local_grad[(st.stage_id - 1, mb)] = grads
                    else:
                        pending += st.comm.send(grads, st.prev_rank, meta_id=("b", st.stage_id - 1))
        for w in pending:
            w.wait()
        if losses is not None:
            losses.extend(loss_vals)
        return torch.stack(loss_vals).mean() if loss_vals else None


def make_pipe_schedule_from_pipe_module(pipe_module, config=None):
    kind = PipeSchedulerType(config.sche_name).value
    if kind == "ScheduleZeroBubble":
        kind = "ScheduleInterleaved1F1B"    # same dependency order; weight-gradient splitting is not separated here
    if kind == "Schedule1F1B" and len(pipe_module.stages) > 1:
        kind = "ScheduleInterleaved1F1B"
    return PipelineSchedule(pipe_module.stages, config.n_microbatches,
                            pipe_module.loss_func if pipe_module.loss_func is not None else pipe_module.ori_loss_func,
                            kind, pipe_module.pp_rank, pipe_module.pp_size)


def make_pipe_schedule(meta_model=None, model_provider=None, loss_func=None, strategy=None, distributed_context=None,
                       config=None):
    from .pipe_module import make_pipe_module

    pm = make_pipe_module(meta_model, model_provider, loss_func, strategy, distributed_context, config)
    return make_pipe_schedule_from_pipe_module(pm, config)
