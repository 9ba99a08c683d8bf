"""Fully automatic strategy search (``auto_accelerate`` without ``load_strategy``).

Stages, as in the reference's planner/executor (atorch/auto/engine/planner.py:6-120, executor.py:36,
strategy.py:49-171, sg_algo/combination_sg.py:16-60, sg_algo/bayes_opt_sg.py:35-161):
  1. prune methods the job cannot use (single process -> no distributed methods; CPU -> no fp8 ...)
  2. analyse the model (:mod:`atorch_b200.auto.analyser`)
  3. generate candidates: the combination generator {none, zero2, fsdp} x {none, amp_native,
     module_replace + amp_native} (+ checkpoint when memory is the problem) on top of
     ``parallel_mode(data = world)``; a Bayesian generator (scikit-learn Gaussian process with
     expected improvement over the categorical method groups) proposes further candidates when the
     space is enlarged with ``included`` methods
  4. dry-run each candidate (rank 0 decides, the decision is broadcast so all ranks build the same
     strategies in the same order) and return the one with the best throughput.
``search_strategy`` runs the loop in-process; ``search_strategy_with_service`` runs it as the reference
does: rank 0 hosts the engine (:mod:`atorch_b200.auto.engine.service`, task queue in
:mod:`atorch_b200.auto.engine.executor`) and every rank asks it for tasks over gRPC.
"""
from __future__ import annotations

import random
import itertools
import logging
import time
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ...distributed import distributed as D
from ..analyser import analyse_model
from ..dry_runner import dry_run_strategy
from ..strategy import Strategy

logger = logging.getLogger("atorch.logger")


class StrategyStatus:
    INIT, TUNED, SUCCEED, FAILED = "init", "tuned", "succeed", "failed"


class StrategyInfo:
    def __init__(self, strategy: Strategy):
        self.strategy, self.status, self.dryrun_result = strategy, StrategyStatus.INIT, None

    @property
    def throughput(self) -> float:
        return (self.dryrun_result or {}).get("throughput", 0.0)


def combination_candidates(world: int, analysis: dict, excluded=None, included=None) -> List[Strategy]:
    excluded = set(excluded or [])
    block = analysis.get("opt_config_submodule_names") or ()
    zero_cfg = {"atorch_wrap_cls": tuple(block)} if block else {}
    zero_opts = [None, ("zero2", dict(zero_cfg)), ("fsdp", dict(zero_cfg, forward_prefetch=True,
                                                                limit_all_gathers=True))]
    amp = ("amp_native", {"dtype": torch.bfloat16})
    amp_opts: List[Optional[list]] = [None, [amp]]
    if analysis.get("replaceable_pairs"):
        amp_opts.append([("module_replace", None), amp])
    out = []
    for z, a in itertools.product(zero_opts, amp_opts):
        items = [("parallel_mode", ([("data", world)], None))]
        if a:
            items += a
        if z:
            items.append(z)
        names = {i[0] for i in items}
        if names & excluded:
            continue
        out.append(Strategy([(n, c, False) for n, c in items]))
        for extra in (included or []):
            if extra == "checkpoint" and block and "checkpoint" not in excluded:
                out.append(Strategy([(n, c, False) for n, c in items] + [("checkpoint", {"wrap_class": tuple(block)},
                                                                         False)]))
    return out


class BayesianGenerator:
    """Gaussian-process search over categorical method groups (amp, zero, checkpoint, module_replace).
    Observations are (one-hot choice vector, throughput); the next candidate maximises expected
    improvement among the untried combinations. Falls back to plain enumeration without scikit-learn."""

    GROUPS = {"amp": [None, "amp_native"], "zero": [None, "zero2", "fsdp"], "ckpt": [None, "checkpoint"],
              "replace": [None, "module_replace"]}

    def __init__(self, max_iter: int = 30, patience: int = 8, random_sample: int = 3, seed: int = 0):
        self.max_iter, self.patience, self.random_sample = max_iter, patience, random_sample
        self.space = list(itertools.product(*self.GROUPS.values()))
        self.X, self.y, self.tried = [], [], set()
        self.rng = random.Random(seed)

    def _encode(self, combo):
        v = []
        for choice, options in zip(combo, self.GROUPS.values()):
            v += [1.0 if choice == o else 0.0 for o in options]
        return v

    def observe(self, combo, throughput: float):
        self.X.append(self._encode(combo))
        self.y.append(throughput)
        self.tried.add(combo)

    def suggest(self):
        rest = [c for c in self.space if c not in self.tried]
        if not rest or len(self.tried) >= self.max_iter:
            return None
        if len(self.y) < self.random_sample:
            return self.rng.choice(rest)
        best = max(self.y)
        if len(self.y) - self.y.index(best) > self.patience:
            return None
        try:
            import numpy as np
            from scipy.stats import norm
            from sklearn.gaussian_process import GaussianProcessRegressor
            from sklearn.gaussian_process.kernels import Matern

            gp = GaussianProcessRegressor(Matern(nu=2.5), normalize_y=True, alpha=1e-6).fit(np.array(self.X),
                                                                                            np.array(self.y))
            mu, sd = gp.predict(np.array([self._encode(c) for c in rest]), return_std=True)
            z = (mu - best) / np.maximum(sd, 1e-9)
            ei = (mu - best) * norm.cdf(z) + sd * norm.pdf(z)
            return rest[int(np.argmax(ei))]
        except Exception:
            return rest[0]

    def to_strategy(self, combo, world: int, analysis: dict) -> Strategy:
        amp, zero, ckpt, rep = combo
        block = tuple(analysis.get("opt_config_submodule_names") or ())
        items = [("parallel_mode", ([("data", world)], None))]
        if rep:
            items.append(("module_replace", None))
        if amp:
            items.append(("amp_native", {"dtype": torch.bfloat16}))
        if zero:
            items.append((zero, {"atorch_wrap_cls": block} if block else {}))
        if ckpt and block:
            items.append(("checkpoint", {"wrap_class": block}))
        return Strategy([(n, c, False) for n, c in items])


def _agree(value: float) -> float:
    """All ranks adopt the slowest rank's throughput so that they rank candidates identically."""
    if D.is_distributed():
        dev = "cuda" if (torch.cuda.is_available() and "nccl" in (D.backend() or "")) else "cpu"
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())
    return value


def search_strategy(mc, opt_lib, excluded=None, included=None, time_limit: Optional[float] = None,
                    verbose: bool = False, algo: str = "combination") -> Tuple[bool, Optional[Strategy]]:
    world = D.world_size() or 1
    analysis = analyse_model(mc.model)
    start = time.time()
    infos: List[StrategyInfo] = []
    cap = torch.cuda.get_device_capability() if torch.cuda.is_available() else None

    def evaluate(st: Strategy):
        if not D.is_distributed():
            st.remove_distributed_method(opt_lib)
        st.remove_device_unsupported_method(opt_lib, cap)
        info = StrategyInfo(st)
        res = dry_run_strategy(mc, st, opt_lib)
        res["throughput"] = _agree(res.get("throughput", 0.0))
        info.dryrun_result = res
        info.status = StrategyStatus.SUCCEED if res["throughput"] > 0 else StrategyStatus.FAILED
        infos.append(info)
        if verbose:
            logger.info("candidate %s -> %.2f samples/s", st.names(), res["throughput"])
        return res["throughput"]

    if algo == "bo":
        gen = BayesianGenerator()
        while True:
            combo = gen.suggest()
            if combo is None or (time_limit and time.time() - start > time_limit):
                break
            gen.observe(combo, evaluate(gen.to_strategy(combo, world, analysis)))
    else:
        seen = set()
        for st in combination_candidates(world, analysis, excluded, included):
            key = tuple(st.names())
            if key in seen:
                continue
            seen.add(key)
            if time_limit and time.time() - start > time_limit:
                break
            evaluate(st)
    ok = [i for i in infos if i.status == StrategyStatus.SUCCEED]
    if not ok:
        return False, None
    best = max(ok, key=lambda i: i.throughput)
    return True, best.strategy


def search_strategy_with_service(mc, opt_lib, excluded=None, included=None, time_limit: Optional[float] = None,
                                 verbose: bool = False, algo: str = "combination") -> Tuple[bool, Optional[Strategy]]:
    """Rank 0 starts the acceleration engine; all ranks (rank 0 too) loop get_task -> run -> report until the
    engine hands out FINISH (best strategy) or FAIL."""
    from ..accelerate import tune_strategy
    from ..opt_lib.parallel_mode import ParallelModeOptimization
    from .service import AccelerationEngine, AutoAccelerationClient, run_worker_loop
    from .task import TaskType

    world, rank = D.world_size() or 1, D.rank() or 0
    engine, port = None, [0]
    if rank == 0:
        ctx = {"node_num": 1, "nproc_per_node": world}
        engine = AccelerationEngine(ctx, included_opts=included, excluded_opts=excluded, time_limit=time_limit,
                                    verbose=verbose, algo=algo)
        port[0] = engine.start_service(0)
    if D.is_distributed():
        dist.broadcast_object_list(port, src=0)
    import os

    client = AutoAccelerationClient(f"{os.environ.get('MASTER_ADDR', '127.0.0.1') if rank else '127.0.0.1'}:{port[0]}",
                                    rank)
    cap = torch.cuda.get_device_capability() if torch.cuda.is_available() else None

    def run_task(task):
        if task.task_type == TaskType.ANALYSE:
            return True, analyse_model(mc.model)
        if task.task_type == TaskType.SETUP_PARALLEL_GROUP:
            if D.is_distributed():
                ParallelModeOptimization.setup_groups(task.task_info)
            return True, None
        st: Strategy = task.task_info
        if not D.is_distributed():
            st.remove_distributed_method(opt_lib)
        st.remove_device_unsupported_method(opt_lib, cap)
        if task.task_type == TaskType.TUNE:
            return bool(tune_strategy(mc, st, opt_lib, time_limit)), st
        res = dry_run_strategy(mc, st, opt_lib) or {}
        res["throughput"] = _agree(res.get("throughput", 0.0))
        if verbose:
            logger.info("candidate %s -> %.2f samples/s", st.names(), res["throughput"])
        return res["throughput"] > 0, res
    try:
        best = run_worker_loop(client, run_task)
    finally:
        client.close()
        if engine is not None:
            engine.tear_down(timeout=30.0)
    return best is not None, best
