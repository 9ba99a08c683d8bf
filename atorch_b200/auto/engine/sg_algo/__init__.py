"""Strategy-generation algorithms of the acceleration engine. An algorithm is called with the executor whenever the
executor has run out of candidates; it appends new candidates to the executor and answers
``(is_done, tasks, new_strategy_num)``. It may be called many times (one stage per call).

``CombinationAlgorithm`` ("combination_sg")  all combinations of {none, zero2, fsdp} x {none, amp, module_replace + amp}
    on top of data parallelism over all processes, in one call.
``BOAlgorithm`` ("bo_sg")  Bayesian optimisation over one categorical variable per method group: every call feeds
    the throughputs measured since the last call to a Gaussian-process model and proposes the untried combination
    with the largest expected improvement; done when the space, the iteration limit or the patience is exhausted.
``StrategyGenerationAlgorithmLibrary``  the algorithms by name (``None`` for an unknown name).
(Reference: atorch/auto/engine/sg_algo/{sg_algorithm.py:1-26, combination_sg.py:16-60, bayes_opt_sg.py:35-161,
sg_algo_lib.py:11-33}.)
"""
from __future__ import annotations

from typing import Optional, Tuple


class StrategyGenerationAlgorithm:
    def __init__(self, name: Optional[str] = None):
        self.name, self.is_done = name, False

    def strategy_generate(self, executor) -> Tuple[bool, Optional[list], int]:
        self.is_done = True
        return True, None, 0

    def __call__(self, executor):
        return self.strategy_generate(executor)


def _known(executor) -> set:
    keys = {tuple(r.strategy.names()) for r in executor.strategies}
    keys |= {tuple(r.strategy.names()) for r in (executor._candidates or ())}
    return keys


class CombinationAlgorithm(StrategyGenerationAlgorithm):
    def __init__(self):
        super().__init__("combination_sg")
        self.new_strategy_num = 0

    def strategy_generate(self, executor):
        from ..executor import StrategyRecord
        from ..search import combination_candidates

        if self.is_done:
            return True, None, 0
        seen, self.new_strategy_num = _known(executor), 0
        for st in combination_candidates(executor.total_process, executor.analysis, executor.excluded,
                                         executor.included):
            key = tuple(st.names())
            if key not in seen:
                seen.add(key)
                executor._candidates.append(StrategyRecord(st))
                self.new_strategy_num += 1
        self.is_done = True
        return True, None, self.new_strategy_num


class BOAlgorithm(StrategyGenerationAlgorithm):
    def __init__(self, max_iter: int = 30, patience: int = 8, random_sample: int = 3, seed: int = 0):
        from ..search import BayesianGenerator

        super().__init__("bo_sg")
        self.model = BayesianGenerator(max_iter, patience, random_sample, seed)
        self._observed = set()

    def strategy_generate(self, executor):
        from ..executor import StrategyRecord

        if self.is_done:
            return True, None, 0
        for rec in executor.strategies:                # results that arrived since the last call
            if rec.combo is not None and rec.combo not in self._observed and \
                    rec.status in (StrategyRecord.SUCCEED, StrategyRecord.FAILED):
                self._observed.add(rec.combo)
                self.model.observe(rec.combo, rec.throughput)
        combo = self.model.suggest()
        if combo is None:
            self.is_done = True
            return True, None, 0
        self.model.tried.add(combo)                    # proposed: not to be proposed again while it runs
        executor._candidates.append(StrategyRecord(self.model.to_strategy(combo, executor.total_process,
                                                                          executor.analysis), combo))
        return False, None, 1


class StrategyGenerationAlgorithmLibrary:
    def __init__(self):
        self.algorithms = {}
        self.add_algorithms()

    def add_algorithms(self) -> None:
        for algo in (CombinationAlgorithm(), BOAlgorithm()):
            self.algorithms[algo.name] = algo

    def __getitem__(self, name):
        return self.algorithms.get(name)
