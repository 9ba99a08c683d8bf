"""Online EWMA outlier test used to drop a replica's pseudo-gradient when its norm spikes.

    mean += a (x - mean);  M2 = (1 - a)(M2 + a (x - mean_old)(x - mean_new));  z = (x - mean)/sqrt(M2)
An observation is an outlier iff ``z > base_threshold * max(1, std(recent z))`` once ``warmup_steps``
observations were seen (z counts as 0 before that).
(Reference: atorch/local_sgd/utils/anomaly_detection.py:7-91.)
"""
from __future__ import annotations

import math
from collections import deque
from typing import Any, Dict


class OnlineDynamicEWMA:
    def __init__(self, alpha: float = 0.02, warmup_steps: int = 100, base_threshold: float = 3):
        self.alpha, self.warmup_steps, self.base_threshold = alpha, warmup_steps, base_threshold
        self.mean = 0.0
        self.M2 = 0.0
        self.count = 0
        self.z_scores_window: deque = deque(maxlen=warmup_steps)

    @staticmethod
    def _f(x) -> float:
        return float(x.item()) if hasattr(x, "item") else float(x)

    def get_std(self) -> float:
        return math.sqrt(self.M2) if self.count >= 2 else 0.0

    def get_mean(self) -> float:
        return self.mean

    def get_z_score(self, value) -> float:
        std = self.get_std()
        if std == 0.0 or self.count < self.warmup_steps:
            return 0.0
        return (self._f(value) - self.mean) / std

    def update(self, value) -> None:
        x = self._f(value)
        self.count += 1
        d = x - self.mean
        self.mean += self.alpha * d
        d2 = x - self.mean
        self.M2 = (1 - self.alpha) * (self.M2 + self.alpha * d * d2)
        self.z_scores_window.append(self.get_z_score(x))

    def dynamic_threshold_factor(self) -> float:
        if self.count < self.warmup_steps or len(self.z_scores_window) < 2:
            return 1.0
        zs = list(self.z_scores_window)
        m = sum(zs) / len(zs)
        var = sum((z - m) ** 2 for z in zs) / (len(zs) - 1)
        return max(1.0, math.sqrt(var))

    def is_outlier(self, value) -> bool:
        if self.count < self.warmup_steps:
            return False
        return self.get_z_score(value) > self.base_threshold * self.dynamic_threshold_factor()

    def state_dict(self) -> Dict[str, Any]:
        return {"mean": self.mean, "M2": self.M2, "count": self.count, "warmup_steps": self.warmup_steps,
                "z_scores_window": list(self.z_scores_window)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.mean = self._f(sd.get("mean", self.mean))
        self.M2 = self._f(sd.get("M2", self.M2))
        self.count = int(sd.get("count", self.count))
        self.warmup_steps = int(sd.get("warmup_steps", self.warmup_steps))
        self.z_scores_window = deque((self._f(z) for z in sd.get("z_scores_window", [])), maxlen=self.warmup_steps)
