"""Masked-LM accuracy, per batch and accumulated over a data set (optionally reduced to rank 0).
(Reference: atorch/utils/metric_util.py:6-60.)"""
import torch
import torch.distributed as dist


def _hits_and_count(outputs, masked_lm_labels):
    logits = outputs.logits if hasattr(outputs, "logits") else outputs["logits"]
    labels = masked_lm_labels.reshape(-1)
    keep = labels != -100
    pred = logits.reshape(-1, logits.shape[-1])[keep].argmax(-1)
    return (pred == labels[keep]).sum(dtype=torch.float), int(keep.sum())


def calc_mlm_acc(outputs, masked_lm_labels) -> torch.Tensor:
    """Fraction of the labelled (``!= -100``) positions whose arg-max prediction is right."""
    hits, n = _hits_and_count(outputs, masked_lm_labels)
    return hits / n


class MaskedLM:
    """``record(outputs, labels)`` every step, ``compute()`` at the end (rank 0 holds the global value when
    ``is_distributed``)."""

    def __init__(self, is_distributed: bool = False):
        device = f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu"
        self.correct_num = torch.tensor(0.0, device=device)
        self.total_num = torch.tensor(0, device=device)
        self.is_distributed = is_distributed

    def record(self, outputs, masked_lm_labels) -> None:
        hits, n = _hits_and_count(outputs, masked_lm_labels)
        self.correct_num += hits.to(self.correct_num.device)
        self.total_num += n

    def compute(self) -> torch.Tensor:
        if self.is_distributed:
            dist.reduce(self.correct_num, 0)
            dist.reduce(self.total_num, 0)
        return self.correct_num / self.total_num
