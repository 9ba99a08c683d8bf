"""Model and statistics helpers of the RLHF trainer: dotted attribute lookup (to find decoder blocks, heads and
norms across Hugging Face architectures), value heads, layer freezing, cross-rank moments, whitening, masked tensor
statistics, running moments for reward scaling and the fixed KL coefficient.
(Reference: atorch/rl/model_utils/model_util.py:14-341.)
"""
from __future__ import annotations

import functools
import random
from collections.abc import MutableMapping
from typing import Iterable, Tuple

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from .ppo_utils import logprobs_of_labels  # noqa: F401  (same definition, exported under this path too)


def set_seed(seed: int) -> None:
    """Rank-dependent seeds for python, numpy and torch (``seed + rank``)."""
    seed += dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def make_head(n_embd: int, out: int, dtype: torch.dtype = torch.float32) -> nn.Sequential:
    """Two-layer MLP head (``n_embd -> 2 n_embd -> out``, ReLU) used as the value head."""
    return nn.Sequential(nn.Linear(n_embd, n_embd * 2, dtype=dtype), nn.ReLU(), nn.Linear(n_embd * 2, out, dtype=dtype))


def rhasattr(obj, attr: str) -> bool:
    """``hasattr`` for a dotted path such as ``"model.decoder.layers"``."""
    for name in attr.split("."):
        if not hasattr(obj, name):
            return False
        obj = getattr(obj, name)
    return True


def rgetattr(obj, attr: str, *default):
    """``getattr`` for a dotted path; an optional default applies at every step."""
    return functools.reduce(lambda o, name: getattr(o, name, *default), attr.split("."), obj)


def findattr(obj, attrs: Iterable[str]):
    """The first of the dotted paths that exists."""
    for attr in attrs:
        if rhasattr(obj, attr):
            return rgetattr(obj, attr)
    raise ValueError(f"Could not find an attribute from `{attrs}` in `{obj}`")


_DECODER_PATHS = ("transformer", "model.decoder", "gpt_neox", "decoder", "glm.transformer", "model")
_FINAL_NORM_PATHS = ("transformer.ln_f", "model.decoder.final_layer_norm", "model.norm", "decoder.final_layer_norm",
                     "gpt_neox.final_layer_norm", "glm.transformer.final_layernorm")
_BLOCK_PATHS = ("transformer.h", "model.decoder.layers", "gpt_neox.layers", "decoder.block", "model.layers",
                "glm.transformer.layers", "layers", "h")
_LM_HEAD_PATHS = ("lm_head", "embed_out", "output_layer")
_HIDDEN_SIZE_NAMES = ("hidden_size", "n_embd", "d_model")
_NUM_LAYER_NAMES = ("num_hidden_layers", "n_layer", "num_layers")


def hf_get_decoder(model: nn.Module) -> nn.Module:
    return findattr(model, _DECODER_PATHS)


def hf_get_decoder_final_norm(model: nn.Module) -> nn.Module:
    return findattr(model, _FINAL_NORM_PATHS)


def hf_get_decoder_blocks(model: nn.Module):
    return findattr(model, _BLOCK_PATHS)


def hf_get_glm_embeddings(model: nn.Module):
    return findattr(model, ("glm.word_embeddings", "word_embeddings", "model.embed_tokens", "transformer.wte"))


def hf_get_lm_head(model: nn.Module) -> nn.Module:
    return findattr(model, _LM_HEAD_PATHS)


def hf_get_hidden_size(config) -> int:
    return findattr(config, _HIDDEN_SIZE_NAMES)


def hf_get_num_hidden_layers(config) -> int:
    return findattr(config, _NUM_LAYER_NAMES)


def freeze_bottom_causal_layers(model: nn.Module, num_layers_unfrozen: int = 0) -> None:
    """Freezes all decoder blocks but the last ``num_layers_unfrozen`` (0: all of them; negative: none)."""
    blocks = list(hf_get_decoder_blocks(model))
    if num_layers_unfrozen == 0:
        frozen = blocks
    elif num_layers_unfrozen > 0:
        frozen = blocks[:-num_layers_unfrozen]
    else:
        frozen = []
    for b in frozen:
        b.requires_grad_(False)


def get_global_statistics(xs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(mean, biased variance, count) of all elements over all ranks: two small all-reduces."""
    sum_count = torch.tensor([xs.sum(), xs.numel()], device=xs.device)
    dist.all_reduce(sum_count)
    total, count = sum_count
    mean = total / count
    sq = torch.sum((xs - mean) ** 2)
    dist.all_reduce(sq)
    return mean, sq / count, count


def whiten(xs: torch.Tensor, shift_mean: bool = True, distributed: bool = True) -> torch.Tensor:
    """Zero mean (unless ``shift_mean`` is off) and unit variance; with a process group the moments are global
    (biased variance), otherwise local (unbiased, as ``torch.var_mean`` gives it)."""
    if distributed and dist.is_available() and dist.is_initialized():
        mean, var, _ = get_global_statistics(xs)
    else:
        var, mean = torch.var_mean(xs)
    out = (xs - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


def flatten_dict(d: MutableMapping, parent_key: str = "", sep: str = "/") -> dict:
    """``{"a": {"b": 1}} -> {"a/b": 1}``."""
    flat = {}
    for k, v in d.items():
        key = parent_key + sep + k if parent_key else k
        if isinstance(v, MutableMapping):
            flat.update(flatten_dict(v, key, sep))
        else:
            flat[key] = v
    return flat


def get_tensor_stats(xs: torch.Tensor, mask: torch.Tensor, n) -> dict:
    """mean / min / max / std of the masked entries (``n`` = number of them)."""
    keep = mask.bool()
    mean = (xs * mask).sum() / n
    inf = torch.tensor(float("inf"), dtype=xs.dtype, device=xs.device)
    return dict(mean=mean.item(), min=torch.where(keep, xs, inf).min().item(),
                max=torch.where(keep, xs, -inf).max().item(),
                std=torch.sqrt(((xs - mean) * mask).pow(2).sum() / n).item())


class RunningMoments:
    """Mean / variance of a stream of batches by the parallel-variance update; ``update`` returns the batch's own
    (mean, unbiased std). With a process group the batch moments are global."""

    def __init__(self):
        self.mean, self.std, self.var, self.count = 0, 1, 1, 1e-24

    def update(self, xs: torch.Tensor):
        if dist.is_available() and dist.is_initialized():
            b_mean, b_var, b_count = get_global_statistics(xs)
        else:
            b_count = xs.numel()
            b_var, b_mean = torch.var_mean(xs, unbiased=False)
        delta = b_mean - self.mean
        total = self.count + b_count
        m2 = self.var * self.count + delta ** 2 * self.count * b_count / total + b_var * b_count
        self.mean += delta * b_count / total
        self.var = m2 / total
        self.std = (self.var * total / (total - 1)).sqrt()
        self.count = total
        return b_mean, (b_var * b_count / (b_count - 1)).sqrt()


class FixedKLController:
    """A KL coefficient that never changes (``update`` is a no-op)."""

    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current: float, n_steps: int) -> None:
        return None


def is_trainable_model(model_name: str) -> bool:
    return "actor" in model_name or "critic" in model_name
