"""Manual tensor-parallel sharding by module-name suffix.

    info = TPInfo()
    info.shard_col({"attn.c_attn": {"stride": 3}}, "mlp.c_fc")      # column-parallel (output split)
    info.shard_row("attn.c_proj", "mlp.c_proj")                     # row-parallel (input split)
    info.shard_vocab("wte")                                         # vocabulary-parallel embedding
    info.replic_drop("resid_dropout"); info.parallel_drop("attn_dropout")
    info.shrink({".attn": {"embed_dim", "num_heads"}})              # divide these attributes by tp size
    model = tp_manual_shard(model, info)                            # replaces the modules in place

(Reference: atorch/tensor_parallel/manual_tp.py:107-255. There the sharding is attached to a
meta-initialised model as deferred build functions; here ``tp_manual_shard`` replaces modules
directly and ``tp_manual_shard_custom_fn`` keeps the deferred form for meta models.)
"""
from __future__ import annotations

from typing import Dict

import torch.nn as nn

from ..distributed import distributed as D
from ..modules.distributed_modules.layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
from ..parallel.randomizer import get_randomizer


class TPInfo:
    def __init__(self):
        self.Shard: Dict = {ColumnParallelLinear: {}, RowParallelLinear: {}, VocabParallelEmbedding: {}}
        self.Drop = {("tensor",): set(), tuple(): set()}
        self.Shrink: Dict = {}

    @staticmethod
    def parse_args(*args) -> dict:
        ret = {}
        for a in args:
            if isinstance(a, str):
                ret[a] = {}
            elif isinstance(a, dict):
                ret.update(a)
            else:
                raise ValueError(f"Arg {a} is not str or dict.")
        return ret

    def shard_col(self, *args):
        self.Shard[ColumnParallelLinear].update(self.parse_args(*args))

    def shard_row(self, *args):
        self.Shard[RowParallelLinear].update(self.parse_args(*args))

    def shard_vocab(self, *args):
        self.Shard[VocabParallelEmbedding].update(self.parse_args(*args))

    def replic_drop(self, *args):
        assert all(isinstance(a, str) for a in args)
        self.Drop[("tensor",)].update(args)

    def parallel_drop(self, *args):
        assert all(isinstance(a, str) for a in args)
        self.Drop[tuple()].update(args)

    def shrink(self, *args):
        self.Shrink.update(self.parse_args(*args))

    def is_vocab_parallelled(self) -> bool:
        return len(self.Shard[VocabParallelEmbedding]) > 0


class _RandomizedDropout(nn.Module):
    """Dropout whose mask is drawn from a named RNG stream: the same on all ranks of ``same_groups``
    (replicated activations) or different per rank (sharded activations)."""

    def __init__(self, inner: nn.Module, same_groups):
        super().__init__()
        self.inner, self.same_groups = inner, tuple(same_groups)

    def forward(self, x):
        with get_randomizer(*self.same_groups).fork():
            return self.inner(x)


def _as_linear(m: nn.Module):
    """``nn.Linear`` view of HF ``Conv1D`` (weight stored transposed) or the module itself."""
    if type(m).__name__ == "Conv1D" and hasattr(m, "nf"):
        lin = nn.Linear(m.weight.shape[0], m.weight.shape[1], bias=m.bias is not None, device=m.weight.device,
                        dtype=m.weight.dtype)
        lin.weight.data = m.weight.data.t().contiguous()
        if m.bias is not None:
            lin.bias.data = m.bias.data
        return lin
    return m


def tp_manual_shard(model: nn.Module, tpinfo: TPInfo, process_group="tensor", sequence_parallel: bool = False,
                    defer_init: bool = False) -> nn.Module:
    size = D.parallel_group_size("tensor") or 1
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent._modules.items()):
            if child is None:
                continue
            full = f"{parent_name}.{child_name}" if parent_name else child_name
            done = False
            for cls, suffixes in tpinfo.Shard.items():
                for suf, kw in suffixes.items():
                    if full.endswith(suf) and not done:
                        kw = dict(kw)
                        if cls is not VocabParallelEmbedding:
                            kw.setdefault("sequence_parallel", sequence_parallel)
                            src = _as_linear(child)
                        else:
                            src = child
                        parent._modules[child_name] = cls(orig_module=src, process_group=process_group,
                                                          defer_init=defer_init, **kw)
                        done = True
            if done:
                continue
            for same, suffixes in tpinfo.Drop.items():
                if any(full.endswith(s) for s in suffixes):
                    parent._modules[child_name] = _RandomizedDropout(child, same)
    for name, m in model.named_modules():
        for suf, attrs in tpinfo.Shrink.items():
            if name.endswith(suf):
                for a in attrs:
                    v = getattr(m, a)
                    assert v % size == 0, f"{name}.{a}={v} is not divisible by the tensor-parallel size {size}"
                    setattr(m, a, v // size)
    return model


def tp_manual_shard_custom_fn(meta_model: nn.Module, tpinfo: TPInfo):
    """Deferred form for meta-initialised models: shards with ``defer_init`` (weights stay on meta
    until the sharded engine or pipeline stage materialises them)."""
    return tp_manual_shard(meta_model, tpinfo, defer_init=any(p.is_meta for p in meta_model.parameters()))


def vocab_parallel_logit_helper(embed, lm_output):
    import torch
    import torch.nn.functional as F

    from ..modules.distributed_modules.mappings import copy_to_group

    if isinstance(lm_output, tuple):
        lm_output = lm_output[0]
    if not isinstance(lm_output, torch.Tensor):
        raise ValueError(f"Expect lm_output as tensor or tuple but get {type(lm_output)}")
    return F.linear(copy_to_group(lm_output, D.parallel_group("tensor")), embed.weight)
