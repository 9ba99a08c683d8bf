"""Which layers live on which pipeline stage.

``get_rank_stage_info`` returns, for one pipeline rank, ``[(stage_id, layer_num, start_layer_idx)]``:
stage ids follow the ``loop`` style (``rank + i * pp_size``) or the ``v`` style (pairs ``(r, S-1-r)``);
layers are split evenly with the remainder going to the first stages, unless
``manual_stage_partition`` fixes all stages (list) or some of them (dict stage -> layers).
(Reference: atorch/pipeline_parallel/pipe_partition.py:24-128.)
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch.nn as nn


def layers_per_stage(total_layer_num: int, total_stages: int,
                     manual: Union[None, Sequence[int], Dict[int, int]] = None) -> List[int]:
    fixed: Dict[int, int] = {}
    if manual is not None:
        if isinstance(manual, dict):
            fixed = dict(manual)
        else:
            assert len(manual) == total_stages and sum(manual) == total_layer_num
            fixed = dict(enumerate(manual))
    free = total_stages - len(fixed)
    rest = total_layer_num - sum(fixed.values())
    base, extra = (rest // free, rest % free) if free > 0 else (0, 0)
    out = []
    for s in range(total_stages):
        if s in fixed:
            out.append(fixed[s])
        else:
            out.append(base + (1 if extra > 0 else 0))
            extra -= 1 if extra > 0 else 0
    assert sum(out) == total_layer_num, (out, total_layer_num)
    return out


def stage_ids_of_rank(pp_rank: int, pp_size: int, virtual_pp_size: int, style: str = "loop") -> List[int]:
    total = pp_size * virtual_pp_size
    if style == "loop":
        return [pp_rank + i * pp_size for i in range(virtual_pp_size)]
    if style == "v":
        assert virtual_pp_size == 2, "v style uses two stages per rank"
        return [pp_rank, total - 1 - pp_rank]
    raise ValueError(f"style={style} not implemented")


def get_rank_stage_info(total_layer_num: int, pp_rank: int, pp_size: int, virtual_pp_size: int, style: str = "loop",
                        manual_stage_partition=None) -> List[Tuple[int, int, int]]:
    per = layers_per_stage(total_layer_num, pp_size * virtual_pp_size, manual_stage_partition)
    return [(s, per[s], sum(per[:s])) for s in stage_ids_of_rank(pp_rank, pp_size, virtual_pp_size, style)]


def partition_model_from_model_provider(model_provider, distributed_context, config):
    pp_size = distributed_context.parallel_group_size("pipe") or 1
    pp_rank = distributed_context.parallel_rank("pipe") or 0
    vpp = config.virtual_pp_size or 1
    total = pp_size * vpp
    style = "loop" if config.partition_method == "default" else config.partition_method
    modules, stage_ids = [], []
    for sid, n, start in get_rank_stage_info(config.total_layer_num, pp_rank, pp_size, vpp, style,
                                             config.manual_stage_partition):
        modules.append(model_provider(model_config=config.model_config, layer_num=n, pre_process=sid == 0,
                                      post_process=sid == total - 1, start_layer_idx=start))
        stage_ids.append(sid)
    return modules, stage_ids, None


class _SequentialStage(nn.Module):
    """One pipeline stage cut out of a model that is a chain ``pre -> layers[i] ... -> post``."""

    def __init__(self, pre, layers, post):
        super().__init__()
        self.pre, self.layers, self.post = nn.ModuleList(pre), nn.ModuleList(layers), nn.ModuleList(post)

    def forward(self, x, *rest):
        for m in list(self.pre) + list(self.layers) + list(self.post):
            x = m(x)
            if isinstance(x, (tuple, list)):
                x = x[0]
        return x


def partition_model_from_meta_model(meta_model, distributed_context, config):
    """Cut a model that is a chain — modules before a layer list, the ``nn.ModuleList`` of layers (the longest one
    found, ``config.total_layer_num`` layers), modules after it — into this rank's stages. The model may live on
    the meta device: only the parts this rank keeps are materialised (``to_empty`` + each module's
    ``reset_parameters``), so a model that does not fit one device can still be partitioned. Models whose data
    flow is not a chain need a ``model_provider`` instead. (The reference declares this entry point and leaves it
    unimplemented: atorch/pipeline_parallel/pipe_partition.py:127-129.)"""
    lists = [(n, m) for n, m in meta_model.named_modules() if isinstance(m, nn.ModuleList)]
    assert lists, "no nn.ModuleList of layers found; pass a model_provider"
    lname, layers = max(lists, key=lambda t: len(t[1]))
    assert config.total_layer_num in (None, len(layers)), (config.total_layer_num, len(layers))
    owner = meta_model.get_submodule(lname.rsplit(".", 1)[0]) if "." in lname else meta_model
    leaf = lname.rsplit(".", 1)[-1]
    pre, post, seen = [], [], False
    # modules of the outer chain: children of the owner around the layer list, then the owner's own siblings
    chain = []
    for n, c in meta_model.named_children():
        if c is owner and owner is not meta_model:
            chain += [(cn, cc) for cn, cc in owner.named_children()]
        else:
            chain.append((n, c))
    for n, c in chain:
        if n == leaf and c is layers:
            seen = True
        elif not seen:
            pre.append(c)
        else:
            post.append(c)
    pp_size = distributed_context.parallel_group_size("pipe") or 1
    pp_rank = distributed_context.parallel_rank("pipe") or 0
    vpp = config.virtual_pp_size or 1
    total = pp_size * vpp
    style = "loop" if config.partition_method == "default" else config.partition_method
    modules, stage_ids = [], []
    for sid, n, start in get_rank_stage_info(len(layers), pp_rank, pp_size, vpp, style, config.manual_stage_partition):
        stage = _SequentialStage(pre if sid == 0 else [], [layers[i] for i in range(start, start + n)],
                                 post if sid == total - 1 else [])
        if any(p.is_meta for p in stage.parameters()):
            stage.to_empty(device="cpu")
            for m in stage.modules():
                if hasattr(m, "reset_parameters"):
                    m.reset_parameters()
        modules.append(stage)
        stage_ids.append(sid)
    return modules, stage_ids, None
