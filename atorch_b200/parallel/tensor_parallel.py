"""Automatic tensor parallelism: plan which modules to shard and how, then rewrite the model.

Planning (rule based, Megatron pairing): inside every block that contains linears, a linear whose
output feeds another linear through element-wise ops is column-parallel and its consumer
row-parallel, so one all-reduce (or a reduce-scatter / all-gather pair with sequence parallelism)
closes each pair; embeddings with a large vocabulary become vocabulary-parallel. The pairing is
read off the module structure: attention blocks (q/k/v[/qkv] -> o), MLP blocks (up/gate -> down).
An optional cost check (``memory_bound``) keeps small layers replicated.

``apply_tensor_parallel(model, config)`` accepts either a ``TPInfo`` (``config["tpinfo"]``), an
explicit ``{"column": [...], "row": [...], "vocab": [...]}`` name map, or nothing (plan first).
(Reference: atorch/auto/opt_lib/tensor_parallel_optimization.py:23-168, shard_planners/
base_tp_planner.py:11-167, mip_tp_planner.py:34-502, compilers/tp_compiler/tp_compiler.py:24-159.)
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Tuple

import torch.nn as nn

from ..distributed import distributed as D
from ..tensor_parallel.manual_tp import TPInfo, tp_manual_shard

_COL_HINTS = ("q_proj", "k_proj", "v_proj", "qkv_proj", "query", "key", "value", "c_attn", "gate_proj", "up_proj",
              "gate_up_proj", "c_fc", "fc1", "w1", "wi", "dense_h_to_4h", "query_key_value", "intermediate.dense")
_ROW_HINTS = ("o_proj", "out_proj", "c_proj", "down_proj", "fc2", "w2", "wo", "dense_4h_to_h", "output.dense",
              "attention.dense")
_VOCAB_HINTS = ("embed_tokens", "wte", "word_embeddings", "tok_embeddings")


def _is_linear(m) -> bool:
    return isinstance(m, nn.Linear) or type(m).__name__ == "Conv1D"


def plan_tensor_parallel(model: nn.Module, config: Optional[dict] = None) -> dict:
    """Returns ``{"column": {name: kwargs}, "row": [names], "vocab": [names]}``.

    ``config["planner"] == "mip"`` with ``config["sample_inputs"]`` (a tuple of example tensors): the layout
    comes from the mixed-integer programme over the traced graph (``auto/mip_tp_planner.py``); a model that
    cannot be traced falls back to the name rules below."""
    config = config or {}
    tp = D.parallel_group_size("tensor") or config.get("tp_size", 1)
    if config.get("planner") == "mip" and config.get("sample_inputs") is not None and tp > 1:
        try:
            from ..auto.mip_tp_planner import MIPTensorParallelPlanner

            lay = MIPTensorParallelPlanner(tp, memory_budget_bytes=config.get("memory_budget_bytes")).plan(
                model, tuple(config["sample_inputs"]))
            mods = dict(model.named_modules())
            return {"column": {n: {} for n, v in lay.items() if v == "col" and _is_linear(mods[n])},
                    "row": [n for n, v in lay.items() if v == "row" and _is_linear(mods[n])],
                    "vocab": [n for n, v in lay.items() if v != "replicate" and isinstance(mods[n], nn.Embedding)],
                    "sequence_parallel": bool(config.get("sequence_parallel")), "planner": "mip"}
        except Exception as e:  # noqa: BLE001 - tracing is best effort
            import logging

            logging.getLogger("atorch.logger").warning("MIP tensor-parallel planner unavailable (%s); using rules", e)
    min_features = config.get("min_features", 2 * max(tp, 1))
    col: Dict[str, dict] = {}
    row: List[str] = []
    vocab: List[str] = []
    for name, m in model.named_modules():
        leaf = name.split(".")[-1] if name else name
        if _is_linear(m):
            w = m.weight
            out_f, in_f = (w.shape[1], w.shape[0]) if type(m).__name__ == "Conv1D" else (w.shape[0], w.shape[1])
            if any(name.endswith(h) or leaf == h for h in _COL_HINTS) and out_f % max(tp, 1) == 0 \
                    and out_f >= min_features:
                kw = {}
                if leaf in ("qkv_proj", "c_attn", "query_key_value") and out_f % (3 * max(tp, 1)) == 0:
                    kw["stride"] = 3
                if leaf == "gate_up_proj":
                    kw["stride"] = 2
                col[name] = kw
            elif any(name.endswith(h) or leaf == h for h in _ROW_HINTS) and in_f % max(tp, 1) == 0:
                row.append(name)
        elif isinstance(m, nn.Embedding) and leaf in _VOCAB_HINTS and m.num_embeddings % max(tp, 1) == 0:
            vocab.append(name)
    # a row-parallel layer is only valid if a column-parallel producer exists in the same parent block
    parents_with_col = {n.rsplit(".", 1)[0] if "." in n else "" for n in col}
    row = [r for r in row if (r.rsplit(".", 1)[0] if "." in r else "") in parents_with_col]
    return {"column": col, "row": row, "vocab": vocab, "sequence_parallel": bool(config.get("sequence_parallel"))}


def _shrink_attention_attrs(model: nn.Module, plan: dict, tp: int) -> None:
    """Head counts of attention blocks whose projections were split must be divided too."""
    parents = {n.rsplit(".", 1)[0] for n in plan["column"] if "." in n}
    for name, m in model.named_modules():
        if name in parents:
            for attr in ("num_heads", "num_attention_heads", "num_key_value_heads", "n_q", "n_kv", "embed_dim",
                         "split_size", "all_head_size"):
                v = getattr(m, attr, None)
                if isinstance(v, int) and v % tp == 0 and any(h in attr for h in ("head", "n_q", "n_kv", "embed",
                                                                                  "split", "all_head")):
                    setattr(m, attr, v // tp)


def apply_tensor_parallel(model: nn.Module, config: Optional[dict] = None) -> nn.Module:
    config = dict(config or {})
    tp = D.parallel_group_size("tensor") or 1
    info = config.get("tpinfo")
    if info is None:
        plan = config if ("column" in config or "row" in config) else plan_tensor_parallel(model, config)
        info = TPInfo()
        colmap = plan.get("column", {})
        info.shard_col(*([{k: v} for k, v in colmap.items()] if isinstance(colmap, dict) else colmap))
        info.shard_row(*plan.get("row", []))
        info.shard_vocab(*plan.get("vocab", []))
        if tp > 1 and config.get("shrink_attention_attrs", True):
            _shrink_attention_attrs(model, {"column": colmap if isinstance(colmap, dict) else {c: {} for c in colmap}},
                                    tp)
    tp_manual_shard(model, info, sequence_parallel=bool(config.get("sequence_parallel")),
                    defer_init=bool(config.get("defer_init", False)))
    for p_name, p in model.named_parameters():
        if any(p_name.startswith(n + ".") for n in list(info.Shard.values())[0]) or \
                any(p_name.startswith(n + ".") for d in info.Shard.values() for n in d):
            p._atb_tp_sharded = True
    return model


def tp_config_from_3d(config) -> Tuple[Optional[dict], Optional[dict]]:
    """Split a 3-D parallel description (object or dict with ``tpinfo`` and pipeline fields) into the
    configs of the tensor-parallel and pipeline wrappers."""
    if config is None:
        return None, None
    get = config.get if isinstance(config, dict) else (lambda k, d=None: getattr(config, k, d))
    tpinfo = get("tpinfo")
    tp_cfg = {"tpinfo": tpinfo} if tpinfo is not None else None
    pipe_cfg = None
    if (D.parallel_group_size("pipe") or D.parallel_group_size("pipeline") or 1) > 1:
        pipe_cfg = {k: get(k) for k in ("total_layer_num", "model_provider", "n_microbatches", "sche_name",
                                        "input_output_mapping") if get(k) is not None}
    return tp_cfg, pipe_cfg


def mark_sequence_parallel_replicated(model: nn.Module, classes=None) -> int:
    """With sequence-parallel activations, parameters that are replicated over the tensor group but see only
    this rank's part of the sequence (normalisation weights) end up with partial gradients. Flag them so that
    :func:`sync_sequence_parallel_grads` can sum those gradients over the tensor group."""
    n = 0
    for m in model.modules():
        is_norm = isinstance(m, classes) if classes else ("norm" in type(m).__name__.lower())
        if is_norm:
            for p in m.parameters(recurse=False):
                p._atb_sp_replicated = True
                n += 1
    return n


def sync_sequence_parallel_grads(model: nn.Module, group=None) -> None:
    """Sum the gradients of the flagged parameters over the tensor group (one all-reduce of one flat tensor).
    Works on a plain module (``.grad``) and on the sharded engine (slices of its gradient shard)."""
    import torch
    import torch.distributed as dist

    group = group if group is not None else D.parallel_group("tensor")
    if group is None or dist.get_world_size(group) == 1:
        return
    eng = getattr(model, "engine", None)
    pieces = []
    if eng is not None:
        g = eng.finalize_grads()
        for u in eng.units:
            for p, (s0, n, _) in zip(u.params, u.param_shard_slices()):
                if n and getattr(p, "_atb_sp_replicated", False):
                    pieces.append(g[u.shard_offset + s0: u.shard_offset + s0 + n])
    else:
        pieces = [p.grad.view(-1) for p in model.parameters()
                  if getattr(p, "_atb_sp_replicated", False) and p.grad is not None]
    if not pieces:
        return
    flat = torch.cat([t.float() for t in pieces])
    dist.all_reduce(flat, group=group)
    off = 0
    for t in pieces:
        t.copy_(flat[off: off + t.numel()])
        off += t.numel()
