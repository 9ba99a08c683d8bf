"""``PartitionAdam``: Adam / AdamW whose moment estimates live in pinned host memory, one block per parameter
group, and visit the GPU only for the group's update.

Per step, for each group: the group's state block (``exp_avg`` and ``exp_avg_sq`` of all its parameters,
back to back, so one copy moves both) is copied host→device on the upload stream, the update runs on the
compute stream over views of that block, and the block is copied device→host on the download stream. The
upload of group ``i+1`` is issued before the update of group ``i``, so with several groups the copies
overlap the arithmetic; device memory holds at most two blocks. Parameters must share one dtype inside a
group; sparse gradients are refused. On a CPU-only run the blocks are updated in place.

(Reference: atorch/optimizers/adam_offload.py:89-309, which drives apex ``FusedAdam`` kernels; here the
update is a few ``torch._foreach`` calls.)
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
from torch.optim import Optimizer


class PartitionAdam(Optimizer):
    def __init__(self, params, lr: float = 1e-3, bias_correction: bool = True, betas=(0.9, 0.999), eps: float = 1e-8,
                 adam_w_mode: bool = True, weight_decay: float = 0.0, amsgrad: bool = False):
        if amsgrad:
            raise RuntimeError("PartitionAdam does not support the AMSGrad variant")
        super().__init__(params, dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                                      weight_decay=weight_decay))
        self.adam_w_mode = adam_w_mode
        self._streams = None

    def _block(self, idx: int, group) -> Optional[dict]:
        st = self.state.setdefault(f"group{idx}", {})
        if "state_block" not in st:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                return None
            dt = ps[0].dtype
            for p in ps:
                if p.grad.is_sparse:
                    raise RuntimeError("PartitionAdam does not support sparse gradients")
                assert p.dtype == dt, f"parameters of one group must share a dtype ({p.dtype} != {dt})"
            numel = sum(p.numel() for p in ps)
            blk = torch.zeros(2 * numel, dtype=dt)
            if torch.cuda.is_available() and ps[0].is_cuda:
                blk = blk.pin_memory()
            st.update(state_block=blk, numel=numel, params=[id(p) for p in ps])
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        work = []
        for i, g in enumerate(self.param_groups):
            st = self._block(i, g)
            if st is not None:
                work.append((g, st))
        if not work:
            return loss
        on_gpu = any(p.is_cuda for g, _ in work for p in g["params"])
        if on_gpu and self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream())
        dev_blocks: List[Optional[torch.Tensor]] = [None] * len(work)

        def upload(k: int) -> None:
            g, st = work[k]
            dev = next(p.device for p in g["params"] if p.grad is not None)
            if dev.type != "cuda":
                dev_blocks[k] = st["state_block"]
                return
            up = self._streams[0]
            with torch.cuda.stream(up):
                dev_blocks[k] = st["state_block"].to(dev, non_blocking=True)
            st["_ready"] = up.record_event()

        upload(0)
        for k, (g, st) in enumerate(work):
            if k + 1 < len(work):
                upload(k + 1)
            blk, n = dev_blocks[k], st["numel"]
            if blk.is_cuda:
                torch.cuda.current_stream().wait_event(st.pop("_ready"))
            g["step"] = g.get("step", 0) + 1
            b1, b2 = g["betas"]
            ps = [p for p in g["params"] if p.grad is not None and id(p) in set(st["params"])]
            ms, vs, off = [], [], 0
            for p in ps:
                ms.append(blk[off: off + p.numel()].view_as(p))
                vs.append(blk[n + off: n + off + p.numel()].view_as(p))
                off += p.numel()
            grads = [p.grad for p in ps]
            if g["weight_decay"] != 0:
                if self.adam_w_mode:
                    torch._foreach_mul_(ps, 1 - g["lr"] * g["weight_decay"])
                else:
                    grads = torch._foreach_add(grads, ps, alpha=g["weight_decay"])
            torch._foreach_lerp_(ms, grads, 1 - b1)
            torch._foreach_mul_(vs, b2)
            torch._foreach_addcmul_(vs, grads, grads, 1 - b2)
            c1 = 1 - b1 ** g["step"] if g["bias_correction"] else 1.0
            c2 = 1 - b2 ** g["step"] if g["bias_correction"] else 1.0
            den = torch._foreach_sqrt(vs)
            torch._foreach_div_(den, math.sqrt(c2))
            torch._foreach_add_(den, g["eps"])
            torch._foreach_addcdiv_(ps, ms, den, -g["lr"] / c1)
            if blk.is_cuda:
                down = self._streams[1]
                down.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(down):
                    st["state_block"].copy_(blk, non_blocking=True)
                blk.record_stream(down)
            dev_blocks[k] = None
        if on_gpu:
            torch.cuda.current_stream().wait_stream(self._streams[1])
        return loss
