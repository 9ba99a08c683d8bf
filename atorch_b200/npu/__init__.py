"""Ascend NPU support of the original package (device patches, NPU flash attention with GLM masks, grouped
matmul binding, ``NpuAdamW``) has no role on B200 hardware. The names are kept as inert shims so that code
written against ``atorch.npu`` imports: availability probes return False and the helpers delegate to the
CUDA implementations of this framework."""
import torch

from ..modules.transformer.layers import FlashAttnModule
from ..ops.moe import grouped_gemm as _grouped_gemm


def is_torch_npu_available() -> bool:
    return False


def npu_fa_with_glm_mask(q, k, v, glm_mask=None, causal=True, dropout_p=0.0, softmax_scale=None, **_):
    m = FlashAttnModule(causal=causal, softmax_scale=softmax_scale, attention_dropout=dropout_p)
    return m(q, k, v, glm_mask=glm_mask)


def gmm(a, b, batch_sizes, trans_b: bool = False):
    return _grouped_gemm(a, b, batch_sizes, trans_b)


NpuAdamW = torch.optim.AdamW
