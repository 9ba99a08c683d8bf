"""Operator layer of atorch_b200: thin autograd wrappers over the sm_100a kernels in ``csrc/``.

Every op has a PyTorch reference implementation (``*_reference``) that is both the CPU path and the
oracle the GPU numerics tests compare against.
"""
from .gemm import gemm, gemm_reference, linear, linear_swiglu
from .norm import rms_norm, rms_norm_reference, layer_norm, layer_norm_reference
from .elementwise import (rope, rope_reference, rope_tables, swiglu, swiglu_reference, bias_gather_add,
                          bias_gather_add_reference)
from .cross_entropy import cross_entropy, cross_entropy_reference
from .optim import (adamw_step, adamw_reference, agd_step, agd_reference, sum_squares, outer_sgd_step,
                    outer_sgd_reference)
from .attention import attention, attention_reference, build_dense_mask

__all__ = [n for n in dir() if not n.startswith("_")]
