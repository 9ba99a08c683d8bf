from .cross_entropy import VocabParallelCrossEntropyLoss, vocab_parallel_cross_entropy
from .layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
from .mappings import (all_gather_from_group, collect_and_reshard, copy_to_group, gather_from_group,
                       reduce_from_group, reduce_scatter_to_group, scatter_to_group,
                       split_first_dim_gather_last_dim, split_last_dim_gather_first_dim)
from .transformer import (BlockSpec, ParallelMLP, ParallelSelfAttention, ParallelTransformerLayer,
                          spec_from_bert_layer, spec_from_gpt2_block, spec_from_llama_layer, tp_checkpoint)
