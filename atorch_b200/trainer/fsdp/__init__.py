from . import fsdp_ckpt_saver
from .fsdp_ckpt_saver import ExtraState, FsdpShardCkptAsyncSaver, FsdpShardDcpCkptLoader

fsdp_shard_async_saver = fsdp_ckpt_saver
fsdp_shard_dcp_loader = fsdp_ckpt_saver
