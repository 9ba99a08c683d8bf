"""Hook used by ``ModelContext.create_dataloader``: returns a shared-memory dataloader when
``ENABLE_SHM_DATALOADER`` is set and a model-parallel group shares batches, else None."""
import os


def maybe_shm_dataloader(dataset, sampler, args):
    if os.environ.get("ENABLE_SHM_DATALOADER", "0") not in ("1", "true", "True"):
        return None
    from .shm_context import build_shm_dataloader

    return build_shm_dataloader(dataset, sampler, args)
