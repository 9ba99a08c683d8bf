"""Mixed-precision helpers with the call shapes of apex ``amp`` (``initialize`` / ``scale_loss`` / ...) and the
gradient scaler for pipeline-parallel training."""
from .amp import initialize, load_state_dict, master_params, scale_loss, state_dict  # noqa: F401
from .pipe_amp import PipeGradScaler  # noqa: F401
