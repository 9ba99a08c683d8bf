from .atorch_args import AtorchArguments
from .atorch_trainer import AtorchTrainer
from .callbacks import TrainerCallback, TrainerControl, TrainerState
