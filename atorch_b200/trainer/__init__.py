from .atorch_args import AtorchArguments
from .atorch_trainer import AtorchTrainer
from .callbacks import TrainerCallback, TrainerControl, TrainerState
from .args import AtorchTrainingArgs
from .atorch_trainer_v2 import AtorchTrainerV2
from .engine import AtorchTrainEngine, NativeTrainEngine
