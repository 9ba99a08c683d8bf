from .ppo_utils import compute_rewards, gae, logprobs_of_labels, ppo_loss, whiten
from .trainer import AtorchRLConfig, ModelEngine, ModelSpec, PPOConfig, PPOTrainer, ReplayBuffer
