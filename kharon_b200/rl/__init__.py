from .grpo import GRPOTrainer, AddTask, ReverseTask, advantages, coefficients

__all__ = ["GRPOTrainer", "AddTask", "ReverseTask", "advantages", "coefficients"]
