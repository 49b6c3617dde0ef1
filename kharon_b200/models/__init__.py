from .layout import Config, ParamStore, n_params, matmul_params
from .gpt import GPT

__all__ = ["Config", "ParamStore", "GPT", "n_params", "matmul_params"]
