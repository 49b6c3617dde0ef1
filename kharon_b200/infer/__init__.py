from .engine import InferEngine, InferStats

__all__ = ["InferEngine", "InferStats"]
