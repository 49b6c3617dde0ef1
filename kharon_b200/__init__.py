"""B200-native GPT training, serving and RL framework (capabilities of UjaanRakshit/kharon)."""
__version__ = "0.1.0"
