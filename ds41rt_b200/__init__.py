"""ds41rt_b200: a B200-native (sm_100a) inference engine for DeepSeek-V4.1-Flash-shaped models."""
from .config import ModelConfig  # noqa: F401

__version__ = "0.1.0"
