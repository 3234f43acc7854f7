"""A GPT-2 inference engine for one NVIDIA B200, in the manner of mlx-lm."""

__version__ = "0.1.0"
