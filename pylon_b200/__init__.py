"""pylon_b200: a single-GPU inference engine for Qwen3 dense on NVIDIA B200 (sm_100a)."""
__version__ = "0.1.0"
