"""ferrl_b200: a Blackwell-native GRPO + LoRA reinforcement-learning fine-tuning
framework (PyTorch framework layer, hand-written sm_100a CUDA kernels, NVLink
peer-memory collectives)."""
__version__ = "0.1.0"
