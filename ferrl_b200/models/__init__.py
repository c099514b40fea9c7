"""Policy model families: dense Qwen3 / Llama-3.x, Qwen3.5/3.6 hybrid
(GatedDeltaNet + gated GQA, dense and MoE) and dense Gemma."""
from .dense import DenseCachedDecoder, DenseGradModel, DenseSpec  # noqa: F401
from .lora import BaseQuantization, DenseLoraTargets, FusedLoraLinear, LoraSpec  # noqa: F401
from .llama import llama_spec  # noqa: F401
from .qwen3 import qwen3_8b_spec, qwen3_spec  # noqa: F401
