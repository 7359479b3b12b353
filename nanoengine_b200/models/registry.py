"""Architecture name -> model class.  Parity: reference runtime/models/registry.py:78-100."""
from __future__ import annotations

from typing import Callable, Dict

_REGISTRY: Dict[str, Callable] = {}


def register(*names):
    def deco(fn):
        for n in names:
            _REGISTRY[n] = fn
        return fn
    return deco


def _deepseek():
    from .deepseek import DeepseekV3ForCausalLM
    return DeepseekV3ForCausalLM


def _qwen3_moe():
    from .qwen3 import Qwen3MoeForCausalLM
    return Qwen3MoeForCausalLM


def _qwen3_5():
    from .qwen3_5 import Qwen35ForCausalLM
    return Qwen35ForCausalLM


def _glm5_next():
    from .glm5_next import Glm5NextForConditionalGeneration
    return Glm5NextForConditionalGeneration


def _kimi_k3():
    from .kimi_k3 import KimiK3ForConditionalGeneration
    return KimiK3ForConditionalGeneration


def _deepseek_v4():
    from .deepseek_v4 import DeepseekV4ForCausalLM
    return DeepseekV4ForCausalLM


def _gemma4():
    from .gemma4 import Gemma4ForCausalLM
    return Gemma4ForCausalLM


_LAZY = {
    "Gemma4ForCausalLM": _gemma4, "Gemma4ForConditionalGeneration": _gemma4,
    "Glm5NextForConditionalGeneration": _glm5_next, "KimiK3ForConditionalGeneration": _kimi_k3,
    "DeepseekV4ForCausalLM": _deepseek_v4,
    "DeepseekV2ForCausalLM": _deepseek, "DeepseekV3ForCausalLM": _deepseek, "DeepseekV32ForCausalLM": _deepseek,
    "GlmMoeDsaForCausalLM": _deepseek, "KimiK2ForCausalLM": _deepseek,
    "Qwen3MoeForCausalLM": _qwen3_moe, "Qwen3ForCausalLM": _qwen3_moe,
    "Qwen3_5ForConditionalGeneration": _qwen3_5, "Qwen3_5MoeForConditionalGeneration": _qwen3_5,
}


def supported_architectures():
    return sorted(set(_LAZY) | set(_REGISTRY))


def get_model_class(architecture: str):
    if architecture in _REGISTRY:
        return _REGISTRY[architecture]
    if architecture in _LAZY:
        return _LAZY[architecture]()
    raise ValueError(f"unsupported architecture {architecture}; supported: {supported_architectures()}")
