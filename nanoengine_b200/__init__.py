"""nanoengine_b200: a Blackwell-native LLM inference engine.

Public surface (mirrors the reference package's ``from dlengine import Config, LLM, LLMComponent,
SamplingParams``, dlengine/__init__.py:1-17)."""
__version__ = "0.1.0"

_LAZY = {
    "Config": ("nanoengine_b200.config", "Config"),
    "LLM": ("nanoengine_b200.engine.llm_component", "LLM"),
    "LLMComponent": ("nanoengine_b200.engine.llm_component", "LLMComponent"),
    "SamplingParams": ("nanoengine_b200._native._core", "SamplingParams"),
    "RequestIn": ("nanoengine_b200._native._core", "RequestIn"),
    "RequestMigrate": ("nanoengine_b200._native._core", "RequestMigrate"),
    "ModelConfig": ("nanoengine_b200.models.config", "ModelConfig"),
}


def _ensure_native():
    import importlib.util
    if importlib.util.find_spec("nanoengine_b200._native._core") is None:
        from .build_native import build_all
        build_all()


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        if "_native" in mod:
            _ensure_native()
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)


__all__ = list(_LAZY)
