"""research-2_b200: a small, whole GPT-2 inference engine for one NVIDIA B200.

Import name: `research_2_b200`. Public entry points: `run`, `generate`, `Engine`
(engine/), `load_model` (models/), `write_model_folder` (weights/).
"""

__version__ = "0.1.0"

_LAZY = {
    "run": ("engine.api", "run"),
    "generate": ("engine.api", "generate"),
    "Engine": ("engine.engine", "Engine"),
    "EngineOptions": ("config.engine_options", "EngineOptions"),
    "load_model": ("models.loading", "load_model"),
    "write_model_folder": ("weights.model_folder", "write_model_folder"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{module}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
