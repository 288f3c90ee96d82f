from . import gpt2  # noqa: F401
from .decoder import DecoderModel, ModelSpec, ScheduleEntry
from .loading import load_model

__all__ = ["DecoderModel", "ModelSpec", "ScheduleEntry", "load_model"]
