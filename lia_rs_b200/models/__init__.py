from .decoder import DecoderModel, ModelSpec, ScheduleEntry
from . import minicpm5_llama, nafevik  # noqa: F401  (register the architectures)

__all__ = ["DecoderModel", "ModelSpec", "ScheduleEntry"]
