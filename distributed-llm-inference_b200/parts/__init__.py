from . import attention, block, mlp, model, norm, rotary  # noqa: F401  (registers the parts)
from .base import BuildEnv, Part, ResidualStream, build_part, register_part, unregister_part
from .model import DecoderModel, declared_tensors

__all__ = ["BuildEnv", "DecoderModel", "Part", "ResidualStream", "build_part", "declared_tensors", "register_part", "unregister_part"]
