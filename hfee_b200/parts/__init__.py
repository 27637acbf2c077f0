from .base import CATEGORIES, Block, Mixer, Part, Runtime, build_part, part_class, register_part
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401  (register the built-in kinds)
from .model import DecoderModel, model_tensor_needs

__all__ = ["CATEGORIES", "Mixer", "Part", "Runtime", "build_part", "part_class", "register_part",
           "DecoderModel", "model_tensor_needs"]
