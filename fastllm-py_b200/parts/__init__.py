from . import attention, block, io, mlp, norm, rotary  # noqa: F401  (registers the built-in parts)
from .base import BuildContext, EngineLimits, Part, ResidualStream, Workspace
from .decoder import Decoder
from .plan import LayerRun, LayerSpec, ModelPlan, PartSpec
from .registry import build_part, part_class, register_part

__all__ = ["BuildContext", "EngineLimits", "Part", "ResidualStream", "Workspace", "Decoder", "LayerRun", "LayerSpec",
           "ModelPlan", "PartSpec", "build_part", "part_class", "register_part"]
