from . import (attention, block, delta, differential, gla, io, latent, mlp, moe, norm, normed_attention,  # noqa: F401
               recurrence, retention, rotary, side_by_side, sink_attention)    # (registers the built-in parts)
from .base import BuildContext, EngineLimits, Part, ResidualStream, Workspace
from .decoder import Decoder
from .plan import LayerRun, LayerSpec, ModelPlan, PartSpec
from .registry import build_part, part_class, register_part

__all__ = ["BuildContext", "EngineLimits", "Part", "ResidualStream", "Workspace", "Decoder", "LayerRun", "LayerSpec",
           "ModelPlan", "PartSpec", "build_part", "part_class", "register_part"]
