from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import BindContext, Part
from .registry import ROLES, build_part, register_part, registered_parts, unregister_part
from .spec import BlockSpec, ModelPlan, PartSpec, ScheduleEntry

__all__ = ["BindContext", "Part", "ROLES", "build_part", "register_part", "registered_parts", "unregister_part",
           "BlockSpec", "ModelPlan", "PartSpec", "ScheduleEntry"]
