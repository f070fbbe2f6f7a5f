from .base import Part
from .plan import LayerCall, LayerPlan, ModelPlan, PartSpec, WeightDecl
from .registry import CATEGORIES, get_part, register_part, registered

__all__ = ["Part", "LayerCall", "LayerPlan", "ModelPlan", "PartSpec", "WeightDecl",
           "CATEGORIES", "get_part", "register_part", "registered"]
