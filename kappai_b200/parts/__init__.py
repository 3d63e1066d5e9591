from .base import (Part, WeightSpec, BuildEnv, register_part, unregister_part, make_part, part_kinds, CATEGORIES)

__all__ = ["Part", "WeightSpec", "BuildEnv", "register_part", "unregister_part", "make_part", "part_kinds",
           "CATEGORIES"]
