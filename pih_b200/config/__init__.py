"""Typed configurations and the architecture registry."""
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (AttentionSpec, BiasedMLPSpec, BlockSpec, ComputedRopeSpec, DiffAttentionSpec, GatedDeltaSpec,
                    LatentAttentionSpec, ModelSpec, MoESpec, NormSpec, RetentionSpec, RGLRUSpec, RopeSpec, ScalarNormSpec,
                    ScheduleEntry, ScoredMoESpec, SwiGLUSpec, HyperSpec, ScaledRopeSpec, WindowAttentionSpec, BigramSpec,
                    PlainMLPSpec)
from .qwen3 import Qwen3Config
from .rigotar import RigotarConfig
from .tuganex import TuganexConfig
from .pegopel import PegopelConfig
from .sagelorn import SagelornConfig

__all__ = ["config_class_for", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures", "AttentionSpec", "BlockSpec", "ModelSpec", "NormSpec",
           "RopeSpec", "ScheduleEntry", "SwiGLUSpec", "Qwen3Config", "GatedDeltaSpec", "LatentAttentionSpec", "MoESpec",
           "RGLRUSpec", "ScalarNormSpec", "RigotarConfig", "BiasedMLPSpec", "ComputedRopeSpec", "DiffAttentionSpec",
           "RetentionSpec", "ScoredMoESpec", "TuganexConfig", "HyperSpec", "ScaledRopeSpec", "WindowAttentionSpec",
           "PegopelConfig", "BigramSpec", "PlainMLPSpec", "SagelornConfig"]
