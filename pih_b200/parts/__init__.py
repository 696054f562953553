"""Model parts: mixers, feed-forwards, norms, position encodings, blocks."""
from .registry import (PagedKVNeed, PagedStateNeed, PagedVectorNeed, Runtime, StateNeed, TensorInfo, part_class, register_block,
                       register_ffn, register_mixer, register_norm, register_position, unregister)
from . import (norm, rope, attention, swiglu, block, gated_delta, rglru, latent_attention, moe, retention,  # noqa: F401
               diff_attention, biased_mlp, scored_moe, window_attention, plain_mlp)                 # (registers the built-in kinds)

__all__ = ["PagedKVNeed", "PagedStateNeed", "PagedVectorNeed", "Runtime", "StateNeed", "TensorInfo", "part_class", "register_block",
           "register_ffn", "register_mixer", "register_norm", "register_position", "unregister"]
