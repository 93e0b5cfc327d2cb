"""B200-native CASTLE attention (causal attention with lookahead keys).

`Castle` is a drop-in for `lookahead_keys_attention.Castle`; `castle_attention`
replaces the reference's `castle_attention_triton` operator.
"""
from .castle import Cache, Castle, ModuleCache, cache_from_buffers
from .ops import castle_attention, castle_attention_packed, castle_decode_step, check_status, release_workspaces

__all__ = ["Castle", "Cache", "ModuleCache", "cache_from_buffers", "release_workspaces", "castle_attention", "castle_attention_packed", "castle_decode_step", "check_status"]
