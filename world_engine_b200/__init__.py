"""world_engine_b200 -- frame-causal DiT attention over the KV ring-buffer
cache of Overworldai/world_engine, hand-written for NVIDIA B200 (sm_100a).

The package is the PyTorch-side mirror of the reference's interface for that
one path (cache object, attention module, patch installer); the work is done
by libwe_b200.so through a C ABI (include/we_b200.h).  There is no CPU or
Triton fallback: using an op without the built library, or on a non-CUDA
tensor, raises.
"""
from ._lib import ABI_VERSION, WeB200Error, load as load_library  # noqa: F401
from .kv_cache import B200LayerKVCache, B200StaticKVCache  # noqa: F401
from .attn import B200Attn, patch_Attn_b200  # noqa: F401
from .sessions import SessionSlab, shard_sessions  # noqa: F401
from . import ops  # noqa: F401

__all__ = [
    "ABI_VERSION", "WeB200Error", "load_library",
    "B200LayerKVCache", "B200StaticKVCache", "B200Attn", "patch_Attn_b200", "SessionSlab", "shard_sessions", "ops",
]
