"""Pinned, NUMA-aware host allocation under the reference's module path
(reference: src/offload_adam/pinned_alloc.py).  Implemented in
``offload_adam_b200.utils.pinned_alloc`` over the C++ arena."""

from .utils.pinned_alloc import *  # noqa: F401,F403
from .utils.pinned_alloc import (PinnedArena, gpu_numa_node, numa_node_free_bytes, resolve_numa_target,
                                 zeros_pinned)

__all__ = ["PinnedArena", "zeros_pinned", "resolve_numa_target", "numa_node_free_bytes", "gpu_numa_node"]
