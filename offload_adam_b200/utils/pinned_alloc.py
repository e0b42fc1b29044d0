"""Pinned host memory with NUMA placement, backed by the C++ arena.

Public functions keep the reference module's names and meaning
(reference: src/offload_adam/pinned_alloc.py:113-277): ``zeros_pinned``,
``resolve_numa_target``, ``numa_node_free_bytes``, ``gpu_numa_node``.  The
difference is underneath: allocation goes through
``csrc/pinned_arena.cpp`` (raw ``mbind`` syscall, so binding works without
libnuma; parallel first touch; one registration per multi-GB segment), and
:class:`PinnedArena` lets an optimizer obtain all of its state tensors from a
few segments instead of one registration per tensor.
"""

from __future__ import annotations

import math
from typing import Iterable, Sequence

import torch

from .. import _ext


def _C():
    C = _ext.load(required=None)
    if C is None:
        raise RuntimeError("offload_adam_b200 native extension is not built")
    return C


def gpu_numa_node(device=None) -> int:
    """NUMA node the CUDA device hangs off (PCI bus id -> sysfs), or -1."""
    if not torch.cuda.is_available():
        return -1
    if device is None:
        device = torch.cuda.current_device()
    if isinstance(device, torch.device):
        device = device.index if device.index is not None else torch.cuda.current_device()
    return int(_C().gpu_numa_node(int(device)))


def numa_node_free_bytes(node: int):
    """``MemFree`` of the node in bytes, or None when it cannot be read."""
    v = int(_C().numa_node_free_bytes(int(node)))
    return None if v < 0 else v


def resolve_numa_target(numa_node, device=None):
    """``'auto'`` -> the GPU's node when known, an int -> itself, None -> None."""
    if numa_node == "auto":
        if torch.cuda.is_available():
            n = gpu_numa_node(device)
            if n >= 0:
                return n
        return None
    if isinstance(numa_node, bool):
        raise ValueError(f"numa_node must be 'auto', an int, or None (got {numa_node!r})")
    if isinstance(numa_node, int):
        return numa_node
    if numa_node is None:
        return None
    raise ValueError(f"numa_node must be 'auto', an int, or None (got {numa_node!r})")


class PinnedArena:
    """All tensors of ``specs`` carved out of a few pinned, NUMA-bound segments.

    ``specs`` is a sequence of ``(shape, dtype)``.  Tensors are zero-filled CPU
    tensors that keep the arena alive; memory is unregistered and unmapped when
    the last of them (and the arena object) is gone.
    """

    def __init__(self, specs: Sequence, numa_node="auto", device=None, register_cuda=None,
                 huge_pages=True, touch_threads=0, segment_bytes=0, alignment=4096):
        self.specs = [(torch.Size(s), d) for s, d in specs]
        sizes = [max(1, math.prod(s) * torch.empty(0, dtype=d).element_size()) for s, d in self.specs]
        target = resolve_numa_target(numa_node, device)
        if register_cuda is None:
            register_cuda = torch.cuda.is_available()
        if register_cuda:
            torch.cuda.init()  # registration needs a primary context
        self._arena = _C().PinnedArena(
            sizes, -1 if target is None else int(target), bool(register_cuda), bool(huge_pages),
            int(touch_threads), int(segment_bytes), int(alignment),
        )
        self.numa_target = target
        self.nbytes = sum(sizes)

    def tensor(self, i: int) -> torch.Tensor:
        shape, dtype = self.specs[i]
        return self._arena.tensor(i, list(shape), dtype)

    def tensors(self) -> Iterable[torch.Tensor]:
        return [self.tensor(i) for i in range(len(self.specs))]

    def stats(self) -> dict:
        return dict(self._arena.stats())


def zeros_pinned(shape, dtype, numa_node="auto"):
    """Zero-initialised pinned CPU tensor of exact size (one-tensor arena)."""
    arena = PinnedArena([(torch.Size(shape), dtype)], numa_node=numa_node)
    return arena.tensor(0)
