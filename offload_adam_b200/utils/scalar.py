"""Read a device scalar on the host without going through a DMA copy engine.

While the optimizer's state write-backs are draining, a ``tensor.item()`` (a 4-byte
D2H ``cudaMemcpy``) waits in the copy engine's queue behind gigabytes of bulk
copies.  ``read_scalar`` has a one-thread kernel store the value into mapped pinned
host memory instead and waits for that kernel only.
"""

from __future__ import annotations

import torch

from .. import _ext

_bufs = {}


def read_scalar(t: torch.Tensor) -> float:
    """Value of a one-element CUDA tensor as a Python float (synchronises with the
    producing stream, not with outstanding bulk copies).  CPU tensors: ``t.item()``."""
    if not t.is_cuda:
        return float(t.item())
    C = _ext.load(required=True)
    dev = t.device.index or 0
    if dev not in _bufs:
        _bufs[dev] = torch.zeros(8, dtype=torch.int32).pin_memory()
    host = _bufs[dev]
    src = t.detach().reshape(1).float().contiguous().view(torch.int32)
    C.mirror_words(src, host)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(t.device))
    ev.synchronize()
    return float(host[:1].view(torch.float32).item())
