"""Fake quantization: a dense tensor rounded to what a packed format can represent.

``fake_quantize(x, NVFP4QWeight)`` returns ``dequantize(quantize(x))`` in ``x``'s
dtype with a straight-through gradient, for experiments that keep dense weights and
only want the quantization error in the forward pass.  The packed formats of this
package train differently (the packed weight is the parameter, the optimizer owns an
fp32 master), so nothing in the optimizers depends on this helper; the reference has
no counterpart.  On CUDA tensors the format's quantize and dequantize kernels run, on
CPU tensors their PyTorch restatements.
"""

from __future__ import annotations

import torch

from .base import QWeightBase


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cls, kwargs):
        if not cls.can_quantize(x, **kwargs):
            raise ValueError(f"{cls.__name__} cannot hold a tensor of shape {tuple(x.shape)}")
        src = x.detach()
        q = cls.from_float(torch.zeros_like(src), **kwargs)  # payload of the right shapes
        q.copy_(src.float() if src.is_cuda else src)         # kernel path on CUDA tensors
        return q.dequantize(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        return grad, None, None  # straight-through


def fake_quantize(x: torch.Tensor, cls: type, **kwargs) -> torch.Tensor:
    """``x`` rounded to the grid of format ``cls`` (a ``QWeightBase`` subclass); keyword
    arguments are the format's (``group_size`` for int4, ``blocksize`` for NF4)."""
    if not (isinstance(cls, type) and issubclass(cls, QWeightBase)):
        raise TypeError("cls must be a QWeightBase subclass")
    return _FakeQuantSTE.apply(x, cls, kwargs)
