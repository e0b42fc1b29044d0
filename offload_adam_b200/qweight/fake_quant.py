"""Fake quantization: a dense tensor rounded to what a packed format can represent.

``fake_quantize(x, NVFP4QWeight)`` returns ``dequantize(quantize(x))`` in ``x``'s
dtype with a straight-through gradient, for experiments that keep dense weights and
only want the quantization error in the forward pass.  The packed formats of this
package train differently (the packed weight is the parameter, the optimizer owns an
fp32 master), so nothing in the optimizers depends on this helper; the reference has
no counterpart.  On CUDA tensors one kernel per format reads ``x`` and writes
``dequantize(quantize(x))`` directly (``csrc/quant.cu`` ``launch_fake_quant``; NVFP4 takes
a reduction for max|x| first): no packed payload is allocated and the Python quantizer is
not involved.  The result is bit-identical to running the format's quantize and
dequantize kernels one after the other.  CPU tensors go through the PyTorch restatements.
"""

from __future__ import annotations

import torch

from .. import _ext
from .base import QWeightBase

_KERNEL_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _fake_quantize_cuda(src, cls, kwargs):
    """One-pass kernel route; None when the kernels do not take this case."""
    fmt = cls.KERNEL_FORMAT
    if not fmt or src.dtype not in _KERNEL_DTYPES or src.dim() != 2:
        return None
    C = _ext.load(required=True)
    in_f = src.shape[1]
    group = {1: 16, 2: kwargs.get("blocksize", 64), 3: kwargs.get("group_size", 128), 4: 0}[fmt]
    scale_dtype = kwargs.get("scale_dtype", torch.bfloat16)
    if scale_dtype not in _KERNEL_DTYPES:
        return None
    if fmt == 1 and in_f % 16:
        return None
    if fmt == 2 and (group not in (16, 32, 64, 128, 256, 512) or in_f % group):
        return None
    if fmt == 3 and (group not in (32, 64, 128) or in_f % group or in_f % 16):
        return None
    x = src if src.is_contiguous() else src.contiguous()
    out = torch.empty_like(x)
    amax = None
    if fmt == 1:
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
        C.absmax(x, amax)
    ids = {torch.float32: C.QDT_F32, torch.bfloat16: C.QDT_BF16, torch.float16: C.QDT_F16}
    C.fake_quant(fmt, x, out, int(group), ids[scale_dtype], amax)
    return out


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cls, kwargs):
        if not cls.can_quantize(x, **kwargs):
            raise ValueError(f"{cls.__name__} cannot hold a tensor of shape {tuple(x.shape)}")
        src = x.detach()
        if src.is_cuda:
            out = _fake_quantize_cuda(src, cls, kwargs)
            if out is not None:
                return out
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
