"""Symmetric per-output-channel int8 weight (compressed-tensors W8A16).

Payload (reference: src/offload_adam/qweight/int8.py:1-9, :240-370):

* ``weight`` ``(out_f, in_f)`` int8;
* ``scales`` ``(out_f,)`` in the scale dtype, ``absmax(row) / 127``.

In memory the int8 values are stored unpacked; the checkpoint layout packs four
``value + 128`` bytes per int32 (``uint8b128``).  The outer dtype is the scale
dtype and dequantization multiplies in that dtype.
"""

from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from .. import _ext
from .base import QWeightBase

_CUDA_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
_BYTE_SHIFTS = (0, 8, 16, 24)


@torch.no_grad()
def quantize_int8_per_channel(tensor: Tensor, eps: float = 1e-12, scale_dtype=None) -> Tuple[Tensor, Tensor]:
    """PyTorch restatement.  Returns ``(weight int8, scales)``; the fp32 scale is rounded
    once, to ``scale_dtype`` (default: the input dtype)."""
    assert tensor.ndim == 2
    t = tensor.float()
    scale = t.abs().amax(dim=1) / 127.0
    q = torch.round(t * (1.0 / scale.clamp(min=eps)).unsqueeze(1)).clamp(-128, 127).to(torch.int8)
    return q, scale.to(scale_dtype or tensor.dtype)


def dequantize_int8_per_channel(weight: Tensor, scales: Tensor) -> Tensor:
    return weight.to(scales.dtype) * scales.unsqueeze(1)


def _quantize_int8_cuda(tensor: Tensor, scale_dtype, weight=None, scales=None):
    C = _ext.load(required=True)
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    if weight is None:
        weight = torch.empty(src.shape, dtype=torch.int8, device=src.device)
        scales = torch.empty((src.shape[0],), dtype=scale_dtype, device=src.device)
    C.int8_quantize(src, weight, scales)
    return weight, scales


def _dequant_int8_cuda(weight: Tensor, scales: Tensor) -> Tensor:
    C = _ext.load(required=True)
    out = torch.empty(weight.shape, dtype=scales.dtype, device=weight.device)
    C.int8_dequantize(weight.contiguous(), scales.contiguous(), out)
    return out


class Int8QWeight(QWeightBase):
    """Per-channel symmetric int8 weight."""

    PAYLOAD = ("weight", "scales")
    META = ()

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, weight, scales):
        return Tensor._make_wrapper_subclass(cls, tuple(weight.shape), dtype=scales.dtype, device=weight.device)

    @torch._dynamo.disable
    def __init__(self, weight, scales):
        assert weight.dtype is torch.int8 and weight.ndim == 2
        assert scales.ndim == 1 and scales.shape[0] == weight.shape[0]
        self.weight = weight
        self.scales = scales

    def _with_outer_dtype(self, payload, dtype):
        return type(self)(payload[0], payload[1].to(dtype))

    @classmethod
    def from_float(cls, tensor: Tensor, scale_dtype: torch.dtype = torch.bfloat16, **_):
        """``scale_dtype`` is both the stored scale dtype and the tensor's outer dtype."""
        weight, scales = quantize_int8_per_channel(tensor.detach())
        out = cls(weight, scales.to(scale_dtype))
        out.requires_grad_(tensor.requires_grad)
        return out

    @classmethod
    def can_quantize(cls, tensor: Tensor, **_) -> bool:
        # four values per int32 in the checkpoint layout
        return tensor.dim() == 2 and tensor.shape[1] % 4 == 0

    def dequantize(self, dtype=None) -> Tensor:
        same = dtype is None or dtype == self.scales.dtype
        if same and self.weight.is_cuda and self.scales.dtype in _CUDA_DTYPES:
            return _dequant_int8_cuda(self.weight, self.scales)
        work = torch.float32 if dtype == torch.float32 else self.scales.dtype
        out = self.weight.to(work) * self.scales.to(work).unsqueeze(1)
        return out if dtype is None else out.to(dtype)

    KERNEL_FORMAT = 4
    KERNEL_PAYLOAD = ("weight", "scales")

    def kernel_scale_dtype(self):
        return self.scales.dtype

    def _payload_rows(self, lo, hi):
        return [self.weight[lo:hi], self.scales[lo:hi]]

    def _quantize_into(self, src: Tensor, amax=None) -> None:
        if self.weight.is_cuda and src.is_cuda and src.dtype in _CUDA_DTYPES and self.scales.dtype in _CUDA_DTYPES:
            _quantize_int8_cuda(src, self.scales.dtype, self.weight, self.scales)
            return
        weight, scales = quantize_int8_per_channel(src.to(self.weight.device), scale_dtype=self.scales.dtype)
        self.weight.copy_(weight)
        self.scales.copy_(scales)

    # ---- checkpoint layout: compressed-tensors pack-quantized, uint8b128
    @classmethod
    def canonical_key_suffixes(cls):
        return ("weight_packed", "weight_scale", "weight_shape")

    def to_plain_state_dict(self) -> dict:
        out_f, in_f = self.weight.shape
        assert in_f % 4 == 0, f"in_features={in_f} must be a multiple of 4 to pack int8 into int32"
        u = ((self.weight.to(torch.int32) + 128) & 0xFF).reshape(out_f, in_f // 4, 4)
        packed = torch.zeros((out_f, in_f // 4), dtype=torch.int32, device=u.device)
        for i, s in enumerate(_BYTE_SHIFTS):
            packed |= u[..., i] << s
        return {
            "weight_packed": packed,
            "weight_scale": self.scales.unsqueeze(1),
            "weight_shape": torch.tensor([out_f, in_f], dtype=torch.int64, device=u.device),
        }

    @classmethod
    def from_plain_state_dict(cls, plain: dict, reference=None):
        packed = plain["weight_packed"]
        u = torch.stack([(packed >> s) & 0xFF for s in _BYTE_SHIFTS], dim=-1)
        weight = (u.reshape(packed.shape[0], packed.shape[1] * 4) - 128).to(torch.int8)
        return cls(weight, plain["weight_scale"].squeeze(-1))

    @classmethod
    def build_hf_quantization_config(cls, skip_patterns=(), **_) -> dict:
        return {
            "quant_method": "compressed-tensors",
            "format": "pack-quantized",
            "config_groups": {
                "group_0": {
                    "weights": {"num_bits": 8, "type": "int", "symmetric": True, "strategy": "channel"},
                    "targets": ["Linear"],
                },
            },
            "ignore": list(skip_patterns),
        }
