"""Symmetric group-wise int4 weight in GPTQ storage.

Payload (reference: src/offload_adam/qweight/int4.py:1-10, :304-437):

* ``qweight`` ``(in_f // 8, out_f)`` int32: eight values of one output column along
  ``in_f``, least-significant nibble first, each stored as ``v + 8``;
* ``scales``  ``(in_f // group_size, out_f)`` in the scale dtype, ``absmax / 8``.

Zero point is the constant 8 (``qzeros`` is synthesised only when saving).  The
outer dtype of the tensor is the scale dtype; dequantization multiplies in that
dtype.  Rounding is half-to-even after multiplying by the correctly rounded
reciprocal of the scale, then clamp to ``[-8, 7]``.
"""

from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from .. import _ext
from .base import QWeightBase

_SHIFTS = tuple(range(0, 32, 4))
_CUDA_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
_KERNEL_GROUPS = (32, 64, 128)


def pack_int4_gptq(int_data: Tensor) -> Tensor:
    """``(out_f, in_f)`` int8 in [-8, 7] -> ``(in_f // 8, out_f)`` int32 GPTQ words."""
    out_f, in_f = int_data.shape
    assert in_f % 8 == 0, f"in_features={in_f} must be a multiple of 8"
    nib = (int_data.to(torch.int32) + 8).reshape(out_f, in_f // 8, 8)
    word = torch.zeros((out_f, in_f // 8), dtype=torch.int32, device=int_data.device)
    for i, s in enumerate(_SHIFTS):
        word |= nib[..., i] << s
    return word.T.contiguous()


def unpack_int4_gptq(packed: Tensor) -> Tensor:
    """Inverse of :func:`pack_int4_gptq`: ``(out_f, in_f)`` int8 in [-8, 7]."""
    rows = packed.T.contiguous()
    nib = torch.stack([(rows >> s) & 0xF for s in _SHIFTS], dim=-1)
    return (nib - 8).to(torch.int8).reshape(rows.shape[0], rows.shape[1] * 8)


@torch.no_grad()
def quantize_int4_groupwise(tensor: Tensor, group_size: int = 128, eps: float = 1e-12,
                            scale_dtype=None) -> Tuple[Tensor, Tensor]:
    """PyTorch restatement.  Returns ``(qweight, scales)``; the fp32 scale is rounded once,
    to ``scale_dtype`` (default: the input dtype)."""
    out_f, in_f = tensor.shape
    assert in_f % group_size == 0, f"in_features={in_f} not divisible by group_size={group_size}"
    assert in_f % 8 == 0, f"in_features={in_f} must be a multiple of 8"
    g = tensor.float().reshape(out_f, in_f // group_size, group_size)
    scale = g.abs().amax(dim=-1) / 8
    q = torch.round(g * (1.0 / scale.clamp(min=eps)).unsqueeze(-1)).clamp(-8, 7).to(torch.int8)
    return pack_int4_gptq(q.reshape(out_f, in_f)), scale.T.contiguous().to(scale_dtype or tensor.dtype)


def _kernel_ok(in_f: int, group: int, *tensors) -> bool:
    return all(t.is_cuda for t in tensors) and in_f % 128 == 0 and group in _KERNEL_GROUPS


def _quantize_pack_int4_cuda(tensor: Tensor, group_size: int, scale_dtype, qweight=None, scales=None):
    C = _ext.load(required=True)
    out_f, in_f = tensor.shape
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    if qweight is None:
        qweight = torch.empty((in_f // 8, out_f), dtype=torch.int32, device=src.device)
        scales = torch.empty((in_f // group_size, out_f), dtype=scale_dtype, device=src.device)
    C.int4_quantize(src, group_size, qweight, scales)
    return qweight, scales


def _dequant_int4_cuda(qweight: Tensor, scales: Tensor, group_size: int) -> Tensor:
    C = _ext.load(required=True)
    out = torch.empty((qweight.shape[1], qweight.shape[0] * 8), dtype=scales.dtype, device=qweight.device)
    C.int4_dequantize(qweight.contiguous(), scales.contiguous(), group_size, out)
    return out


class Int4QWeight(QWeightBase):
    """Group-wise symmetric int4 weight, raw GPTQ storage."""

    PAYLOAD = ("qweight", "scales")
    META = ("group_size",)

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, qweight, scales, group_size):
        return Tensor._make_wrapper_subclass(
            cls, (qweight.shape[1], qweight.shape[0] * 8), dtype=scales.dtype, device=qweight.device)

    @torch._dynamo.disable
    def __init__(self, qweight, scales, group_size):
        assert qweight.dtype is torch.int32 and qweight.ndim == 2 and scales.ndim == 2
        self.qweight = qweight
        self.scales = scales
        self.group_size = group_size

    def _with_outer_dtype(self, payload, dtype):
        return type(self)(payload[0], payload[1].to(dtype), self.group_size)

    @classmethod
    def from_float(cls, tensor: Tensor, group_size: int = 128, scale_dtype: torch.dtype = torch.bfloat16):
        """``scale_dtype`` is both the stored scale dtype and the tensor's outer dtype."""
        qweight, scales = quantize_int4_groupwise(tensor.detach(), group_size)
        out = cls(qweight, scales.to(scale_dtype), group_size)
        out.requires_grad_(tensor.requires_grad)
        return out

    @classmethod
    def can_quantize(cls, tensor: Tensor, group_size: int = 128, **_) -> bool:
        return tensor.dim() == 2 and tensor.shape[1] % group_size == 0 and tensor.shape[1] % 8 == 0

    def dequantize(self, dtype=None) -> Tensor:
        same = dtype is None or dtype == self.scales.dtype
        if same and self.scales.dtype in _CUDA_DTYPES and _kernel_ok(self.shape[1], self.group_size, self.qweight):
            return _dequant_int4_cuda(self.qweight, self.scales, self.group_size)
        # multiply in the scale dtype, except for an explicit fp32 request
        work = torch.float32 if dtype == torch.float32 else self.scales.dtype
        vals = unpack_int4_gptq(self.qweight).reshape(self.shape[0], -1, self.group_size).to(work)
        out = (vals * self.scales.T.to(work).unsqueeze(-1)).reshape(self.shape)
        return out if dtype is None else out.to(dtype)

    KERNEL_FORMAT = 3
    KERNEL_PAYLOAD = ("qweight", "scales")

    def kernel_group(self):
        return self.group_size

    def kernel_scale_dtype(self):
        return self.scales.dtype

    def _payload_rows(self, lo, hi):
        # GPTQ stores (in, out): output rows are columns of both tensors
        return [self.qweight[:, lo:hi], self.scales[:, lo:hi]]

    def _quantize_into(self, src: Tensor, amax=None) -> None:
        if src.dtype in _CUDA_DTYPES and self.scales.dtype in _CUDA_DTYPES and \
                _kernel_ok(self.shape[1], self.group_size, self.qweight, src):
            _quantize_pack_int4_cuda(src, self.group_size, self.scales.dtype, self.qweight, self.scales)
            return
        qweight, scales = quantize_int4_groupwise(src.to(self.qweight.device), self.group_size,
                                                  scale_dtype=self.scales.dtype)
        self.qweight.copy_(qweight)
        self.scales.copy_(scales)

    # ---- checkpoint layout: GPTQ (g_idx omitted: no activation reordering)
    @classmethod
    def canonical_key_suffixes(cls):
        return ("qweight", "scales", "qzeros")

    def to_plain_state_dict(self) -> dict:
        n_groups, out_f = self.scales.shape
        assert out_f % 8 == 0, f"out_features={out_f} must be a multiple of 8 to serialize symmetric qzeros"
        # zero point 8 in every nibble = 0x88888888
        qzeros = torch.full((n_groups, out_f // 8), -0x77777778, dtype=torch.int32, device=self.qweight.device)
        return {"qweight": self.qweight, "scales": self.scales, "qzeros": qzeros}

    @classmethod
    def from_plain_state_dict(cls, plain: dict, reference=None):
        qweight, scales = plain["qweight"], plain["scales"]
        return cls(qweight, scales, qweight.shape[0] * 8 // scales.shape[0])

    @classmethod
    def build_hf_quantization_config(cls, skip_patterns=(), group_size: int = 128, **_) -> dict:
        return {
            "quant_method": "gptq",
            "bits": 4,
            "group_size": group_size,
            "desc_act": False,
            "sym": True,
            "modules_to_not_convert": list(skip_patterns),
        }
