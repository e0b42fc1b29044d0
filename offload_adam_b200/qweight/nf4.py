"""NF4 weight (bitsandbytes storage, no double quantization).

Payload (reference: src/offload_adam/qweight/nf4.py:1-12, :380-537):

* ``weight_packed`` ``(out_f, in_f // 2)`` uint8, two codebook indices per byte, even
  column in the HIGH nibble (the opposite of NVFP4);
* ``absmax``        ``(out_f * in_f // blocksize,)`` fp32, row-major over blocks.

An element is ``NF4_LUT[index] * absmax[block]``.  Quantization normalises by
``1 / max(absmax, 1e-12)`` (reciprocal, then multiply) and picks the nearest of
the 16 entries, the lowest index winning exact ties.
"""

from __future__ import annotations

import json
from typing import Tuple

import torch
from torch import Tensor

from .. import _ext
from .base import QWeightBase

# bitsandbytes' NF4 codebook: quantiles of N(0, 1) rescaled to [-1, 1]
NF4_LUT = (
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
)
_DTYPE_NAMES = {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32"}
_NAME_DTYPES = {v: k for k, v in _DTYPE_NAMES.items()}
_CUDA_DTYPES = tuple(_DTYPE_NAMES)
_KERNEL_BLOCKSIZES = (16, 32, 64, 128, 256, 512)


def _lut(device, dtype=torch.float32) -> Tensor:
    return torch.tensor(NF4_LUT, dtype=dtype, device=device)


def pack_nf4(indices: Tensor) -> Tensor:
    """``(rows, cols)`` uint8 indices -> bytes with the even column in the high nibble."""
    assert indices.dtype is torch.uint8 and indices.shape[1] % 2 == 0
    return ((indices[:, 0::2] << 4) | indices[:, 1::2]).to(torch.uint8)


def unpack_nf4(packed: Tensor) -> Tensor:
    assert packed.dtype is torch.uint8
    out = torch.empty((packed.shape[0], packed.shape[1] * 2), dtype=torch.uint8, device=packed.device)
    out[:, 0::2] = packed >> 4
    out[:, 1::2] = packed & 0xF
    return out


@torch.no_grad()
def quantize_nf4_blockwise(tensor: Tensor, blocksize: int = 64) -> Tuple[Tensor, Tensor]:
    """PyTorch restatement.  Returns ``(weight_packed, absmax)``."""
    assert tensor.ndim == 2
    out_f, in_f = tensor.shape
    assert in_f % blocksize == 0 and in_f % 2 == 0
    blocks = tensor.float().reshape(out_f, in_f // blocksize, blocksize)
    absmax = blocks.abs().amax(dim=-1)
    x = blocks * (1.0 / absmax.clamp(min=1e-12)).unsqueeze(-1)
    # sequential scan with a strict '<': the first (lowest) index wins ties
    best = torch.zeros_like(x, dtype=torch.uint8)
    best_d = torch.full_like(x, float("inf"))
    for i, v in enumerate(NF4_LUT):
        d = (x - torch.tensor(v, dtype=torch.float32, device=x.device)).abs()
        closer = d < best_d
        best = torch.where(closer, torch.tensor(i, dtype=torch.uint8, device=x.device), best)
        best_d = torch.where(closer, d, best_d)
    return pack_nf4(best.reshape(out_f, in_f)), absmax.reshape(-1)


def dequantize_nf4_blockwise(packed, absmax, in_f, blocksize=64, dtype=torch.float32):
    out_f = packed.shape[0]
    vals = _lut(packed.device)[unpack_nf4(packed).long()].reshape(out_f, in_f // blocksize, blocksize)
    return (vals * absmax.float().reshape(out_f, -1, 1)).reshape(out_f, in_f).to(dtype)


def _kernel_ok(t: Tensor, blocksize: int, dtype) -> bool:
    return t.is_cuda and dtype in _CUDA_DTYPES and blocksize in _KERNEL_BLOCKSIZES


def _quantize_nf4_cuda(tensor: Tensor, blocksize: int, packed=None, absmax=None):
    C = _ext.load(required=True)
    out_f, in_f = tensor.shape
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    if packed is None:
        packed = torch.empty((out_f, in_f // 2), dtype=torch.uint8, device=src.device)
        absmax = torch.empty((out_f * (in_f // blocksize),), dtype=torch.float32, device=src.device)
    C.nf4_quantize(src, blocksize, packed, absmax)
    return packed, absmax


def _dequant_nf4_cuda(packed, absmax, in_f, blocksize, out_dtype):
    C = _ext.load(required=True)
    out = torch.empty((packed.shape[0], in_f), dtype=out_dtype, device=packed.device)
    C.nf4_dequantize(packed.contiguous(), absmax.contiguous(), blocksize, out)
    return out


class NF4QWeight(QWeightBase):
    """NF4 blockwise weight in bitsandbytes layout."""

    PAYLOAD = ("weight_packed", "absmax")
    META = ("in_f", "blocksize", "outer_dtype")

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, weight_packed, absmax, in_f, blocksize, outer_dtype):
        return Tensor._make_wrapper_subclass(
            cls, (weight_packed.shape[0], in_f), dtype=outer_dtype, device=weight_packed.device)

    @torch._dynamo.disable
    def __init__(self, weight_packed, absmax, in_f, blocksize, outer_dtype):
        assert weight_packed.dtype is torch.uint8 and weight_packed.ndim == 2
        assert absmax.dtype is torch.float32 and absmax.ndim == 1
        self.weight_packed = weight_packed
        self.absmax = absmax
        self.in_f = in_f
        self.blocksize = blocksize
        self.outer_dtype = outer_dtype

    def _with_outer_dtype(self, payload, dtype):
        return self._rebuild(payload, outer_dtype=dtype)

    @classmethod
    def from_float(cls, tensor: Tensor, blocksize: int = 64, **_):
        packed, absmax = quantize_nf4_blockwise(tensor.detach(), blocksize)
        out = cls(packed, absmax, tensor.shape[1], blocksize, tensor.dtype)
        out.requires_grad_(tensor.requires_grad)
        return out

    @classmethod
    def can_quantize(cls, tensor: Tensor, blocksize: int = 64, **_) -> bool:
        return tensor.dim() == 2 and tensor.shape[1] % blocksize == 0 and tensor.shape[1] % 2 == 0

    def dequantize(self, dtype=None) -> Tensor:
        dtype = dtype or self.outer_dtype
        if _kernel_ok(self.weight_packed, self.blocksize, dtype):
            return _dequant_nf4_cuda(self.weight_packed, self.absmax, self.in_f, self.blocksize, dtype)
        return dequantize_nf4_blockwise(self.weight_packed, self.absmax, self.in_f, self.blocksize, dtype)

    KERNEL_FORMAT = 2
    KERNEL_PAYLOAD = ("weight_packed", "absmax")

    def kernel_group(self):
        return self.blocksize

    def _payload_rows(self, lo, hi):
        per_row = self.in_f // self.blocksize
        return [self.weight_packed[lo:hi], self.absmax[lo * per_row:hi * per_row]]

    def _quantize_into(self, src: Tensor, amax=None) -> None:
        if src.is_cuda and _kernel_ok(self.weight_packed, self.blocksize, src.dtype):
            _quantize_nf4_cuda(src, self.blocksize, self.weight_packed, self.absmax)
            return
        packed, absmax = quantize_nf4_blockwise(src.to(self.weight_packed.device), self.blocksize)
        self.weight_packed.copy_(packed)
        self.absmax.copy_(absmax)

    # ---- checkpoint layout: what bitsandbytes' QuantState.from_dict consumes
    @classmethod
    def canonical_key_suffixes(cls):
        return ("weight", "weight.absmax", "weight.quant_map", "weight.quant_state.bitsandbytes__nf4")

    def to_plain_state_dict(self) -> dict:
        out_f, half = self.weight_packed.shape
        dev = self.weight_packed.device
        meta = {"quant_type": "nf4", "blocksize": self.blocksize,
                "dtype": _DTYPE_NAMES[self.outer_dtype], "shape": [out_f, half * 2]}
        blob = torch.tensor(list(json.dumps(meta).encode("utf-8")), dtype=torch.uint8, device=dev)
        return {
            "weight": self.weight_packed.reshape(-1, 1),  # bnb keeps a flat column vector
            "weight.absmax": self.absmax,
            "weight.quant_map": _lut(dev),
            "weight.quant_state.bitsandbytes__nf4": blob,
        }

    @classmethod
    def from_plain_state_dict(cls, plain: dict, reference=None):
        meta = json.loads(bytes(plain["weight.quant_state.bitsandbytes__nf4"].cpu().tolist()).decode("utf-8"))
        out_f, in_f = meta["shape"]
        return cls(plain["weight"].reshape(out_f, in_f // 2), plain["weight.absmax"], in_f,
                   meta["blocksize"], _NAME_DTYPES[meta["dtype"]])

    @classmethod
    def build_hf_quantization_config(cls, skip_patterns=(), compute_dtype: str = "bfloat16", **_) -> dict:
        return {
            "quant_method": "bitsandbytes",
            "load_in_4bit": True,
            "bnb_4bit_quant_type": "nf4",
            "bnb_4bit_use_double_quant": False,
            "bnb_4bit_compute_dtype": compute_dtype,
            "llm_int8_skip_modules": list(skip_patterns),
        }
