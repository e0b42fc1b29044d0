"""NVFP4 weight (compressed-tensors W4A16 ``nvfp4-pack-quantized`` layout).

Payload (reference: src/offload_adam/qweight/nvfp4.py:1-15, :740-885):

* ``weight_packed``  ``(out_f, in_f // 2)`` uint8, two E2M1 codes per byte, even
  column in the low nibble;
* ``block_scale_fp8`` ``(out_f, in_f // 16)`` float8_e4m3fn, one scale per 16 values;
* ``global_scale``    ``()`` fp32, ``amax / (448 * 6)``; the value of an element is
  ``e2m1 * fp32(block_scale) * global_scale``.

``quantize_nvfp4_blockwise`` / ``dequantize_nvfp4_blockwise`` are the PyTorch
restatements (CPU path and test oracle); on CUDA the sm_100a kernels in
``csrc/quant.cu`` produce bit-identical results with the hardware E2M1 converts.
"""

from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from .. import _ext
from .base import QWeightBase

NVFP4_BLOCKSIZE = 16
FP4_E2M1_MAX = 6.0
FP8_E4M3_MAX = 448.0
_EPS = 1e-12

# value of each 4-bit code: bit 3 sign, bits 2..1 exponent (bias 1), bit 0 mantissa
FP4_E2M1_LUT = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
# decision boundaries between neighbouring magnitudes
_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)

_CUDA_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def pack_fp4(codes: Tensor) -> Tensor:
    """``(rows, cols)`` uint8 codes -> ``(rows, cols // 2)`` bytes, even column low."""
    assert codes.dtype is torch.uint8 and codes.shape[1] % 2 == 0
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)


def unpack_fp4(packed: Tensor) -> Tensor:
    assert packed.dtype is torch.uint8
    out = torch.empty((packed.shape[0], packed.shape[1] * 2), dtype=torch.uint8, device=packed.device)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = packed >> 4
    return out


def _quantize_fp4_e2m1_rne(x: Tensor) -> Tensor:
    """fp32 -> E2M1 code with round-to-nearest, ties to the even mantissa, saturating
    at 6, sign taken from the sign bit (so -0.0 keeps code 8): the behaviour of
    ``cvt.rn.satfinite.e2m1x2.f32``."""
    mag = x.abs()
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for i, b in enumerate(_E2M1_BOUNDS):
        # the lower neighbour of boundary i is code i; even codes keep ties
        code += ((mag > b) if i % 2 == 0 else (mag >= b)).to(torch.uint8)
    return code | (torch.signbit(x).to(torch.uint8) << 3)


def _scales(t: Tensor, eps: float, amax=None):
    """Shared head of the quantizer: tensor scale, per-block e4m3 scale and the
    reciprocal of the effective scale.  ``amax`` overrides max|t| (row shards of a
    larger weight pass the whole weight's)."""
    out_f, in_f = t.shape
    groups = in_f // NVFP4_BLOCKSIZE
    amax = (t.abs().amax() if amax is None else amax.to(t.device, torch.float32).reshape(())).clamp(min=eps)
    global_scale = amax / (FP8_E4M3_MAX * FP4_E2M1_MAX)
    inv_global = 1.0 / global_scale.clamp(min=eps)
    blocks = t.reshape(out_f, groups, NVFP4_BLOCKSIZE)
    bamax = blocks.abs().amax(dim=-1).clamp(min=eps)
    scale_fp8 = ((bamax / FP4_E2M1_MAX) * inv_global).to(torch.float8_e4m3fn)
    inv_eff = 1.0 / (scale_fp8.to(torch.float32) * global_scale).clamp(min=eps)
    return blocks, scale_fp8, global_scale, inv_eff


@torch.no_grad()
def quantize_nvfp4_blockwise(tensor: Tensor, eps: float = _EPS, amax=None) -> Tuple[Tensor, Tensor, Tensor]:
    """PyTorch restatement of the NVFP4 quantizer.  ``in_f % 16 == 0`` required.
    Returns ``(weight_packed, block_scale_fp8, global_scale)``."""
    assert tensor.ndim == 2 and tensor.shape[1] % NVFP4_BLOCKSIZE == 0
    out_f, in_f = tensor.shape
    blocks, scale_fp8, global_scale, inv_eff = _scales(tensor.float(), eps, amax)
    codes = _quantize_fp4_e2m1_rne(blocks * inv_eff.unsqueeze(-1)).reshape(out_f, in_f)
    return pack_fp4(codes), scale_fp8, global_scale


def dequantize_nvfp4_blockwise(packed, block_scale_fp8, global_scale, in_f, dtype=torch.float32):
    out_f = packed.shape[0]
    groups = in_f // NVFP4_BLOCKSIZE
    lut = torch.tensor(FP4_E2M1_LUT, dtype=torch.float32, device=packed.device)
    vals = lut[unpack_fp4(packed).long()].reshape(out_f, groups, NVFP4_BLOCKSIZE)
    eff = (block_scale_fp8.to(torch.float32) * global_scale).reshape(out_f, groups, 1)
    return (vals * eff).reshape(out_f, in_f).to(dtype)


def _supports_native_fp4() -> bool:
    """True when the CUDA kernels (hardware E2M1 converts, sm_100a) can run."""
    if not torch.cuda.is_available():
        return False
    try:
        return torch.cuda.get_device_capability()[0] >= 10
    except Exception:
        return False


def _quantize_nvfp4_cuda(tensor: Tensor, packed=None, scale=None, gscale=None, amax=None):
    """Kernel path: amax pre-pass (skipped when ``amax`` is supplied, e.g. by the
    fused optimizer step) + one quantize pass writing straight into the payload."""
    C = _ext.load(required=True)
    out_f, in_f = tensor.shape
    src = tensor if tensor.is_contiguous() else tensor.contiguous()
    dev = src.device
    if packed is None:
        packed = torch.empty((out_f, in_f // 2), dtype=torch.uint8, device=dev)
        scale = torch.empty((out_f, in_f // NVFP4_BLOCKSIZE), dtype=torch.float8_e4m3fn, device=dev)
        gscale = torch.empty((), dtype=torch.float32, device=dev)
    if amax is None:
        amax = torch.zeros(1, dtype=torch.float32, device=dev)
        C.absmax(src, amax)
    C.nvfp4_quantize(src, amax, packed, scale, gscale)
    return packed, scale, gscale


def _dequant_nvfp4_cuda(packed, block_scale_fp8, global_scale, in_f, out_dtype):
    C = _ext.load(required=True)
    out = torch.empty((packed.shape[0], in_f), dtype=out_dtype, device=packed.device)
    C.nvfp4_dequantize(packed.contiguous(), block_scale_fp8.contiguous(), global_scale, out)
    return out


class NVFP4QWeight(QWeightBase):
    """NVFP4 blockwise weight; looks like a dense ``(out_f, in_f)`` tensor of ``outer_dtype``."""

    PAYLOAD = ("weight_packed", "block_scale_fp8", "global_scale")
    META = ("in_f", "outer_dtype")

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, weight_packed, block_scale_fp8, global_scale, in_f, outer_dtype):
        return Tensor._make_wrapper_subclass(
            cls, (weight_packed.shape[0], in_f), dtype=outer_dtype, device=weight_packed.device)

    @torch._dynamo.disable
    def __init__(self, weight_packed, block_scale_fp8, global_scale, in_f, outer_dtype):
        assert weight_packed.dtype is torch.uint8 and weight_packed.ndim == 2
        assert block_scale_fp8.dtype is torch.float8_e4m3fn and block_scale_fp8.ndim == 2
        assert global_scale.dtype is torch.float32
        self.weight_packed = weight_packed
        self.block_scale_fp8 = block_scale_fp8
        self.global_scale = global_scale
        self.in_f = in_f
        self.outer_dtype = outer_dtype

    def _with_outer_dtype(self, payload, dtype):
        return self._rebuild(payload, outer_dtype=dtype)

    @classmethod
    def from_float(cls, tensor: Tensor, **_):
        packed, scale, gs = quantize_nvfp4_blockwise(tensor.detach())
        out = cls(packed, scale, gs, tensor.shape[1], tensor.dtype)
        out.requires_grad_(tensor.requires_grad)
        return out

    @classmethod
    def can_quantize(cls, tensor: Tensor, **_) -> bool:
        return tensor.dim() == 2 and tensor.shape[1] % NVFP4_BLOCKSIZE == 0

    def dequantize(self, dtype=None) -> Tensor:
        dtype = dtype or self.outer_dtype
        if self.weight_packed.is_cuda and dtype in _CUDA_DTYPES and _supports_native_fp4():
            return _dequant_nvfp4_cuda(self.weight_packed, self.block_scale_fp8, self.global_scale,
                                       self.in_f, dtype)
        return dequantize_nvfp4_blockwise(self.weight_packed, self.block_scale_fp8, self.global_scale,
                                          self.in_f, dtype)

    USES_TENSOR_AMAX = True
    KERNEL_FORMAT = 1
    KERNEL_PAYLOAD = ("weight_packed", "block_scale_fp8")

    def kernel_group(self):
        return NVFP4_BLOCKSIZE

    def _payload_rows(self, lo, hi):
        return [self.weight_packed[lo:hi], self.block_scale_fp8[lo:hi], self.global_scale]

    def _quantize_into(self, src: Tensor, amax=None) -> None:
        if self.weight_packed.is_cuda and src.is_cuda and src.dtype in _CUDA_DTYPES and _supports_native_fp4():
            _quantize_nvfp4_cuda(src, self.weight_packed, self.block_scale_fp8, self.global_scale, amax=amax)
            return
        packed, scale, gs = quantize_nvfp4_blockwise(src.to(self.weight_packed.device), amax=amax)
        self.weight_packed.copy_(packed)
        self.block_scale_fp8.copy_(scale)
        self.global_scale.copy_(gs)

    # ---- checkpoint layout (compressed-tensors): the tensor scale is stored as
    # its reciprocal with shape (1,)
    @classmethod
    def canonical_key_suffixes(cls):
        return ("weight_packed", "weight_scale", "weight_global_scale")

    def to_plain_state_dict(self) -> dict:
        return {
            "weight_packed": self.weight_packed,
            "weight_scale": self.block_scale_fp8,
            "weight_global_scale": (1.0 / self.global_scale).reshape(1),
        }

    @classmethod
    def from_plain_state_dict(cls, plain: dict, reference=None):
        if reference is None:
            raise ValueError(
                "NVFP4QWeight.from_plain_state_dict requires a reference instance to resolve "
                "outer_dtype; the canonical state_dict carries no outer-dtype field."
            )
        packed = plain["weight_packed"]
        gs = (1.0 / plain["weight_global_scale"]).reshape(())
        return cls(packed, plain["weight_scale"], gs, packed.shape[1] * 2, reference.outer_dtype)

    @classmethod
    def build_hf_quantization_config(cls, skip_patterns=(), **_) -> dict:
        return {
            "quant_method": "compressed-tensors",
            "format": "nvfp4-pack-quantized",
            "config_groups": {
                "group_0": {
                    "weights": {
                        "num_bits": 4,
                        "type": "float",
                        "symmetric": True,
                        "strategy": "tensor_group",
                        "group_size": NVFP4_BLOCKSIZE,
                    },
                    "targets": ["Linear"],
                },
            },
            "ignore": list(skip_patterns),
        }
