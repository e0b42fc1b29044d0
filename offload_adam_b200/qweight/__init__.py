"""Weight-only quantized tensor subclasses for quantization-aware training."""

from .apply import QuantizeReport, quantize_linears, save_quantized_pretrained
from .base import QWeightBase
from .fake_quant import fake_quantize
from .int4 import Int4QWeight
from .int8 import Int8QWeight
from .nf4 import NF4QWeight
from .nvfp4 import NVFP4QWeight

__all__ = [
    "QWeightBase",
    "Int4QWeight",
    "Int8QWeight",
    "NF4QWeight",
    "NVFP4QWeight",
    "quantize_linears",
    "save_quantized_pretrained",
    "QuantizeReport",
    "fake_quantize",
]
