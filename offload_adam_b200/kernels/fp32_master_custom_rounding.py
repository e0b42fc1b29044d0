"""adam_step_fp32_master_custom_rounding under the reference's module path
(reference: src/offload_adam/kernels/fp32_master_custom_rounding.py)."""

from ..ops.adam_step import adam_step_fp32_master_custom_rounding

__all__ = ["adam_step_fp32_master_custom_rounding"]
