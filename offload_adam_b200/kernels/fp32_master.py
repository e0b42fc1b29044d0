"""adam_step_fp32_master under the reference's module path
(reference: src/offload_adam/kernels/fp32_master.py)."""

from ..ops.adam_step import adam_step_fp32_master

__all__ = ["adam_step_fp32_master"]
