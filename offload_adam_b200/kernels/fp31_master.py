"""adam_step_fp31_master under the reference's module path
(reference: src/offload_adam/kernels/fp31_master.py)."""

from ..ops.adam_step import adam_step_fp31_master

__all__ = ["adam_step_fp31_master"]
