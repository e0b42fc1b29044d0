"""adam_step_stochastic_rounding under the reference's module path
(reference: src/offload_adam/kernels/stochastic_rounding.py)."""

from ..ops.adam_step import adam_step_stochastic_rounding

__all__ = ["adam_step_stochastic_rounding"]
