"""Functional entry points of the fused Adam step, one per precision mode.

Import path kept for users of the reference package, which exposes its step
functions as ``offload_adam.kernels.adam_step_<mode>``
(reference: src/offload_adam/kernels/__init__.py:1-15).  The implementations live in
``offload_adam_b200.ops.adam_step`` (CUDA kernels for device tensors, the PyTorch
restatement for CPU tensors).
"""

from ..ops.adam_step import (adam_step_fp31_master, adam_step_fp32_master,
                             adam_step_fp32_master_custom_rounding, adam_step_stochastic_rounding)

__all__ = [
    "adam_step_stochastic_rounding",
    "adam_step_fp32_master",
    "adam_step_fp31_master",
    "adam_step_fp32_master_custom_rounding",
]
