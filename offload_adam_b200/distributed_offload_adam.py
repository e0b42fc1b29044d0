"""``DistributedOffloadAdam`` under the reference's module path
(reference: src/offload_adam/distributed_offload_adam.py).  Implemented in
``offload_adam_b200.parallel.distributed_offload_adam``."""

from .parallel.distributed_offload_adam import DistributedOffloadAdam

__all__ = ["DistributedOffloadAdam"]
