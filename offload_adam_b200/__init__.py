"""offload_adam_b200: host-offloaded Adam/AdamW for bf16 models on B200 (sm_100a).

Public classes (reference: src/offload_adam/__init__.py:1-6): ``Adam`` (on-GPU
baseline), ``OffloadAdam`` (single GPU, state in pinned host memory) and
``DistributedOffloadAdam`` (ZeRO-1 sharded state across ranks).
"""

from .adam import Adam
from .offload_adam import OffloadAdam
from .parallel.distributed_offload_adam import DistributedOffloadAdam

__version__ = "0.1.0"
__all__ = ["Adam", "OffloadAdam", "DistributedOffloadAdam"]
