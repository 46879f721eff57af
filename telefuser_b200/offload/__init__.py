from .async_offload import AsyncOffloadManager, attach_layer_hooks
from .sequential_offload import (OffloadUnit, enable_sequential_cpu_offload, move_tensors_to_device,
                                 move_tensors_to_pinned_cpu)  # fmt: skip

__all__ = ["AsyncOffloadManager", "attach_layer_hooks", "OffloadUnit", "enable_sequential_cpu_offload",
           "move_tensors_to_device", "move_tensors_to_pinned_cpu"]  # fmt: skip
