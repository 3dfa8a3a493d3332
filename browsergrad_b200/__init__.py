"""B200-native realizer bridge for browsergrad-jit's forward hot path.

``CudaBridge`` implements the reference's realizer-bridge protocol over ``libbgcuda.so``
(hand-written sm_100a kernels); ``realize_cuda`` is the realizer front; ``graph`` builds the
same lazy UOp graphs where browsergrad-jit is not installed.
"""
from .bridge import CudaBridge, create_cuda_realizer_bridge
from .errors import JitNotImplementedError, KernelError, RealizationError
from .front import (DeviceBufferTable, build_plan, materialize_resident, realize_cuda, realize_cuda_resident,
                    register_cuda_bridge, release_resident_leaves, unregister_cuda_bridge)

__all__ = [
    "CudaBridge", "create_cuda_realizer_bridge", "KernelError", "RealizationError", "JitNotImplementedError",
    "DeviceBufferTable", "build_plan", "realize_cuda", "realize_cuda_resident", "materialize_resident",
    "register_cuda_bridge", "unregister_cuda_bridge", "release_resident_leaves",
]
