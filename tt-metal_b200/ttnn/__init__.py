"""ttnn on NVIDIA B200: the block-float weight-matmul path of TT-NN behind the unchanged `ttnn` API.

from_torch(dtype=bfloat8_b | bfloat4_b, layout=TILE_LAYOUT) -> matmul / linear -> to_torch, plus all_gather for
tensor-parallel decode. The native extension must be built first (see build.py next to this package); importing
fails loudly when it is missing - there is no CPU implementation behind this API."""
try:
    from . import _ttnn
except ImportError as e:  # pragma: no cover
    raise ImportError("ttnn: the native extension _ttnn is not built; run `python tt-metal_b200/build.py` (or "
                      "`__graft_entry__.build()`) first") from e

from ._flags import TTNN_ENABLE_MODEL_CACHE, TTNN_ENABLE_FAST_RUNTIME_MODE, TTNN_ENABLE_LOGGING, get_bool_env_var  # noqa: F401
from .logger import logger
if TTNN_ENABLE_MODEL_CACHE:
    logger.info("ttnn: model cache was enabled")
if TTNN_ENABLE_FAST_RUNTIME_MODE:
    logger.info("ttnn: fast runtime mode was enabled")
if TTNN_ENABLE_LOGGING:
    logger.info("ttnn: enabled logging (every top-level operation synchronises the device)")

from .types import *  # noqa: F401,F403
from .types import (DataType, Layout, StorageType, Shape, Tensor, Device, CoreGrid, MemoryConfig, MathFidelity, DeviceGrid,
                    bfloat16, bfloat8_b, bfloat4_b, float32, uint16, uint32, TILE_LAYOUT, ROW_MAJOR_LAYOUT, TILE_SIZE,
                    DRAM_MEMORY_CONFIG, L1_MEMORY_CONFIG, WormholeComputeKernelConfig, GrayskullComputeKernelConfig,
                    DeviceComputeKernelConfig)
from .device import open_device, close_device, manage_device, synchronize_device
from .multi_device import (DeviceMesh, MultiDeviceTensor, open_device_mesh, close_device_mesh, create_device_mesh, get_num_devices,
                           get_device_ids, get_device_tensors, aggregate_as_tensor, TensorToMesh, MeshToTensor,
                           ShardTensorToMesh, ReplicateTensorToMesh, ConcatMeshToTensor, ListMeshToTensor)
from .operations.core import (from_torch, to_torch, to_layout, to_device, from_device, deallocate, reshape, dump_tensor,
                              load_tensor, as_tensor, is_tensor_storage_on_device)
from .operations.matmul import (matmul, linear, mul, MatmulProgramConfig, MatmulDefaultProgramConfig, MatmulMultiCoreReuseProgramConfig,
                                MatmulMultiCoreReuseMultiCastProgramConfig, MatmulMultiCoreReuseMultiCast1DProgramConfig)
from .operations.ccl import all_gather, linear_all_gather, linear_gated, linear_multi, wait_for_gather

from . import decorators
from .decorators import register_operation, register_pre_operation_hook, register_post_operation_hook

# every public operation goes through the per-operation wrapper (logging, hooks, NVTX) unless fast runtime mode is on
for _name in ("from_torch", "to_torch", "to_layout", "to_device", "from_device", "reshape", "as_tensor", "dump_tensor", "load_tensor",
              "matmul", "linear", "mul", "all_gather", "linear_all_gather", "linear_gated", "linear_multi"):
    globals()[_name] = register_operation("ttnn." + _name)(globals()[_name])
del _name

Tensor.__matmul__ = lambda self, other: matmul(self, other)
MultiDeviceTensor.__matmul__ = lambda self, other: matmul(self, other)
