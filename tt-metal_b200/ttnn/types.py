"""Types and constants of the ttnn surface (mirrors ttnn/ttnn/types.py of the reference)."""
import dataclasses
from enum import Enum

from . import _ttnn

DataType = _ttnn.DataType
uint16 = DataType.UINT16
uint32 = DataType.UINT32
float32 = DataType.FLOAT32
bfloat16 = DataType.BFLOAT16
bfloat8_b = DataType.BFLOAT8_B
bfloat4_b = DataType.BFLOAT4_B

BufferType = _ttnn.BufferType
TensorMemoryLayout = _ttnn.TensorMemoryLayout
MemoryConfig = _ttnn.MemoryConfig
MathFidelity = _ttnn.MathFidelity
# A GPU has one kind of device memory: both configurations mean "HBM". They are kept so call sites do not change.
DRAM_MEMORY_CONFIG = MemoryConfig(TensorMemoryLayout.INTERLEAVED, BufferType.DRAM)
L1_MEMORY_CONFIG = MemoryConfig(TensorMemoryLayout.INTERLEAVED, BufferType.L1)

Layout = _ttnn.Layout
ROW_MAJOR_LAYOUT = Layout.ROW_MAJOR
TILE_LAYOUT = Layout.TILE

StorageType = _ttnn.StorageType
DEVICE_STORAGE_TYPE = StorageType.DEVICE
MULTI_DEVICE_STORAGE_TYPE = StorageType.MULTI_DEVICE

TILE_SIZE = 32

Shape = _ttnn.Shape
Tensor = _ttnn.Tensor
Device = _ttnn.Device
CoreGrid = _ttnn.CoreGrid

# Tensix-specific kernel knobs: accepted and ignored (fp32 accumulation at full operand precision always).
DeviceComputeKernelConfig = _ttnn.ComputeKernelConfig
WormholeComputeKernelConfig = _ttnn.ComputeKernelConfig
GrayskullComputeKernelConfig = _ttnn.ComputeKernelConfig


@dataclasses.dataclass
class CoreRange:
    start: CoreGrid
    end: CoreGrid


@dataclasses.dataclass
class DeviceGrid:
    y: int
    x: int

    @property
    def num_devices(self):
        return self.y * self.x

    def as_tuple(self):
        return (self.y, self.x)


class ShardStrategy(Enum):
    HEIGHT = 1
    WIDTH = 2
    BLOCK = 3


class ShardOrientation(Enum):
    ROW_MAJOR = 1
    COLUMN_MAJOR = 2
